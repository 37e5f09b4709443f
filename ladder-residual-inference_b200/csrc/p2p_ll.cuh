// Consumer side of the low-latency all-reduce, usable from inside other kernels.
//
// A producer (lri_comm_push) stores its partial as 16-byte lines {data, epoch, data, epoch}
// into slot `rank` of every peer's inbox.  A consumer does not need a reduce kernel: it polls
// the lines of its own inbox for the elements it is about to use and sums them in rank order
// together with its own partial.  The fused add + RMSNorm kernel does exactly that, so that an
// all-reduce costs the compute stream one small push kernel and no kernel on the consumer side.
// With `push` set the consumer is its own producer as well: every thread first stores the elements
// it is about to sum into the peers' inboxes and then polls for theirs, which makes the kernel a
// complete all-reduce + add + RMSNorm in one launch (no producer kernel, no stream hop).
#pragma once

#include "common.cuh"

namespace lri {

struct LlSource {
  const uint8_t* region;          // this rank's inbox: start of the channel's line region (both buffers)
  unsigned int* epoch_ptr;        // the channel's counter of consumed messages (this rank's memory)
  unsigned int* ticket_ptr;       // arrival counter of the consumer's CTAs (self-resetting)
  int* status_ptr;                // receives LRI_ERR_TIMEOUT when a bounded poll gives up
  const void* own;                // this rank's own partial (same layout as the message)
  uint8_t* peer_region[8];        // push != 0: the channel's line region in every rank's inbox, as mapped here
  int64_t slot_bytes;             // bytes of one (buffer, source rank) slot
  unsigned long long timeout_ns;
  int world, rank;
  int enabled;
  int push;                       // the consumer stores its own partial to the peers before it polls
};

struct GatherArgs {
  LlSource s1, s2;  // sources of the first and the second addend (enabled == 0: plain pointer or none)
};

__device__ __forceinline__ uint4 ll_ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ll_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Producer step of a consumer that is its own producer: 8 consecutive elements of this rank's
// partial, starting at flat element index `elem` (a multiple of 8), go as two lines into slot `rank`
// of every peer's region.
template <typename T>
__device__ __forceinline__ void ll_push8(const LlSource& s, unsigned int epoch, int64_t elem) {
  const uint4 own = *reinterpret_cast<const uint4*>(static_cast<const T*>(s.own) + elem);
  const size_t off = (static_cast<size_t>(epoch & 1u) * s.world + s.rank) * s.slot_bytes + (elem >> 2) * 16;
#pragma unroll
  for (int r = 0; r < 8; ++r) {  // constant indices: the argument block is not copied to local memory
    if (r >= s.world || r == s.rank) continue;
    uint8_t* dst = s.peer_region[r] + off;
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(own.x), "r"(epoch), "r"(own.y), "r"(epoch)
                 : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 16), "r"(own.z), "r"(epoch), "r"(own.w),
                 "r"(epoch)
                 : "memory");
  }
}

// Sum over ranks of 8 consecutive elements starting at flat element index `elem` (a multiple of
// 8) of the message with epoch `epoch`, in rank order, rounded once to T (what an all-reduce
// kernel would have written).  The wait is bounded; on expiry the status word is set and the
// values seen so far are used.
template <typename T>
__device__ __noinline__ void ll_gather8(const LlSource& s, unsigned int epoch, int64_t elem, float (&out)[8],
                                           unsigned long long t0) {
  const int buf = epoch & 1u;
  const uint8_t* base = s.region + static_cast<size_t>(buf) * s.world * s.slot_bytes + (elem >> 2) * 16;
  uint4 got[8][2];
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (r < s.world && r != s.rank) {
      got[r][0] = ll_ld_volatile16(base + static_cast<size_t>(r) * s.slot_bytes);
      got[r][1] = ll_ld_volatile16(base + static_cast<size_t>(r) * s.slot_bytes + 16);
    }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  bool gave_up = false;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if (r >= s.world) continue;
    uint4 payload;
    if (r == s.rank) {
      payload = *reinterpret_cast<const uint4*>(static_cast<const T*>(s.own) + elem);
    } else {
      unsigned int spins = 0;
      while (!gave_up && (got[r][0].y != epoch || got[r][0].w != epoch || got[r][1].y != epoch || got[r][1].w != epoch)) {
        if ((++spins & 63u) == 0u && ll_global_ns() - t0 > s.timeout_ns) {
          gave_up = true;
          atomicExch(s.status_ptr, LRI_ERR_TIMEOUT);
          break;
        }
        got[r][0] = ll_ld_volatile16(base + static_cast<size_t>(r) * s.slot_bytes);
        got[r][1] = ll_ld_volatile16(base + static_cast<size_t>(r) * s.slot_bytes + 16);
      }
      payload = make_uint4(got[r][0].x, got[r][0].z, got[r][1].x, got[r][1].z);
    }
    float f[8];
    unpack8<T>(payload, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += f[e];
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] = rnd<T>(acc[e]);
}

// After a consumer kernel has read everything it needs from message `epoch`: the last of its
// CTAs marks the message as consumed (thread 0 of every CTA calls this after a __syncthreads()).
__device__ __forceinline__ void ll_mark_consumed(const LlSource& s, unsigned int epoch) {
  __threadfence();
  const unsigned int t = atomicAdd(s.ticket_ptr, 1u);
  if (t == gridDim.x - 1) {
    *s.ticket_ptr = 0u;
    __threadfence();
    *reinterpret_cast<volatile unsigned int*>(s.epoch_ptr) = epoch;
  }
}

// defined in add_rmsnorm.cu: the fused add + RMSNorm whose addends may be gathered from peers
int launch_add_rmsnorm_gather(int dtype, const void* residual, const void* add1, const void* add2, float scale,
                              const void* weight, float eps, void* residual_out, void* normed_out, int64_t rows,
                              int dim, const GatherArgs& g, cudaStream_t st);

}  // namespace lri
