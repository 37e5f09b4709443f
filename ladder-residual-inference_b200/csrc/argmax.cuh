// Greedy token choice fused behind the LM-head projection, for an output projection whose rows are
// split over the tensor-parallel ranks.
//
// A candidate is packed into one 64-bit key, (order-preserving bits of the logit) << 32 | ~index,
// so that the numeric maximum of keys is "largest logit, lowest index on ties".  Every CTA of the
// producing kernel folds its candidates into one key per sequence in global memory: an atomic max
// that is only issued when the candidate beats the value it reads first (on random logits about
// ln(n) times per sequence), so the projection's CTAs retire as fast as without it (a per-CTA
// arrival ticket was measured to cost the 128 K-row projection 30 %: 32 K dependent atomics).  One
// warp launched behind the projection (programmatic dependent launch) owns the rank's result: with
// more than one rank it stores the keys as 16-byte lines {low, epoch, high, epoch} into every
// peer's inbox, polls its own inbox (bounded) for the peers' lines, and the maximum over ranks is
// the token every rank writes.  The keys are left at zero for the next call.
#pragma once

#include "common.cuh"

namespace lri {

constexpr int kArgmaxMaxRows = 64;  // sequences per call
constexpr size_t kArgmaxScratchBytes = kArgmaxMaxRows * 8;

struct ArgmaxArgs {
  unsigned long long* keys;  // [kArgmaxMaxRows], zero between calls
  int32_t* token_out;        // [rows]
  int64_t index_offset;      // vocabulary index of the first row of this rank's slice
  int rows;                  // sequences
  // exchange over peer memory (world == 1: none)
  uint8_t* inbox[8];          // every rank's inbox as mapped by this rank
  size_t region_off;          // offset of the head's line region inside an inbox
  int64_t slot_bytes;         // bytes of one (buffer, source rank) slot
  unsigned int* epoch_ptr;    // this rank's count of completed exchanges
  int* status_ptr;            // receives LRI_ERR_TIMEOUT when the bounded poll gives up
  unsigned long long timeout_ns;
  int world, rank;
};

__device__ __forceinline__ unsigned long long argmax_key(float v, int64_t index) {
  const unsigned int b = __float_as_uint(v);
  const unsigned int ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - static_cast<unsigned int>(index));
}

// Folds one candidate per sequence into the global keys.  Called by the thread that holds the
// CTA's best key of sequence m.
__device__ __forceinline__ void argmax_offer(const ArgmaxArgs& a, int m, unsigned long long key) {
  const unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(a.keys + m);
  if (key > cur) atomicMax(a.keys + m, key);
}

__device__ __forceinline__ unsigned long long argmax_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Run by one full warp after every producing CTA has completed (a kernel of its own behind the
// producer, all 32 lanes).
__device__ __forceinline__ void argmax_finish(const ArgmaxArgs& a) {
  const int lane = threadIdx.x & 31;
  unsigned int epoch = 0;
  int buf = 0;
  if (a.world > 1) {
    epoch = *reinterpret_cast<volatile unsigned int*>(a.epoch_ptr) + 1u;
    buf = epoch & 1u;
  }
  const unsigned long long t0 = argmax_global_ns();
  for (int m = 0; m < a.rows; ++m) {
    unsigned long long key = __ldcg(a.keys + m);  // L2: the other CTAs' atomics landed there
    if (a.world > 1) {
      // lane r talks to rank r: send this rank's key, then fetch rank r's
      unsigned long long theirs = 0ull;
      if (lane < a.world && lane != a.rank) {
        const size_t mine = a.region_off + (static_cast<size_t>(buf) * a.world + a.rank) * a.slot_bytes + static_cast<size_t>(m) * 16;
        const unsigned int lo = static_cast<unsigned int>(key), hi = static_cast<unsigned int>(key >> 32);
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(a.inbox[lane] + mine), "r"(lo), "r"(epoch),
                     "r"(hi), "r"(epoch)
                     : "memory");
        const uint8_t* src = a.inbox[a.rank] + a.region_off + (static_cast<size_t>(buf) * a.world + lane) * a.slot_bytes +
                             static_cast<size_t>(m) * 16;
        uint4 got;
        unsigned int spins = 0;
        while (true) {
          asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(got.x), "=r"(got.y), "=r"(got.z), "=r"(got.w)
                       : "l"(src)
                       : "memory");
          if (got.y == epoch && got.w == epoch) {
            theirs = (static_cast<unsigned long long>(got.z) << 32) | got.x;
            break;
          }
          if ((++spins & 63u) == 0u && argmax_global_ns() - t0 > a.timeout_ns) {
            atomicExch(a.status_ptr, LRI_ERR_TIMEOUT);
            break;
          }
        }
      }
      const unsigned long long cand = (lane == a.rank) ? key : theirs;
      unsigned long long best = cand;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
      }
      key = best;
    }
    if (lane == 0) {
      a.token_out[m] = static_cast<int32_t>(0xffffffffu - static_cast<unsigned int>(key));
      a.keys[m] = 0ull;  // ready for the next call
    }
  }
  __syncwarp();
  if (a.world > 1 && lane == 0) {
    __threadfence();
    *reinterpret_cast<volatile unsigned int*>(a.epoch_ptr) = epoch;
  }
}

}  // namespace lri
