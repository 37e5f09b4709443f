// F8: one-shot all-reduce over NVLink peer memory for small decode messages.
//
// Every rank owns an inbox that all peers have mapped (CUDA IPC):
//   data  [2][world][max_bytes]      double buffered, one slot per source rank
//   flags [2][world][kMaxCtas]       epoch-valued arrival flags, one per (source rank, CTA index)
//   epoch, ticket, status            device-resident bookkeeping
// A call launches the same grid on every rank.  CTA c of rank r copies its range of the input
// into slot r of every rank's inbox (plain 16-byte stores over NVLink), publishes the epoch to
// flag [r][c] of every rank with a system-scope release, waits (bounded by a timer) until all
// `world` flags [.][c] of its own inbox carry the epoch, and sums the `world` slots of its range
// in fp32 in rank order, so every rank produces bit-identical results.  The epoch advances from
// device memory when the last CTA of the grid retires, which keeps replays of a captured CUDA
// graph correct.  Two buffers are enough: a rank cannot enter call n+2 before every peer has
// entered call n+1, i.e. finished reading call n.
#include <cstddef>
#include <cstring>

#include "linear.cuh"
#include "p2p_comm.cuh"
#include "p2p_ll.cuh"

namespace lri {
namespace {

struct ArParams {
  uint8_t* inbox[kMaxWorld];
  const void* in;
  void* out;
  int64_t nvec;  // 16-byte vectors in the message
  int64_t max_bytes;
  int rank, world;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_volatile16(void* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// One-shot all-reduce, low-latency protocol.  p.nvec counts 8-byte payload units here.  Thread i
// of the grid owns unit i: it sends the unit as one 16-byte line into slot `rank` of every
// peer's low-latency region, then polls the `world` lines of that unit in its own region until
// both halves carry the current epoch, and sums them in rank order (its own contribution comes
// from registers).  One NVLink crossing, no fence, no flag store.
template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_ll_kernel(const ArParams p) {
  uint8_t* mine = p.inbox[p.rank];
  Control* ctl = reinterpret_cast<Control*>(mine + control_offset(p.world, p.max_bytes));
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&ctl->epoch) + 1u;
  const int buf = epoch & 1u;
  const size_t region = ll_offset(p.world, p.max_bytes);
  const size_t my_slot = region + (static_cast<size_t>(buf) * p.world + p.rank) * kLlSlotBytes;
  const uint2* src = reinterpret_cast<const uint2*>(p.in);
  uint2* dst = reinterpret_cast<uint2*>(p.out);
  const unsigned long long t0 = global_ns();
  bool gave_up = false;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * kArThreads + threadIdx.x; u < p.nvec;
       u += static_cast<int64_t>(gridDim.x) * kArThreads) {
    const uint2 own = src[u];
    const uint4 line = make_uint4(own.x, epoch, own.y, epoch);
#pragma unroll 1
    for (int r = 0; r < p.world; ++r)
      if (r != p.rank) st_volatile16(p.inbox[r] + my_slot + u * 16, line);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* lines = mine + region + static_cast<size_t>(buf) * p.world * kLlSlotBytes + u * 16;
    // Look at all peers' lines at once (independent loads), then keep re-reading ALL lines that are still
    // late in one round of independent loads per iteration.  Re-polling peer after peer costs one L2 round
    // trip per late peer in sequence (measured: 4.4 us at 2 ranks, 7.7 us at 8, about 0.55 us per extra
    // peer); polled together the wait is the latest arrival plus one round trip.
    uint4 got[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < p.world && r != p.rank) got[r] = ld_volatile16(lines + static_cast<size_t>(r) * kLlSlotBytes);
    unsigned int spins = 0;
    while (!gave_up) {
      bool late = false;
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < p.world && r != p.rank && (got[r].y != epoch || got[r].w != epoch)) late = true;
      if (!late) break;
      if ((++spins & 63u) == 0u && global_ns() - t0 > p.timeout_ns) {
        gave_up = true;
        atomicExch(&ctl->status, LRI_ERR_TIMEOUT);
        break;
      }
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < p.world && r != p.rank && (got[r].y != epoch || got[r].w != epoch))
          got[r] = ld_volatile16(lines + static_cast<size_t>(r) * kLlSlotBytes);
    }
    // sum in rank order (this rank's own contribution comes from registers)
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
      if (r >= p.world) continue;
      const uint2 payload = (r == p.rank) ? own : make_uint2(got[r].x, got[r].z);
      float lo0, hi0, lo1, hi1;
      Num<T>::unpack2(payload.x, lo0, hi0);
      Num<T>::unpack2(payload.y, lo1, hi1);
      acc[0] += lo0, acc[1] += hi0, acc[2] += lo1, acc[3] += hi1;
    }
    dst[u] = make_uint2(pack2<T>(acc[0], acc[1]), pack2<T>(acc[2], acc[3]));
  }
  // the last CTA to retire advances the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(&ctl->ticket, 1u);
    if (t == gridDim.x - 1) {
      ctl->ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(&ctl->epoch) = epoch;
    }
  }
}

// Producer half of the split all-reduce as a kernel of its own (used when the projection that
// produced the partial cannot push from its epilogue): store this rank's partial as lines into
// slot `rank` of every peer's region of push channel `ch` (1-based).  The epoch is the channel's
// count of consumed messages plus one; the consumer advances the count.
__global__ void __launch_bounds__(kArThreads) ll_push_kernel(const ArParams p, int ch) {
  pdl_launch_dependents();
  pdl_wait();  // the partial comes from the preceding kernel
  uint8_t* mine = p.inbox[p.rank];
  Control* ctl = reinterpret_cast<Control*>(mine + control_offset(p.world, p.max_bytes));
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&ctl->chan_epoch[ch]) + 1u;
  const int buf = epoch & 1u;
  const size_t my_slot = ll_region(p.world, p.max_bytes, ch) + (static_cast<size_t>(buf) * p.world + p.rank) * kLlSlotBytes;
  const uint2* src = reinterpret_cast<const uint2*>(p.in);
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * kArThreads + threadIdx.x; u < p.nvec;
       u += static_cast<int64_t>(gridDim.x) * kArThreads) {
    const uint2 own = src[u];
    const uint4 line = make_uint4(own.x, epoch, own.y, epoch);
#pragma unroll 1
    for (int r = 0; r < p.world; ++r)
      if (r != p.rank) st_volatile16(p.inbox[r] + my_slot + u * 16, line);
  }
}

template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
  uint8_t* mine = p.inbox[p.rank];
  Control* ctl = reinterpret_cast<Control*>(mine + control_offset(p.world, p.max_bytes));
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&ctl->epoch) + 1u;
  const int buf = epoch & 1u;
  const int64_t per_cta = (p.nvec + gridDim.x - 1) / gridDim.x;
  const int64_t v0 = blockIdx.x * per_cta;
  const int64_t v1 = (v0 + per_cta < p.nvec) ? v0 + per_cta : p.nvec;
  const size_t slot_off = (static_cast<size_t>(buf) * p.world + p.rank) * static_cast<size_t>(p.max_bytes);

  // ---- push my range into slot `rank` of every inbox ------------------------------------------------
  const uint4* src = reinterpret_cast<const uint4*>(p.in);
  for (int64_t v = v0 + threadIdx.x; v < v1; v += kArThreads) {
    const uint4 val = src[v];
#pragma unroll 1
    for (int r = 0; r < p.world; ++r) reinterpret_cast<uint4*>(p.inbox[r] + slot_off)[v] = val;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world) {
    unsigned int* flag = reinterpret_cast<unsigned int*>(p.inbox[threadIdx.x] + flags_offset(p.world, p.max_bytes)) +
                         (static_cast<size_t>(buf) * p.world + p.rank) * kMaxCtas + blockIdx.x;
    st_release_sys(flag, epoch);
  }

  // ---- wait for the same CTA of every rank (bounded) --------------------------------------------------
  __shared__ int gave_up;
  if (threadIdx.x == 0) gave_up = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const unsigned int* flag =
        reinterpret_cast<const unsigned int*>(mine + flags_offset(p.world, p.max_bytes)) +
        (static_cast<size_t>(buf) * p.world + threadIdx.x) * kMaxCtas + blockIdx.x;
    const unsigned long long t0 = global_ns();
    while (ld_acquire_sys(flag) != epoch) {
      if (global_ns() - t0 > p.timeout_ns) {
        gave_up = 1;
        atomicExch(&ctl->status, LRI_ERR_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();

  // ---- reduce the slots of my range in rank order ------------------------------------------------------
  if (!gave_up) {
    uint4* dst = reinterpret_cast<uint4*>(p.out);
    const uint8_t* base = mine + static_cast<size_t>(buf) * p.world * static_cast<size_t>(p.max_bytes);
    for (int64_t v = v0 + threadIdx.x; v < v1; v += kArThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        float f[8];
        // volatile-strength load: the data was written by another GPU
        uint4 raw;
        const uint4* ptr = reinterpret_cast<const uint4*>(base + static_cast<size_t>(r) * p.max_bytes) + v;
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "l"(ptr)
                     : "memory");
        unpack8<T>(raw, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
      dst[v] = pack8<T>(acc);
    }
  }

  // ---- the last CTA to retire advances the epoch ---------------------------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(&ctl->ticket, 1u);
    if (t == gridDim.x - 1) {
      ctl->ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(&ctl->epoch) = epoch;
    }
  }
}

}  // namespace
}  // namespace lri

using namespace lri;

extern "C" int lri_comm_create(int rank, int world, int64_t max_elems, lri_comm** comm_out,
                               unsigned char ipc_handle_out[64]) {
  LRI_REQUIRE(comm_out && ipc_handle_out, LRI_ERR_ARG, "comm_create: NULL output");
  LRI_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, LRI_ERR_ARG,
              "comm_create: rank=%d world=%d (world <= %d)", rank, world, kMaxWorld);
  LRI_REQUIRE(max_elems > 0 && max_elems <= (1ll << 28), LRI_ERR_ARG, "comm_create: max_elems=%lld",
              (long long)max_elems);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  lri_comm* c = new lri_comm();
  c->rank = rank, c->world = world;
  c->max_bytes = ((max_elems * 2 + 255) / 256) * 256;
  c->total_bytes = ll_region(world, c->max_bytes, kLlRegions);
  for (int i = 0; i < 8; ++i) c->peer[i] = nullptr;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->local), c->total_bytes);
  if (e != cudaSuccess) {
    delete c;
    return fail(LRI_ERR_CUDA, "comm_create: cudaMalloc(%zu) failed: %s", c->total_bytes, cudaGetErrorString(e));
  }
  e = cudaMemset(c->local, 0, c->total_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->local);
  if (e != cudaSuccess) {
    cudaFree(c->local);
    delete c;
    return fail(LRI_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
  }
  memcpy(ipc_handle_out, &h, 64);
  c->peer[rank] = c->local;
  *comm_out = c;
  return LRI_OK;
}

extern "C" int lri_comm_connect(lri_comm* c, const unsigned char* ipc_handles) {
  LRI_REQUIRE(c && ipc_handles, LRI_ERR_ARG, "comm_connect: NULL argument");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handles + 64 * r, 64);
    void* ptr = nullptr;
    LRI_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer[r] = static_cast<uint8_t*>(ptr);
  }
  return LRI_OK;
}

extern "C" int lri_allreduce(lri_comm* c, int dtype, const void* in, void* out, int64_t count, int timeout_ms,
                             lri_stream_t stream) {
  LRI_REQUIRE(c && in && out, LRI_ERR_ARG, "allreduce: NULL argument");
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "allreduce: dtype %d", dtype);
  LRI_REQUIRE(count > 0 && count % 8 == 0, LRI_ERR_UNSUPPORTED, "allreduce: count=%lld must be a positive multiple of 8",
              (long long)count);
  LRI_REQUIRE(count * 2 <= c->max_bytes, LRI_ERR_ARG, "allreduce: %lld elements exceed the inbox slot (%lld bytes)",
              (long long)count, (long long)c->max_bytes);
  LRI_REQUIRE(aligned16(in) && aligned16(out), LRI_ERR_ALIGN, "allreduce: in/out must be 16-byte aligned");
  for (int r = 0; r < c->world; ++r)
    LRI_REQUIRE(c->peer[r] != nullptr, LRI_ERR_ARG, "allreduce: peer %d is not connected", r);
  ArParams p{};
  for (int r = 0; r < c->world; ++r) p.inbox[r] = c->peer[r];
  p.in = in, p.out = out, p.nvec = count / 8, p.max_bytes = c->max_bytes, p.rank = c->rank, p.world = c->world;
  p.timeout_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull;
  cudaStream_t st0 = static_cast<cudaStream_t>(stream);
  if (count * 2 <= kLlMaxPayload && c->world > 1) {
    // small message: low-latency lines, one 8-byte payload unit per thread
    p.nvec = count / 4;
    int64_t blocks = (p.nvec + kArThreads - 1) / kArThreads;
    blocks = blocks > kMaxCtas ? kMaxCtas : blocks;
    if (dtype == LRI_BF16)
      allreduce_ll_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kArThreads, 0, st0>>>(p);
    else
      allreduce_ll_kernel<__half><<<static_cast<unsigned>(blocks), kArThreads, 0, st0>>>(p);
    LRI_LAUNCH_CHECK("allreduce_ll_kernel");
    return LRI_OK;
  }
  // one CTA per 8 KiB of message, at most kMaxCtas (every rank derives the same grid from count)
  int64_t ctas = (p.nvec + 511) / 512;
  ctas = ctas < 1 ? 1 : (ctas > kMaxCtas ? kMaxCtas : ctas);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == LRI_BF16)
    allreduce_oneshot_kernel<__nv_bfloat16><<<static_cast<unsigned>(ctas), kArThreads, 0, st>>>(p);
  else
    allreduce_oneshot_kernel<__half><<<static_cast<unsigned>(ctas), kArThreads, 0, st>>>(p);
  LRI_LAUNCH_CHECK("allreduce_oneshot_kernel");
  return LRI_OK;
}

extern "C" int64_t lri_comm_push_max_elems(void) { return kLlMaxPayload / 2; }

extern "C" int lri_comm_push(lri_comm* c, int channel, int dtype, const void* in, int64_t count, lri_stream_t stream) {
  LRI_REQUIRE(c && in, LRI_ERR_ARG, "comm_push: NULL argument");
  LRI_REQUIRE(channel >= 1 && channel <= kPushChannels, LRI_ERR_ARG, "comm_push: channel %d outside 1..%d", channel,
              kPushChannels);
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "comm_push: dtype %d", dtype);
  LRI_REQUIRE(count > 0 && count % 8 == 0 && count * 2 <= kLlMaxPayload, LRI_ERR_UNSUPPORTED,
              "comm_push: count=%lld must be a positive multiple of 8 and at most %lld", (long long)count,
              (long long)(kLlMaxPayload / 2));
  LRI_REQUIRE(aligned16(in), LRI_ERR_ALIGN, "comm_push: input must be 16-byte aligned");
  for (int r = 0; r < c->world; ++r)
    LRI_REQUIRE(c->peer[r] != nullptr, LRI_ERR_ARG, "comm_push: peer %d is not connected", r);
  ArParams p{};
  for (int r = 0; r < c->world; ++r) p.inbox[r] = c->peer[r];
  p.in = in, p.out = nullptr, p.nvec = count / 4, p.max_bytes = c->max_bytes, p.rank = c->rank, p.world = c->world;
  int64_t blocks = (p.nvec + kArThreads - 1) / kArThreads;
  blocks = blocks > kMaxCtas ? kMaxCtas : blocks;
  LRI_CUDA(launch_pdl(ll_push_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kArThreads), 0,
                      static_cast<cudaStream_t>(stream), p, channel));
  LRI_LAUNCH_CHECK("ll_push_kernel");
  return LRI_OK;
}

// lri_linear with the push fused into the projection's epilogue (decode, M <= 8 rows).
extern "C" int lri_linear_push(lri_comm* c, int channel, int dtype, const void* x, const void* w, const void* addend,
                               void* y, int64_t M, int N, int K, lri_stream_t stream) {
  LRI_REQUIRE(c && x && w && y, LRI_ERR_ARG, "linear_push: NULL argument");
  LRI_REQUIRE(channel >= 1 && channel <= kPushChannels, LRI_ERR_ARG, "linear_push: channel %d outside 1..%d", channel,
              kPushChannels);
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "linear_push: dtype %d", dtype);
  LRI_REQUIRE(M >= 1 && M <= kGemvMaxRows, LRI_ERR_UNSUPPORTED, "linear_push: M=%lld outside 1..%d", (long long)M,
              kGemvMaxRows);
  LRI_REQUIRE(N > 0 && N % 8 == 0 && K > 0 && K % 8 == 0 && M * N * 2 <= kLlMaxPayload, LRI_ERR_UNSUPPORTED,
              "linear_push: N=%d K=%d must be multiples of 8 and M*N*2 <= %lld bytes", N, K, (long long)kLlMaxPayload);
  LRI_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y), LRI_ERR_ALIGN, "linear_push: pointers must be 16-byte aligned");
  for (int r = 0; r < c->world; ++r)
    LRI_REQUIRE(c->peer[r] != nullptr, LRI_ERR_ARG, "linear_push: peer %d is not connected", r);
  LinearParams p{};
  p.x = x, p.w = w, p.y = y, p.addend = addend, p.m = static_cast<int>(M), p.n = N, p.k = K;
  for (int r = 0; r < c->world; ++r) p.push.inbox[r] = c->peer[r];
  uint8_t* ctl = c->local + control_offset(c->world, c->max_bytes);
  p.push.epoch_ptr = reinterpret_cast<const unsigned int*>(ctl + offsetof(Control, chan_epoch)) + channel;
  p.push.region_off = ll_region(c->world, c->max_bytes, channel);
  p.push.slot_bytes = kLlSlotBytes;
  p.push.world = c->world, p.push.rank = c->rank, p.push.enabled = 1;
  return gemv_launch(dtype, EPI_PLAIN, p, static_cast<cudaStream_t>(stream));
}

static int fill_source(lri_comm* c, int channel, const void* own, int64_t count, int timeout_ms, bool push, LlSource* s) {
  s->enabled = 0;
  s->push = 0;
  if (channel <= 0) return LRI_OK;
  LRI_REQUIRE(channel <= kPushChannels, LRI_ERR_ARG, "add_rmsnorm_gather: channel %d outside 1..%d", channel,
              kPushChannels);
  LRI_REQUIRE(own != nullptr && aligned16(own), LRI_ERR_ARG,
              "add_rmsnorm_gather: the rank's own partial is required (16-byte aligned) for a gathered addend");
  LRI_REQUIRE(count * 2 <= kLlMaxPayload, LRI_ERR_UNSUPPORTED, "add_rmsnorm_gather: %lld elements exceed a push message",
              (long long)count);
  uint8_t* ctl = c->local + control_offset(c->world, c->max_bytes);
  s->region = c->local + ll_region(c->world, c->max_bytes, channel);
  s->epoch_ptr = reinterpret_cast<unsigned int*>(ctl + offsetof(Control, chan_epoch)) + channel;
  s->ticket_ptr = reinterpret_cast<unsigned int*>(ctl + offsetof(Control, chan_ticket)) + channel;
  s->status_ptr = reinterpret_cast<int*>(ctl + offsetof(Control, status));
  s->own = own;
  s->slot_bytes = kLlSlotBytes;
  s->timeout_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull;
  s->world = c->world, s->rank = c->rank;
  s->enabled = 1;
  if (push) {
    for (int r = 0; r < c->world; ++r) {
      LRI_REQUIRE(c->peer[r] != nullptr, LRI_ERR_ARG, "add_rmsnorm_allreduce: peer %d is not connected", r);
      s->peer_region[r] = c->peer[r] + ll_region(c->world, c->max_bytes, channel);
    }
    s->push = 1;
  }
  return LRI_OK;
}

static int gather_norm(lri_comm* c, int dtype, const void* residual, int channel1, const void* add1, int channel2,
                       const void* add2, float residual_scale, const void* weight, float eps, void* residual_out,
                       void* normed_out, int64_t rows, int dim, int timeout_ms, bool push, lri_stream_t stream) {
  LRI_REQUIRE(c && residual, LRI_ERR_ARG, "add_rmsnorm_gather: NULL argument");
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "add_rmsnorm_gather: dtype %d", dtype);
  LRI_REQUIRE(rows >= 0 && rows < (1ll << 31) && dim > 0, LRI_ERR_ARG, "add_rmsnorm_gather: rows=%lld dim=%d",
              (long long)rows, dim);
  LRI_REQUIRE((normed_out == nullptr) == (weight == nullptr), LRI_ERR_ARG,
              "add_rmsnorm_gather: weight and normed_out must both be given or both be NULL");
  LRI_REQUIRE(normed_out != nullptr || residual_out != nullptr, LRI_ERR_ARG, "add_rmsnorm_gather: no output");
  LRI_REQUIRE(aligned16(residual) && aligned16(add1) && aligned16(add2) && aligned16(weight) &&
                  aligned16(residual_out) && aligned16(normed_out),
              LRI_ERR_ALIGN, "add_rmsnorm_gather: pointers must be 16-byte aligned");
  GatherArgs g{};
  int rc = fill_source(c, channel1, add1, rows * dim, timeout_ms, push, &g.s1);
  if (rc != LRI_OK) return rc;
  rc = fill_source(c, channel2, add2, rows * dim, timeout_ms, push, &g.s2);
  if (rc != LRI_OK) return rc;
  return launch_add_rmsnorm_gather(dtype, residual, add1, add2, residual_scale, weight, eps, residual_out, normed_out,
                                   rows, dim, g, static_cast<cudaStream_t>(stream));
}

extern "C" int lri_add_rmsnorm_gather(lri_comm* c, int dtype, const void* residual, int channel1, const void* add1,
                                      int channel2, const void* add2, float residual_scale, const void* weight,
                                      float eps, void* residual_out, void* normed_out, int64_t rows, int dim,
                                      int timeout_ms, lri_stream_t stream) {
  return gather_norm(c, dtype, residual, channel1, add1, channel2, add2, residual_scale, weight, eps, residual_out,
                     normed_out, rows, dim, timeout_ms, false, stream);
}

// All-reduce + add + RMSNorm in one launch: as lri_add_rmsnorm_gather, but nothing has been pushed
// beforehand; the kernel stores this rank's partials into the peers' inboxes itself before it polls.
extern "C" int lri_add_rmsnorm_allreduce(lri_comm* c, int dtype, const void* residual, int channel1, const void* add1,
                                         int channel2, const void* add2, float residual_scale, const void* weight,
                                         float eps, void* residual_out, void* normed_out, int64_t rows, int dim,
                                         int timeout_ms, lri_stream_t stream) {
  return gather_norm(c, dtype, residual, channel1, add1, channel2, add2, residual_scale, weight, eps, residual_out,
                     normed_out, rows, dim, timeout_ms, true, stream);
}

extern "C" int lri_comm_status(lri_comm* c, lri_stream_t stream) {
  LRI_REQUIRE(c, LRI_ERR_ARG, "comm_status: NULL comm");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Control h;
  uint8_t* ctl = c->local + control_offset(c->world, c->max_bytes);
  LRI_CUDA(cudaMemcpyAsync(&h, ctl, sizeof(Control), cudaMemcpyDeviceToHost, st));
  LRI_CUDA(cudaStreamSynchronize(st));
  if (h.status != LRI_OK) {
    LRI_CUDA(cudaMemsetAsync(ctl + offsetof(Control, status), 0, sizeof(int), st));
    LRI_CUDA(cudaStreamSynchronize(st));
    return fail(LRI_ERR_TIMEOUT, "allreduce: a peer flag did not arrive within the timeout (rank %d)", c->rank);
  }
  return LRI_OK;
}

extern "C" int lri_comm_destroy(lri_comm* c) {
  if (!c) return LRI_OK;
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank && c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
  cudaFree(c->local);
  delete c;
  return LRI_OK;
}
