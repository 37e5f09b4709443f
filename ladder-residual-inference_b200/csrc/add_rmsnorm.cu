// F1: residual add (two- or three-way, optional residual scale) fused with RMSNorm, plus the
// embedding gather.  One CTA per token row; the row stays in registers between the add, the
// mean-square reduction and the normalisation, so it is read once and each output written once.
#include "p2p_ll.cuh"

namespace lri {
namespace {

constexpr int kNormThreads = 256;    // threads of a CTA when there are many rows (prompt pass)
constexpr int kMaxVecPerThread = 8;  // 256 threads * 8 vectors * 8 elements = dim up to 16384
constexpr int kFewRows = 16;         // up to here a row gets up to 1024 threads: the kernel is a latency chain

// GATHER: an addend whose source is enabled in `g` is not read from a pointer but summed over the
// ranks' low-latency lines (the reduction half of an all-reduce, done where the sum is used).
// NV = 16-byte vectors a thread keeps in registers (dim <= THREADS * 8 * NV): sized to the row so that a
// 4096-wide row costs a quarter of the registers of a 16384-wide one and more rows are resident per SM.
// THREADS: 256 for many rows; a decode step has a handful of rows, one CTA each, and the kernel's
// duration is the latency of one thread's loads and polls, so the row is spread over up to 1024 threads.
template <typename T, bool GATHER, int NV, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(const T* residual /* may alias residual_out */, const T* __restrict__ add1, const T* __restrict__ add2,
                   float residual_scale, const T* __restrict__ weight, float eps, T* residual_out,
                   T* __restrict__ normed_out, int dim, const GatherArgs g) {
  const int64_t row = blockIdx.x;
  const int nvec = dim >> 3;
  const uint4* r4 = reinterpret_cast<const uint4*>(residual + row * dim);
  const uint4* a4 = add1 ? reinterpret_cast<const uint4*>(add1 + row * dim) : nullptr;
  const uint4* b4 = add2 ? reinterpret_cast<const uint4*>(add2 + row * dim) : nullptr;
  uint4* ro4 = residual_out ? reinterpret_cast<uint4*>(residual_out + row * dim) : nullptr;

  // the norm weight is a constant of the model: fetch it while the preceding kernel drains
  uint4 wq[NV];
  if (weight != nullptr) {
    const uint4* w4 = reinterpret_cast<const uint4*>(weight);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) wq[i] = __ldg(w4 + v);
    }
  }
  // A kernel that gathers from the peers waits for NVLink: dependents launched now would sit resident
  // on the SMs for that long and take them from the kernels of the other stream.  It lets them go
  // once the peers' lines have arrived.
  const bool waits_for_peers = GATHER && (g.s1.enabled || g.s2.enabled);
  if (!waits_for_peers) pdl_launch_dependents();
  pdl_wait();  // the residual and the addends come from the preceding kernels
  unsigned int epoch1 = 0, epoch2 = 0;
  unsigned long long t0 = 0;
  if (GATHER) {
    // the message to read is the one after the last consumed one
    if (g.s1.enabled) epoch1 = *reinterpret_cast<const volatile unsigned int*>(g.s1.epoch_ptr) + 1u;
    if (g.s2.enabled) epoch2 = *reinterpret_cast<const volatile unsigned int*>(g.s2.epoch_ptr) + 1u;
    t0 = ll_global_ns();
    // a consumer that is its own producer sends everything it owns before it waits for anything
    if ((g.s1.enabled && g.s1.push) || (g.s2.enabled && g.s2.push)) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
          const int64_t elem = row * dim + static_cast<int64_t>(v) * 8;
          if (g.s1.enabled && g.s1.push) ll_push8<T>(g.s1, epoch1, elem);
          if (g.s2.enabled && g.s2.push) ll_push8<T>(g.s2, epoch2, elem);
        }
      }
    }
  }
  float vals[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float x[8];
      unpack8<T>(r4[v], x);
      if (residual_scale != 1.0f) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = rnd<T>(x[e] * residual_scale);
      }
      if (GATHER && g.s1.enabled) {
        float a[8];
        ll_gather8<T>(g.s1, epoch1, row * dim + static_cast<int64_t>(v) * 8, a, t0);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = rnd<T>(x[e] + a[e]);
      } else if (a4) {
        float a[8];
        unpack8<T>(a4[v], a);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = rnd<T>(x[e] + a[e]);
      }
      if (GATHER && g.s2.enabled) {
        float b[8];
        ll_gather8<T>(g.s2, epoch2, row * dim + static_cast<int64_t>(v) * 8, b, t0);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = rnd<T>(x[e] + b[e]);
      } else if (b4) {
        float b[8];
        unpack8<T>(b4[v], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = rnd<T>(x[e] + b[e]);
      }
      if (ro4) ro4[v] = pack8<T>(x);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        vals[i][e] = x[e];
        ss += x[e] * x[e];
      }
    }
  }
  if (waits_for_peers) pdl_launch_dependents();
  if (GATHER) {
    __syncthreads();  // every thread of this CTA has finished reading the peers' lines
    if (threadIdx.x == 0) {
      if (g.s1.enabled) ll_mark_consumed(g.s1, epoch1);
      if (g.s2.enabled) ll_mark_consumed(g.s2, epoch2);
    }
  }
  if (normed_out == nullptr) return;

  __shared__ float warp_part[THREADS / 32];
  __shared__ float inv_shared;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < THREADS / 32 ? warp_part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) inv_shared = rsqrtf(t / static_cast<float>(dim) + eps);
  }
  __syncthreads();
  const float inv = inv_shared;
  uint4* n4 = reinterpret_cast<uint4*>(normed_out + row * dim);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float w[8], y[8];
      unpack8<T>(wq[i], w);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = rnd<T>(vals[i][e] * inv) * w[e];
      n4[v] = pack8<T>(y);
    }
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(128)
embedding_kernel(const T* __restrict__ table, const I* __restrict__ idx, T* __restrict__ out, int dim,
                 int64_t vocab) {
  const int64_t tok = blockIdx.x;
  int64_t id = static_cast<int64_t>(idx[tok]);
  // An id outside the table would be an index error in the reference; clamp so that the
  // read stays inside the table instead of faulting.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + id * dim);
  uint4* dst = reinterpret_cast<uint4*>(out + tok * dim);
  for (int v = threadIdx.x; v < (dim >> 3); v += blockDim.x) dst[v] = src[v];
}

template <typename T, bool GATHER, int NV, int THREADS>
int launch_nv(const void* residual, const void* add1, const void* add2, float scale, const void* weight, float eps,
              void* residual_out, void* normed_out, int64_t rows, int dim, const GatherArgs& g, cudaStream_t st) {
  LRI_CUDA(launch_pdl(add_rmsnorm_kernel<T, GATHER, NV, THREADS>, dim3(static_cast<unsigned>(rows)), dim3(THREADS), 0, st,
                      static_cast<const T*>(residual), static_cast<const T*>(add1), static_cast<const T*>(add2), scale,
                      static_cast<const T*>(weight), eps, static_cast<T*>(residual_out), static_cast<T*>(normed_out),
                      dim, g));
  LRI_LAUNCH_CHECK(GATHER ? "add_rmsnorm_kernel<gather>" : "add_rmsnorm_kernel");
  return LRI_OK;
}

template <typename T, bool GATHER>
int launch_sized(const void* residual, const void* add1, const void* add2, float scale, const void* weight, float eps,
                 void* residual_out, void* normed_out, int64_t rows, int dim, const GatherArgs& g, cudaStream_t st) {
#define LRI_NORM(NV, THREADS) \
  return launch_nv<T, GATHER, NV, THREADS>(residual, add1, add2, scale, weight, eps, residual_out, normed_out, rows, dim, g, st)
  const int nvec = dim / 8;
  if (rows <= kFewRows && nvec > kNormThreads) {
    if (nvec <= 512) LRI_NORM(1, 512);
    if constexpr (GATHER) {
      // the polling code keeps the peers' lines of a vector in registers: 512 threads is what fits without spilling
      if (nvec <= 1024) LRI_NORM(2, 512);
      LRI_NORM(4, 512);
    } else {
      if (nvec <= 1024) LRI_NORM(1, 1024);
      LRI_NORM(2, 1024);
    }
  }
  const int nv = (nvec + kNormThreads - 1) / kNormThreads;  // vectors per thread
  if (nv <= 1) LRI_NORM(1, kNormThreads);
  if (nv <= 2) LRI_NORM(2, kNormThreads);
  if (nv <= 4) LRI_NORM(4, kNormThreads);
  LRI_NORM(kMaxVecPerThread, kNormThreads);
#undef LRI_NORM
}

template <typename T>
int launch_add_rmsnorm(const void* residual, const void* add1, const void* add2, float scale,
                       const void* weight, float eps, void* residual_out, void* normed_out, int64_t rows,
                       int dim, cudaStream_t st) {
  return launch_sized<T, false>(residual, add1, add2, scale, weight, eps, residual_out, normed_out, rows, dim, GatherArgs{}, st);
}

template <typename T>
int launch_gather_typed(const void* residual, const void* add1, const void* add2, float scale, const void* weight,
                        float eps, void* residual_out, void* normed_out, int64_t rows, int dim, const GatherArgs& g,
                        cudaStream_t st) {
  return launch_sized<T, true>(residual, add1, add2, scale, weight, eps, residual_out, normed_out, rows, dim, g, st);
}

}  // namespace

int launch_add_rmsnorm_gather(int dtype, const void* residual, const void* add1, const void* add2, float scale,
                              const void* weight, float eps, void* residual_out, void* normed_out, int64_t rows,
                              int dim, const GatherArgs& g, cudaStream_t st) {
  if (dim <= 0 || dim % 8 != 0 || dim > kNormThreads * kMaxVecPerThread * 8)
    return fail(LRI_ERR_UNSUPPORTED, "add_rmsnorm_gather: dim=%d", dim);
  if (rows <= 0) return LRI_OK;
  return dtype == LRI_BF16 ? launch_gather_typed<__nv_bfloat16>(residual, add1, add2, scale, weight, eps, residual_out,
                                                                normed_out, rows, dim, g, st)
                           : launch_gather_typed<__half>(residual, add1, add2, scale, weight, eps, residual_out,
                                                         normed_out, rows, dim, g, st);
}
}  // namespace lri

extern "C" int lri_add_rmsnorm(int dtype, const void* residual, const void* add1, const void* add2,
                               float residual_scale, const void* weight, float eps, void* residual_out,
                               void* normed_out, int64_t rows, int dim, lri_stream_t stream) {
  using namespace lri;
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "add_rmsnorm: dtype %d", dtype);
  LRI_REQUIRE(residual != nullptr, LRI_ERR_ARG, "add_rmsnorm: residual is NULL");
  LRI_REQUIRE(rows >= 0 && rows < (1ll << 31), LRI_ERR_ARG, "add_rmsnorm: rows=%lld", (long long)rows);
  LRI_REQUIRE(dim > 0 && dim % 8 == 0, LRI_ERR_UNSUPPORTED, "add_rmsnorm: dim=%d must be a positive multiple of 8", dim);
  LRI_REQUIRE(dim <= kNormThreads * kMaxVecPerThread * 8, LRI_ERR_UNSUPPORTED, "add_rmsnorm: dim=%d > %d", dim,
              kNormThreads * kMaxVecPerThread * 8);
  LRI_REQUIRE((normed_out == nullptr) == (weight == nullptr), LRI_ERR_ARG,
              "add_rmsnorm: weight and normed_out must both be given or both be NULL");
  LRI_REQUIRE(normed_out != nullptr || residual_out != nullptr, LRI_ERR_ARG, "add_rmsnorm: no output");
  LRI_REQUIRE(aligned16(residual) && aligned16(add1) && aligned16(add2) && aligned16(weight) &&
                  aligned16(residual_out) && aligned16(normed_out),
              LRI_ERR_ALIGN, "add_rmsnorm: pointers must be 16-byte aligned");
  if (rows == 0) return LRI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == LRI_BF16
             ? launch_add_rmsnorm<__nv_bfloat16>(residual, add1, add2, residual_scale, weight, eps, residual_out,
                                                 normed_out, rows, dim, st)
             : launch_add_rmsnorm<__half>(residual, add1, add2, residual_scale, weight, eps, residual_out,
                                          normed_out, rows, dim, st);
}

extern "C" int lri_embedding(int dtype, const void* table, const void* idx, int idx_is_i64, void* out,
                             int64_t n_tokens, int dim, int64_t vocab, lri_stream_t stream) {
  using namespace lri;
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "embedding: dtype %d", dtype);
  LRI_REQUIRE(table && idx && out, LRI_ERR_ARG, "embedding: NULL pointer");
  LRI_REQUIRE(n_tokens >= 0 && n_tokens < (1ll << 31) && vocab > 0, LRI_ERR_ARG, "embedding: bad extent");
  LRI_REQUIRE(dim > 0 && dim % 8 == 0, LRI_ERR_UNSUPPORTED, "embedding: dim=%d must be a multiple of 8", dim);
  LRI_REQUIRE(aligned16(table) && aligned16(out), LRI_ERR_ALIGN, "embedding: pointers must be 16-byte aligned");
  if (n_tokens == 0) return LRI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(n_tokens);
  // both 16-bit types move as raw 16-byte vectors
  using T = __nv_bfloat16;
  if (idx_is_i64)
    embedding_kernel<T, int64_t><<<grid, 128, 0, st>>>(static_cast<const T*>(table), static_cast<const int64_t*>(idx),
                                                       static_cast<T*>(out), dim, vocab);
  else
    embedding_kernel<T, int32_t><<<grid, 128, 0, st>>>(static_cast<const T*>(table), static_cast<const int32_t*>(idx),
                                                       static_cast<T*>(out), dim, vocab);
  LRI_LAUNCH_CHECK("embedding_kernel");
  return LRI_OK;
}
