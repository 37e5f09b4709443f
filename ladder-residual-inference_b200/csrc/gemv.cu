// Weight-streaming GEMV family for small-batch decode (M <= 8 token rows).
//
// y[m, n] = sum_k x[m, k] * W[n, k], W row-major [N, K] (the nn.Linear layout, K contiguous).
// The kernel is HBM-bound: every weight byte is read exactly once with 16-byte streaming
// loads that bypass L1, and a thread keeps R*U such loads in flight.  A CTA owns R weight
// rows; its warps split K in interleaved 256-element chunks, reduce with shuffles and then
// through shared memory; the few threads holding the final sums run the fused epilogue:
//   PLAIN   store (optionally + addend)                       wo / w2 / LM head
//   SWIGLU  rows (j, I + j) -> silu(gate) * up                 w1
//   QKV     rotate adjacent pairs, scatter q / k-cache / v-cache   wqkv
//   ARGMAX  no logits stored: arg-max over rows and ranks           LM head, greedy decoding (argmax.cuh)
#include <cstdlib>

#include "linear.cuh"

namespace lri {
namespace {

constexpr int kGemvMaxWarps = 8;

template <typename T, int M, int R, int U, int EPI>
__global__ void __launch_bounds__(kGemvMaxWarps * 32) gemv_kernel(const LinearParams p) {
  static_assert(R % 2 == 0, "epilogues work on pairs of rows");
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int W = blockDim.x >> 5;
  const int K = p.k;
  const T* __restrict__ w = static_cast<const T*>(p.w);
  const T* __restrict__ x = static_cast<const T*>(p.x);

  // weight rows of this CTA (clamped: rows past the end recompute the last row and are not stored)
  const T* wrow[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    int64_t row;
    if (EPI == EPI_SWIGLU) {
      int64_t j = static_cast<int64_t>(blockIdx.x) * (R / 2) + (r >> 1);
      j = j < p.n ? j : p.n - 1;
      row = (r & 1) ? p.n + j : j;  // even slot: up row j, odd slot: gate row I + j
    } else {
      row = static_cast<int64_t>(blockIdx.x) * R + r;
      row = row < p.n ? row : p.n - 1;
    }
    wrow[r] = w + row * K;
  }
  const T* xrow[M];
#pragma unroll
  for (int m = 0; m < M; ++m) xrow[m] = x + static_cast<int64_t>(m < p.m ? m : p.m - 1) * K;

  float acc[M][R];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[m][r] = 0.f;

  const int nchunks = (K + 255) >> 8;
  uint4 wv[U][R];
  auto load_w = [&](int c0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((c0 + u * W) << 8) + lane * 8;
      const bool ok = k < K;
#pragma unroll
      for (int r = 0; r < R; ++r) wv[u][r] = ok ? ld_stream16(wrow[r] + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // The weights do not depend on the preceding kernel: start streaming them, let the next kernel
  // begin its own prologue, and only then wait for the activations to be complete.
  int c0 = warp;
  load_w(c0);
  pdl_launch_dependents();
  pdl_wait();
  while (true) {
    uint4 xv[U][M];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((c0 + u * W) << 8) + lane * 8;
      const bool ok = k < K;
#pragma unroll
      for (int m = 0; m < M; ++m)
        xv[u][m] = ok ? __ldg(reinterpret_cast<const uint4*>(xrow[m] + k)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float xf[M][8];
#pragma unroll
      for (int m = 0; m < M; ++m) unpack8<T>(xv[u][m], xf[m]);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float wf[8];
        unpack8<T>(wv[u][r], wf);
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[m][r] = fmaf(wf[e], xf[m][e], acc[m][r]);
      }
    }
    c0 += W * U;
    if (c0 >= nchunks) break;
    load_w(c0);
  }

  __shared__ float red[kGemvMaxWarps][M * R];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float s = warp_sum(acc[m][r]);
      if (lane == 0) red[warp][m * R + r] = s;
    }
  __syncthreads();

  if (EPI == EPI_ARGMAX) {
    __shared__ unsigned long long best[M][R / 2];
    if (threadIdx.x < M * (R / 2)) {
      const int m = threadIdx.x / (R / 2), j = threadIdx.x % (R / 2);
      float s0 = 0.f, s1 = 0.f;
      for (int wi = 0; wi < W; ++wi) {
        s0 += red[wi][m * R + 2 * j];
        s1 += red[wi][m * R + 2 * j + 1];
      }
      // compare what the projection would have stored: logits rounded to the storage type
      const int64_t n = static_cast<int64_t>(blockIdx.x) * R + 2 * j;
      unsigned long long k = 0ull;
      if (n < p.n) k = argmax_key(rnd<T>(s0), p.am.index_offset + n);
      if (n + 1 < p.n) {
        const unsigned long long k1 = argmax_key(rnd<T>(s1), p.am.index_offset + n + 1);
        k = k1 > k ? k1 : k;
      }
      best[m][j] = k;
    }
    __syncthreads();
    if (threadIdx.x < p.m) {
      unsigned long long k = best[threadIdx.x][0];
#pragma unroll
      for (int j = 1; j < R / 2; ++j) k = best[threadIdx.x][j] > k ? best[threadIdx.x][j] : k;
      argmax_offer(p.am, threadIdx.x, k);
    }
    return;
  }
  if (threadIdx.x >= M * (R / 2)) return;
  const int m = threadIdx.x / (R / 2);
  const int j = threadIdx.x % (R / 2);
  if (m >= p.m) return;
  float s0 = 0.f, s1 = 0.f;
  for (int wi = 0; wi < W; ++wi) {
    s0 += red[wi][m * R + 2 * j];
    s1 += red[wi][m * R + 2 * j + 1];
  }
  // the projection's own rounding to the storage type (nn.Linear output)
  const float v0 = rnd<T>(s0), v1 = rnd<T>(s1);

  if (EPI == EPI_PLAIN) {
    const int64_t n = static_cast<int64_t>(blockIdx.x) * R + 2 * j;
    T* y = static_cast<T*>(p.y) + static_cast<int64_t>(m) * p.n;
    const T* add = p.addend ? static_cast<const T*>(p.addend) + static_cast<int64_t>(m) * p.n : nullptr;
    const float o0 = n < p.n ? rnd<T>(add ? v0 + Num<T>::to_f(add[n]) : v0) : 0.f;
    const float o1 = n + 1 < p.n ? rnd<T>(add ? v1 + Num<T>::to_f(add[n + 1]) : v1) : 0.f;
    if (n < p.n) y[n] = Num<T>::from_f(o0);
    if (n + 1 < p.n) y[n + 1] = Num<T>::from_f(o1);
    if (p.push.enabled && n + 1 < p.n) {
      // also hand the pair to every peer: 8 bytes {2 elements, epoch}, valid as soon as they land
      const unsigned int epoch = *reinterpret_cast<const volatile unsigned int*>(p.push.epoch_ptr) + 1u;
      const size_t off = p.push.region_off +
                         (static_cast<size_t>(epoch & 1u) * p.push.world + p.push.rank) * p.push.slot_bytes +
                         static_cast<size_t>((static_cast<int64_t>(m) * p.n + n) >> 1) * 8;
      const unsigned int data = pack2<T>(o0, o1);
#pragma unroll 1
      for (int r = 0; r < p.push.world; ++r)
        if (r != p.push.rank)
          asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p.push.inbox[r] + off), "r"(data), "r"(epoch)
                       : "memory");
    }
  } else if (EPI == EPI_SWIGLU) {
    const int64_t jj = static_cast<int64_t>(blockIdx.x) * (R / 2) + j;
    if (jj < p.n) static_cast<T*>(p.y)[static_cast<int64_t>(m) * p.n + jj] = swiglu_rounded<T>(v0, v1);
  } else {
    const int64_t n = static_cast<int64_t>(blockIdx.x) * R + 2 * j;  // even
    if (n >= p.n) return;
    qkv_epilogue_pair<T>(p, m, n, v0, v1);
  }
}

template <typename T, int M, int R, int U, int EPI>
int launch_gemv(const LinearParams& p, cudaStream_t st) {
  const int nchunks = (p.k + 255) >> 8;
  int W = (nchunks + U - 1) / U;
  W = W < 1 ? 1 : (W > kGemvMaxWarps ? kGemvMaxWarps : W);
  const int64_t per_cta = EPI == EPI_SWIGLU ? R / 2 : R;
  const int64_t grid = (p.n + per_cta - 1) / per_cta;
  LRI_CUDA(launch_pdl(gemv_kernel<T, M, R, U, EPI>, dim3(static_cast<unsigned>(grid)), dim3(W * 32), 0, st, p));
  LRI_LAUNCH_CHECK("gemv_kernel");
  return LRI_OK;
}

// Rows per CTA.  A CTA keeps R * U = 16 / M-dependent 16-byte weight loads in flight per thread
// whatever R is; fewer rows per CTA mean more, shorter CTAs (less wave quantisation on small
// projections), more rows mean fewer reductions.  Measured on the 8B shard shapes of 1, 2, 4 and 8
// ranks, 4 rows win everywhere except for a very short K (the output projection of a 1/8 shard,
// K = 512: one warp per CTA, 1.89 us with 8 rows against 2.21 us).  LRI_GEMV_R=2|4|8 overrides the choice.
int rows_per_cta(const LinearParams& p) {
  const int forced = option(OPT_GEMV_R);
  if (forced) return forced;
  return p.k <= 512 ? 8 : 4;
}

template <typename T, int EPI>
int dispatch_m(const LinearParams& p, cudaStream_t st) {
  const int r = rows_per_cta(p);
  // Half the loads in flight per thread: fewer registers, more resident CTAs.  For one token row it wins where a
  // long K meets 3072..6144 weight rows: 8B w2 21.95 -> 20.32 us (K = 14336), its half shard 11.94 -> 10.94 us
  // (K = 7168), QKV and wo at K = 4096 by 0.15-0.2 us, and the whole one-GPU decode step by 1.9 %; shorter K (the
  // 1/4 and 1/8 shards) and wider projections are unchanged or slightly slower with it, and the 2048-row w2 of
  // the 1B shape loses about 1 us.  LRI_GEMV_U=2 forces it for every one-row projection.
  const bool half_depth = option(OPT_GEMV_U) == 2 || (p.k >= 4096 && p.n >= 3072 && p.n <= 6144);
  if (half_depth && p.m <= 1 && r == 4) return launch_gemv<T, 1, 4, 2, EPI>(p, st);
#define LRI_GEMV_CASE(M_, U2, U4, U8)                                   \
  if (p.m <= M_) {                                                      \
    if (r == 2) return launch_gemv<T, M_, 2, U2, EPI>(p, st);           \
    if (r == 8) return launch_gemv<T, M_, 8, U8, EPI>(p, st);           \
    return launch_gemv<T, M_, 4, U4, EPI>(p, st);                       \
  }
  LRI_GEMV_CASE(1, 8, 4, 2)
  LRI_GEMV_CASE(2, 8, 4, 2)
  LRI_GEMV_CASE(4, 4, 2, 1)
  LRI_GEMV_CASE(8, 2, 1, 1)
#undef LRI_GEMV_CASE
  return fail(LRI_ERR_ARG, "gemv: m=%d", p.m);
}

template <typename T>
int dispatch_epi(int epi, const LinearParams& p, cudaStream_t st) {
  switch (epi) {
    case EPI_PLAIN: return dispatch_m<T, EPI_PLAIN>(p, st);
    case EPI_SWIGLU: return dispatch_m<T, EPI_SWIGLU>(p, st);
    case EPI_ARGMAX: return dispatch_m<T, EPI_ARGMAX>(p, st);
    default: return dispatch_m<T, EPI_QKV>(p, st);
  }
}

}  // namespace

int gemv_launch(int dtype, int epi, const LinearParams& p, cudaStream_t st) {
  if (p.m < 1 || p.m > kGemvMaxRows) return fail(LRI_ERR_ARG, "gemv: m=%d outside 1..%d", p.m, kGemvMaxRows);
  return dtype == LRI_BF16 ? dispatch_epi<__nv_bfloat16>(epi, p, st) : dispatch_epi<__half>(epi, p, st);
}

}  // namespace lri
