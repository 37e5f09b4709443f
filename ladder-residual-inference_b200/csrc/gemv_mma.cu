// Weight-streaming linear layer for 2..16 token rows: the same HBM-bound row streaming as the
// SIMT GEMV, but the multiply-accumulate runs on the tensor cores (mma.sync m16n8k16) so that
// the instruction issue rate does not become the limit when every weight byte is used 16 times.
//
// A CTA owns one, two or four tiles of 16 weight rows (the M side of the MMA); the tokens are the
// N side (one or two 8-token tiles).  Operand fragments come straight from global memory with 16-byte loads: the
// MMA sums over k whatever order the k slots are in, as long as A and B agree, so each thread's
// four 2-element k slots of two consecutive MMAs are simply the 8 consecutive elements it loaded
// (thread c of a quad holds elements 8c..8c+7 of a 32-element block, for the weight row and for
// the token row alike).  Warps split K in interleaved chunks and reduce through
// shared memory; the first warps run the same fused epilogues as the SIMT kernel.  The two rows a thread
// holds (MMA row slots a and a+8) are mapped to the row pairs the epilogues need: (n, n+1) for
// the plain and QKV forms, (up j, gate I+j) for SwiGLU.
#include <cstdlib>

#include "linear.cuh"

namespace lri {
namespace {

constexpr int kMmaMaxWarps = 8;

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = number of 8-token tiles (1: up to 8 rows of x, 2: up to 16).
// MT = number of 16-row weight tiles per CTA.  Every CTA reads the whole activation block once
// (through L1/L2), so with MT tiles the activation traffic per weight byte drops by MT; wide
// projections use MT = 4, narrow ones keep MT = 1 so that there are enough CTAs.
template <typename T, int NT, int MT, int EPI>
__global__ void __launch_bounds__(kMmaMaxWarps * 32) gemv_mma_kernel(const LinearParams p) {
  constexpr int BLK = 4 / MT;  // 32-element k blocks per warp iteration: 8 weight loads in flight per thread
  constexpr int kChunk = 32 * BLK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int a = lane >> 2;  // MMA row slot (and slot a + 8); also the token column of the B fragment
  const int c = lane & 3;   // which 8 of the 32 elements of a k block
  const int K = p.k;
  const T* __restrict__ w = static_cast<const T*>(p.w);
  const T* __restrict__ x = static_cast<const T*>(p.x);

  // the two weight rows of this thread in every tile (clamped; rows past the end are computed, not stored)
  const T* w0[MT];
  const T* w1[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    int64_t row0, row1;
    if (EPI == EPI_SWIGLU) {
      int64_t j = (static_cast<int64_t>(blockIdx.x) * MT + mt) * 8 + a;
      j = j < p.n ? j : p.n - 1;
      row0 = j;        // up
      row1 = p.n + j;  // gate
    } else {
      row0 = (static_cast<int64_t>(blockIdx.x) * MT + mt) * 16 + 2 * a;
      row1 = row0 + 1;
      row0 = row0 < p.n ? row0 : p.n - 1;
      row1 = row1 < p.n ? row1 : p.n - 1;
    }
    w0[mt] = w + row0 * K + c * 8;
    w1[mt] = w + row1 * K + c * 8;
  }
  const T* xr[NT];
  bool xok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int tok = t * 8 + a;
    xok[t] = tok < p.m;
    xr[t] = x + static_cast<int64_t>(xok[t] ? tok : 0) * K + c * 8;
  }

  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][t][e] = 0.f;

  const int nchunks = (K + kChunk - 1) / kChunk;
  // One register buffer of weight vectors per thread.  (A second buffer, prefetching the warp's
  // next chunk during the MMAs, was measured slower: the registers cost a resident CTA per SM.)
  uint4 wa[MT][BLK], wb[MT][BLK];
  auto load_w = [&](int ch) {
#pragma unroll
    for (int j = 0; j < BLK; ++j) {
      const int k = ch * kChunk + j * 32;
      const bool ok = k + c * 8 < K;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        wa[mt][j] = ok ? ld_stream16(w0[mt] + k) : make_uint4(0, 0, 0, 0);
        wb[mt][j] = ok ? ld_stream16(w1[mt] + k) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  int ch = warp;
  load_w(ch);  // weights do not depend on the preceding kernel
  pdl_launch_dependents();
  pdl_wait();
  while (true) {
    uint4 xv[NT][BLK];
#pragma unroll
    for (int j = 0; j < BLK; ++j) {
      const int k = ch * kChunk + j * 32;
      const bool ok = k + c * 8 < K;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        xv[t][j] = (ok && xok[t]) ? __ldg(reinterpret_cast<const uint4*>(xr[t] + k)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < BLK; ++j) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816<T>(acc[mt][t], wa[mt][j].x, wb[mt][j].x, wa[mt][j].y, wb[mt][j].y, xv[t][j].x, xv[t][j].y);
          mma16816<T>(acc[mt][t], wa[mt][j].z, wb[mt][j].z, wa[mt][j].w, wb[mt][j].w, xv[t][j].z, xv[t][j].w);
        }
      }
    }
    ch += W;
    if (ch >= nchunks) break;
    load_w(ch);
  }

  // ---- reduce the K slices of the warps; warp mt finishes tile mt -----------------------------------
  __shared__ float red[kMmaMaxWarps][MT * NT * 4][32];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) red[warp][(mt * NT + t) * 4 + e][lane] = acc[mt][t][e];
  __syncthreads();
  // tiles are finished by the first warps of the CTA (a CTA with fewer warps than tiles loops)
  for (int mt = warp; mt < MT; mt += W) {
    float fin[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float s = 0.f;
        for (int wi = 0; wi < W; ++wi) s += red[wi][(mt * NT + t) * 4 + e][lane];
        fin[t][e] = s;
      }
    // fin[t][0], fin[t][1]: row slot a,     tokens t*8 + 2c, + 1
    // fin[t][2], fin[t][3]: row slot a + 8, tokens t*8 + 2c, + 1
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int tok = t * 8 + 2 * c + q;
        if (tok >= p.m) continue;
        const float v0 = rnd<T>(fin[t][q]);      // row0 of this thread
        const float v1 = rnd<T>(fin[t][2 + q]);  // row1
        if (EPI == EPI_SWIGLU) {
          const int64_t j = (static_cast<int64_t>(blockIdx.x) * MT + mt) * 8 + a;
          if (j < p.n) static_cast<T*>(p.y)[static_cast<int64_t>(tok) * p.n + j] = swiglu_rounded<T>(v0, v1);
        } else {
          const int64_t n = (static_cast<int64_t>(blockIdx.x) * MT + mt) * 16 + 2 * a;
          if (n >= p.n) continue;
          if (EPI == EPI_PLAIN) {
            T* y = static_cast<T*>(p.y) + static_cast<int64_t>(tok) * p.n;
            const T* add = p.addend ? static_cast<const T*>(p.addend) + static_cast<int64_t>(tok) * p.n : nullptr;
            y[n] = Num<T>::from_f(add ? v0 + Num<T>::to_f(add[n]) : v0);
            if (n + 1 < p.n) y[n + 1] = Num<T>::from_f(add ? v1 + Num<T>::to_f(add[n + 1]) : v1);
          } else {
            qkv_epilogue_pair<T>(p, tok, n, v0, v1);
          }
        }
      }
    }
  }
}

template <typename T, int NT, int MT, int EPI>
int launch_mma(const LinearParams& p, cudaStream_t st) {
  constexpr int kChunk = 32 * (4 / MT);
  const int nchunks = (p.k + kChunk - 1) / kChunk;
  int W = nchunks < kMmaMaxWarps ? nchunks : kMmaMaxWarps;
  W = W < 1 ? 1 : W;
  const int64_t per_cta = (EPI == EPI_SWIGLU ? 8 : 16) * MT;
  const int64_t grid = (p.n + per_cta - 1) / per_cta;
  LRI_CUDA(launch_pdl(gemv_mma_kernel<T, NT, MT, EPI>, dim3(static_cast<unsigned>(grid)), dim3(W * 32), 0, st, p));
  LRI_LAUNCH_CHECK("gemv_mma_kernel");
  return LRI_OK;
}

// Row tiles per CTA: as many as still leave about two CTAs per SM (LRI_GEMV_MT=1|2|4 overrides).
template <typename T, int NT, int EPI>
int launch_tiles(const LinearParams& p, cudaStream_t st) {
  const int forced = option(OPT_GEMV_MT);
  const int64_t tiles = (p.n + (EPI == EPI_SWIGLU ? 8 : 16) - 1) / (EPI == EPI_SWIGLU ? 8 : 16);
  int mt = tiles >= 4 * 296 ? 4 : (tiles >= 2 * 296 ? 2 : 1);
  if (forced) mt = forced;
  if (mt == 4) return launch_mma<T, NT, 4, EPI>(p, st);
  if (mt == 2) return launch_mma<T, NT, 2, EPI>(p, st);
  return launch_mma<T, NT, 1, EPI>(p, st);
}

template <typename T>
int dispatch(int epi, const LinearParams& p, cudaStream_t st) {
  const bool one = p.m <= 8;
  switch (epi) {
    case EPI_PLAIN: return one ? launch_tiles<T, 1, EPI_PLAIN>(p, st) : launch_tiles<T, 2, EPI_PLAIN>(p, st);
    case EPI_SWIGLU: return one ? launch_tiles<T, 1, EPI_SWIGLU>(p, st) : launch_tiles<T, 2, EPI_SWIGLU>(p, st);
    default: return one ? launch_tiles<T, 1, EPI_QKV>(p, st) : launch_tiles<T, 2, EPI_QKV>(p, st);
  }
}

}  // namespace

int gemv_mma_launch(int dtype, int epi, const LinearParams& p, cudaStream_t st) {
  if (p.m < 1 || p.m > kGemvMmaMaxRows) return fail(LRI_ERR_ARG, "gemv_mma: m=%d outside 1..%d", p.m, kGemvMmaMaxRows);
  return dtype == LRI_BF16 ? dispatch<__nv_bfloat16>(epi, p, st) : dispatch<__half>(epi, p, st);
}

}  // namespace lri
