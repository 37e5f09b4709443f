// Small-batch linear layers (9..64 token rows) on the tcgen05 tensor cores: a weight-streaming
// "stream-K" GEMM.
//
// The weights are the 128-row operand of tcgen05.mma (the token rows sit on the N side, 16, 32
// or 64 wide), so a decode batch does not waste the tensor-core tile.  The kernel is HBM-bound:
// what matters is that all SMs stream weights all the time.  The work is therefore not cut by
// output tile but by bytes: the (tile, K tile) pairs are numbered tile-major and dealt out to
// one persistent CTA per SM in equal contiguous runs, whatever the shape of the projection.  A
// CTA's run covers the end of one tile, some whole tiles and the start of another; each of these
// segments is accumulated in TMEM.  A segment that is a whole tile gets the projection's epilogue
// straight from registers (store + addend, SwiGLU).  A segment of a tile that is shared with
// other CTAs is written as an fp32 partial tile to the workspace, and a second, wide kernel sums
// the segments of those tiles in a fixed order and applies the epilogue (RoPE + KV-cache scatter
// always takes this route: its dependent loads want many threads, not 128).
//
// For the gate/up projection a tile is 128 up rows plus the 128 matching gate rows, accumulated
// side by side in TMEM, so that a thread holds both halves of its SwiGLU outputs.
//
// Warp roles as in the prefill GEMM: warp 0 TMA producer, warp 1 MMA issuer (and TMEM owner),
// warps 2-5 epilogue; shared-memory ring of (full, empty) mbarriers running across segments;
// two accumulator buffers in TMEM so that an epilogue overlaps the next segment's main loop.
// Weight tiles are fetched as single 128-row boxes (measured: two 64-row boxes cost 8 %).
// Every mbarrier wait is bounded (device status word, see lri_gemm_status).
#include "linear.cuh"
#include "tcgen05.cuh"

namespace lri {
namespace {

using namespace tc;

__device__ int g_streamk_status = 0;

struct StreamKParams {
  LinearParams lin;  // m token rows, n outputs (SWIGLU: n = I, the weight has 2 I rows), k, epilogue fields
  float* partial;    // [tiles][max_seg][accumulators][BN][128] fp32
  int tiles;         // tiles of 128 outputs
  int total_kt;      // K tiles of 64 elements
  int max_seg;       // segments a tile may be cut into (capacity of `partial`)
  int ctas;          // CTAs of the GEMM kernel (the finishing kernel repeats its partition)
  int stages;
};

// units = (tile, K tile) pairs, tile-major; CTA b owns units [U b / G, U (b + 1) / G)
__device__ __forceinline__ int unit_start(int b, int64_t units, int ctas) {
  return static_cast<int>(units * b / ctas);
}
__device__ __forceinline__ int cta_of_unit(int64_t u, int64_t units, int ctas) {
  return static_cast<int>(((u + 1) * ctas - 1) / units);
}
// CTAs that hold a piece of `tile`: first one and how many
__device__ __forceinline__ void tile_segments(int tile, const StreamKParams& p, int& first_cta, int& nseg) {
  const int64_t units = static_cast<int64_t>(p.tiles) * p.total_kt;
  first_cta = cta_of_unit(static_cast<int64_t>(tile) * p.total_kt, units, p.ctas);
  const int last_cta = cta_of_unit(static_cast<int64_t>(tile + 1) * p.total_kt - 1, units, p.ctas);
  nseg = min(last_cta - first_cta + 1, p.max_seg);  // the host keeps the count within max_seg
}

template <int EPI>
struct Acc {
  static constexpr int kCount = EPI == EPI_SWIGLU ? 2 : 1;  // accumulators per tile (up, gate)
};

template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const StreamKParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int kAcc = Acc<EPI>::kCount;
  constexpr uint32_t kTileW = kBM * kBK * 2;
  constexpr uint32_t kTileX = BN * kBK * 2;
  constexpr uint32_t kStageBytes = kAcc * kTileW + kTileX;
  constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;      // TMEM columns of one accumulator
  constexpr uint32_t kBufCols = kAcc * kAccCols;        // one buffer = the accumulators of a segment
  constexpr uint32_t kTmemCols = 2 * kBufCols;          // 64 .. 256, a power of two

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint64_t bars[2 * 8 + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int64_t units = static_cast<int64_t>(p.tiles) * p.total_kt;
  const int u_begin = unit_start(blockIdx.x, units, p.ctas);
  const int u_end = unit_start(blockIdx.x + 1, units, p.ctas);

  const uint32_t full0 = smem_u32(&bars[0]);
  const uint32_t empty0 = smem_u32(&bars[8]);
  const uint32_t acc_full0 = smem_u32(&bars[16]);
  const uint32_t acc_empty0 = smem_u32(&bars[18]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t g = 0;
      bool ok = true;
      for (int u = u_begin; u < u_end && ok; ++u, ++g) {
        const int tile = u / p.total_kt;
        const int kt = u - tile * p.total_kt;
        const uint32_t s = g % static_cast<uint32_t>(stages);
        const uint32_t round = g / static_cast<uint32_t>(stages);
        ok = mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, &abort_flag, 11, &g_streamk_status);
        if (!ok) break;
        mbar_expect_tx(full0 + 8 * s, kStageBytes);
        const uint32_t dst = base + s * kStageBytes;
        tma_load_2d(dst, &tmap_w, full0 + 8 * s, kt * kBK, tile * kBM);
        if (kAcc == 2) tma_load_2d(dst + kTileW, &tmap_w, full0 + 8 * s, kt * kBK, p.lin.n + tile * kBM);  // gate rows
        tma_load_2d(dst + kAcc * kTileW, &tmap_x, full0 + 8 * s, kt * kBK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc<T>(BN);
      uint32_t g = 0;
      bool ok = true;
      int seg = 0;
      for (int u = u_begin; u < u_end && ok; ++seg) {
        const int tile = u / p.total_kt;
        const int kt0 = u - tile * p.total_kt;
        const int nk = min(p.total_kt - kt0, u_end - u);
        const uint32_t a = seg & 1;
        const uint32_t use = static_cast<uint32_t>(seg) >> 1;
        ok = mbar_wait(acc_empty0 + 8 * a, (use & 1u) ^ 1u, &abort_flag, 14, &g_streamk_status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + a * kBufCols;
        for (int kt = 0; kt < nk; ++kt, ++g) {
          const uint32_t s = g % static_cast<uint32_t>(stages);
          const uint32_t round = g / static_cast<uint32_t>(stages);
          ok = mbar_wait(full0 + 8 * s, round & 1u, &abort_flag, 12, &g_streamk_status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t pa = base + s * kStageBytes;
          const uint64_t xdesc = smem_desc_sw128(pa + kAcc * kTileW);
#pragma unroll
          for (int h = 0; h < kAcc; ++h) {
            const uint64_t wdesc = smem_desc_sw128(pa + h * kTileW);
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk)
              umma_f16(d_tmem + h * kAccCols, wdesc + 2 * kk, xdesc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);
        }
        if (ok) umma_commit(acc_full0 + 8 * a);
        u += nk;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int i = quarter * 32 + lane;  // row of the accumulator = output within the tile
    const int m = p.lin.m;
    int seg = 0;
    for (int u = u_begin; u < u_end; ++seg) {
      const int tile = u / p.total_kt;
      const int kt0 = u - tile * p.total_kt;
      const int nk = min(p.total_kt - kt0, u_end - u);
      u += nk;
      const uint32_t a = seg & 1;
      const uint32_t use = static_cast<uint32_t>(seg) >> 1;
      // tcgen05.ld below is warp-collective: the warp leaves together or not at all
      const bool ok = mbar_wait(acc_full0 + 8 * a, use & 1u, &abort_flag, 13, &g_streamk_status);
      if (!__all_sync(0xffffffffu, ok)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

      // accumulators -> registers (thread i holds output i of the tile for every token), then
      // the MMA warp may have the buffer back
      uint32_t acc[kAcc][kAccCols];
#pragma unroll
      for (int h = 0; h < kAcc; ++h)
#pragma unroll
        for (int cc = 0; cc < BN; cc += 32) {
          const uint32_t taddr =
              tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kBufCols + h * kAccCols + cc;
          tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&acc[h][cc]));
        }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(acc_empty0 + 8 * a);

      int first_cta, nseg;
      tile_segments(tile, p, first_cta, nseg);
      if (nseg > 1 || EPI == EPI_QKV) {
        // shared tile (or RoPE epilogue): leave the segment for the finishing kernel
        const int slot = static_cast<int>(blockIdx.x) - first_cta;
        if (slot < nseg) {
          float* dst = p.partial + (static_cast<int64_t>(tile) * p.max_seg + slot) * (kAcc * BN * kBM) + i;
#pragma unroll
          for (int h = 0; h < kAcc; ++h)
#pragma unroll
            for (int e = 0; e < BN; ++e)
              if (e < m) dst[(h * BN + e) * kBM] = __uint_as_float(acc[h][e]);
        }
        continue;
      }

      // whole tile: the projection's epilogue straight from registers
      const int64_t n = static_cast<int64_t>(tile) * kBM + i;
      if (n >= p.lin.n) continue;
      T* y = static_cast<T*>(p.lin.y) + n;
      if (EPI == EPI_PLAIN) {
        const T* add = p.lin.addend ? static_cast<const T*>(p.lin.addend) + n : nullptr;
#pragma unroll
        for (int e = 0; e < BN; ++e) {
          if (e < m) {
            float v = rnd<T>(__uint_as_float(acc[0][e]));
            if (add) v = rnd<T>(v + Num<T>::to_f(add[static_cast<int64_t>(e) * p.lin.n]));
            y[static_cast<int64_t>(e) * p.lin.n] = Num<T>::from_f(v);
          }
        }
      } else if (EPI == EPI_SWIGLU) {
#pragma unroll
        for (int e = 0; e < BN; ++e)
          if (e < m)
            y[static_cast<int64_t>(e) * p.lin.n] =
                swiglu_rounded<T>(rnd<T>(__uint_as_float(acc[0][e])), rnd<T>(__uint_as_float(acc[kAcc - 1][e])));
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land before shared memory is released
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Finishing kernel: grid (tile, group of tokens), one thread per token and output pair (PLAIN /
// QKV: 4 tokens per CTA) or output (SWIGLU: 2 tokens per CTA).  Tiles that the GEMM kernel
// completed itself are skipped; for the others the segments are summed in slot order and the
// epilogue is applied.
template <int EPI>
struct FinishShape {
  static constexpr int kTokens = EPI == EPI_SWIGLU ? 2 : 4;
};

template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(256) streamk_finish_kernel(const StreamKParams p) {
  constexpr int kAcc = Acc<EPI>::kCount;
  constexpr int kSlot = kAcc * BN * kBM;
  const int tile = blockIdx.x;
  int first_cta, nseg;
  tile_segments(tile, p, first_cta, nseg);
  pdl_wait();
  pdl_launch_dependents();
  if (nseg == 1 && EPI != EPI_QKV) return;
  const float* tile_partial = p.partial + static_cast<int64_t>(tile) * p.max_seg * kSlot;
  if (EPI == EPI_SWIGLU) {
    const int tok = blockIdx.y * FinishShape<EPI>::kTokens + (threadIdx.x >> 7);
    const int c = threadIdx.x & 127;
    const int64_t j = static_cast<int64_t>(tile) * kBM + c;
    if (tok >= p.lin.m || j >= p.lin.n) return;
    float up = 0.f, gate = 0.f;
    for (int z = 0; z < nseg; ++z) {
      up += tile_partial[z * kSlot + tok * kBM + c];
      gate += tile_partial[z * kSlot + (BN + tok) * kBM + c];
    }
    static_cast<T*>(p.lin.y)[static_cast<int64_t>(tok) * p.lin.n + j] = swiglu_rounded<T>(rnd<T>(up), rnd<T>(gate));
    return;
  }
  const int tok = blockIdx.y * FinishShape<EPI>::kTokens + (threadIdx.x >> 6);
  const int c = 2 * (threadIdx.x & 63);
  const int64_t n = static_cast<int64_t>(tile) * kBM + c;
  if (tok >= p.lin.m || n >= p.lin.n) return;
  float s0 = 0.f, s1 = 0.f;
  for (int z = 0; z < nseg; ++z) {
    const float2 v = *reinterpret_cast<const float2*>(tile_partial + z * kSlot + tok * kBM + c);
    s0 += v.x;
    s1 += v.y;
  }
  const float v0 = rnd<T>(s0), v1 = rnd<T>(s1);
  if (EPI == EPI_PLAIN) {
    float o0 = v0, o1 = v1;
    if (p.lin.addend) {
      const T* add = static_cast<const T*>(p.lin.addend) + static_cast<int64_t>(tok) * p.lin.n + n;
      o0 = rnd<T>(v0 + Num<T>::to_f(add[0]));
      o1 = rnd<T>(v1 + Num<T>::to_f(add[1]));
    }
    *reinterpret_cast<uint32_t*>(static_cast<T*>(p.lin.y) + static_cast<int64_t>(tok) * p.lin.n + n) = pack2<T>(o0, o1);
  } else {
    qkv_epilogue_pair<T>(p.lin, tok, n, v0, v1);
  }
}

int tiles_of(int n) { return (n + kBM - 1) / kBM; }
int token_tile(int64_t m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }
// A tile's K range is cut at CTA boundaries; with CTAs owning at least 1/148 of all units a tile
// spans at most ceil(148 / tiles) + 1 of them.  The launch keeps to min(that, kMaxSplitK).
int max_segments(int tiles) {
  const int s = (sm_count() + tiles - 1) / tiles + 1;
  return s < kMaxSplitK ? s : kMaxSplitK;
}

// CTAs of the GEMM kernel: one per SM, fewer when the projection is so small that a CTA would get
// less than q_min K tiles.  q_min K tiles per CTA bound the CTAs that can share one tile (a tile
// is total_kt consecutive units) by ceil(total_kt / q_min) + 1 <= max_seg, the capacity of the
// partial-tile workspace; the kernels rely on it.
int plan_ctas(int tiles, int total_kt, int max_seg) {
  const int64_t units = static_cast<int64_t>(tiles) * total_kt;
  const int q_min = (total_kt + max_seg - 2) / (max_seg - 1);
  int64_t ctas = units / q_min;
  ctas = ctas < 1 ? 1 : (ctas > sm_count() ? sm_count() : ctas);
  return static_cast<int>(ctas);
}

template <typename T, int BN, int EPI>
int launch(int dtype, const LinearParams& lin, float* partial, cudaStream_t st) {
  constexpr int kAcc = Acc<EPI>::kCount;
  StreamKParams p{};
  p.lin = lin;
  p.partial = partial;
  p.tiles = tiles_of(lin.n);
  p.total_kt = (lin.k + kBK - 1) / kBK;
  p.max_seg = max_segments(p.tiles);
  const int64_t w_rows = EPI == EPI_SWIGLU ? 2 * static_cast<int64_t>(lin.n) : lin.n;
  CUtensorMap tw, tx;
  int rc = make_tmap(&tw, dtype, lin.w, w_rows, lin.k, kBM);
  if (rc != LRI_OK) return rc;
  rc = make_tmap(&tx, dtype, lin.x, lin.m, lin.k, BN);
  if (rc != LRI_OK) return rc;
  constexpr int kStageBytes = (kAcc * kBM + BN) * kBK * 2;
  const int stages = kSmemBudget / kStageBytes;
  p.stages = stages > 8 ? 8 : stages;
  const int smem = p.stages * kStageBytes + 1024;
  auto kern = gemm_streamk_kernel<T, BN, EPI>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  LRI_ONCE_PER_DEVICE(attr_set, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024));
  const int64_t ctas = plan_ctas(p.tiles, p.total_kt, p.max_seg);
  p.ctas = static_cast<int>(ctas);
  LRI_CUDA(launch_pdl(kern, dim3(static_cast<unsigned>(ctas)), dim3(kGemmThreads), static_cast<size_t>(smem), st, tw, tx,
                      p));
  LRI_LAUNCH_CHECK("gemm_streamk_kernel");
  const unsigned token_groups = static_cast<unsigned>((lin.m + FinishShape<EPI>::kTokens - 1) / FinishShape<EPI>::kTokens);
  LRI_CUDA(launch_pdl(streamk_finish_kernel<T, BN, EPI>, dim3(static_cast<unsigned>(p.tiles), token_groups), dim3(256),
                      0, st, p));
  LRI_LAUNCH_CHECK("streamk_finish_kernel");
  return LRI_OK;
}

template <typename T, int BN>
int launch_epi(int dtype, int epi, const LinearParams& lin, float* partial, cudaStream_t st) {
  if (epi == EPI_PLAIN) return launch<T, BN, EPI_PLAIN>(dtype, lin, partial, st);
  if (epi == EPI_SWIGLU) return launch<T, BN, EPI_SWIGLU>(dtype, lin, partial, st);
  return launch<T, BN, EPI_QKV>(dtype, lin, partial, st);
}

template <typename T>
int launch_bn(int dtype, int epi, const LinearParams& lin, float* partial, cudaStream_t st) {
  if (lin.m <= 16) return launch_epi<T, 16>(dtype, epi, lin, partial, st);
  if (lin.m <= 32) return launch_epi<T, 32>(dtype, epi, lin, partial, st);
  return launch_epi<T, 64>(dtype, epi, lin, partial, st);
}

}  // namespace

size_t gemm_streamk_workspace_bytes(int epi, int64_t m, int n) {
  if (m < 1 || m > kSplitKMaxRows || n < 1) return 0;
  const int tiles = tiles_of(n);
  return static_cast<size_t>(tiles) * max_segments(tiles) * (epi == EPI_SWIGLU ? 2 : 1) * token_tile(m) * kBM *
         sizeof(float);
}

bool gemm_streamk_supports(int epi, const LinearParams& lin, const void* workspace, size_t workspace_bytes) {
  if (lin.m < 1 || lin.m > kSplitKMaxRows || lin.n < 2 || lin.n % 2 != 0 || lin.k < 8 || lin.k % 8 != 0) return false;
  if (!aligned16(lin.x) || !aligned16(lin.w) || workspace == nullptr || !aligned16(workspace)) return false;
  const size_t need = gemm_streamk_workspace_bytes(epi, lin.m, lin.n);
  return need > 0 && workspace_bytes >= need;
}

int gemm_streamk_launch(int dtype, int epi, const LinearParams& lin, void* workspace, size_t workspace_bytes,
                        cudaStream_t st) {
  if (!gemm_streamk_supports(epi, lin, workspace, workspace_bytes))
    return fail(LRI_ERR_ARG, "gemm stream-K: unsupported shape or workspace");
  float* partial = static_cast<float*>(workspace);
  return dtype == LRI_BF16 ? launch_bn<__nv_bfloat16>(dtype, epi, lin, partial, st)
                           : launch_bn<__half>(dtype, epi, lin, partial, st);
}

// The partition a launch would use (host arithmetic only; lets the plan be checked without a GPU).
void gemm_streamk_plan(int epi, int64_t m, int n, int k, int* tiles, int* k_tiles, int* max_seg, int* ctas,
                       int* token_tile_out) {
  (void)epi;
  *tiles = tiles_of(n);
  *k_tiles = (k + kBK - 1) / kBK;
  *max_seg = max_segments(*tiles);
  *ctas = plan_ctas(*tiles, *k_tiles, *max_seg);
  *token_tile_out = token_tile(m);
}

int gemm_streamk_status_read_and_clear(int* status_out) {
  int v = 0;
  LRI_CUDA(cudaMemcpyFromSymbol(&v, g_streamk_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    LRI_CUDA(cudaMemcpyToSymbol(g_streamk_status, &zero, sizeof(int)));
  }
  *status_out = v;
  return LRI_OK;
}

}  // namespace lri
