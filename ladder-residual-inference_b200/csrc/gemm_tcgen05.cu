// tcgen05 GEMM for sm_100a:  C[m, n] = sum_k A[m, k] * W[n, k]   (both operands K-major).
//
// Persistent CTAs (one per SM) work through 128 x BN output tiles.  Warp 0 is the TMA producer,
// warp 1 allocates TMEM and issues tcgen05.mma (one elected thread), warps 2-5 are the epilogue
// (each reads its own 32-lane quarter of TMEM with tcgen05.ld and stores C).  Operand tiles are
// 64 K-elements wide (128 bytes per row) and land in shared memory through plain single-CTA TMA
// loads in the 128-byte swizzle, which is also the layout the shared-memory matrix descriptors
// name.  A ring of mbarrier pairs (full / empty) pipelines the K loop and keeps running from one
// tile to the next; tcgen05.commit releases a stage.  Two accumulator buffers in TMEM let the
// epilogue of one tile overlap the main loop of the next.
//
// The 128-row operand of the instruction is the activation tile for prefill-sized m; for
// m <= 64 the operands are swapped (weights take the 128 rows, tokens the N side) so that
// small decode batches do not waste seven eighths of the tensor-core tile.
//
// Every wait on an mbarrier is bounded: when the poll budget runs out the kernel records an
// error in a device status word, stops waiting everywhere, frees its TMEM and returns.
#include <cstdlib>

#include "linear.cuh"
#include "tcgen05.cuh"

namespace lri {
namespace {

using namespace tc;

__device__ int g_gemm_status = 0;  // 0 ok, else the code of the first wait that gave up

struct GemmShape {
  int m, n, k;
};

// One unit of work of a persistent CTA: an output tile and a slice of K.
struct WorkItem {
  int tile_p, tile_q;
};
struct GemmGrid {
  int tiles_p, tiles_q;
  int group;  // P tiles per panel
};
// Order of the output tiles.  The P tiles are taken in panels of `group`; inside a panel the
// Q tile is the slow index.  The CTAs that run at the same time then share one panel of P
// (a few MB, stays in L2) and a handful of Q tiles, each of which all of them use at once, so
// that both operands come from DRAM about once per panel instead of once per P tile.
__device__ __forceinline__ WorkItem work_item(int item, const GemmGrid& g) {
  WorkItem w;
  const int panel_items = g.group * g.tiles_q;
  const int panel = item / panel_items;
  const int r = item - panel * panel_items;
  const int p0 = panel * g.group;
  const int gm = min(g.group, g.tiles_p - p0);
  w.tile_q = r / gm;
  w.tile_p = p0 + (r - w.tile_q * gm);
  return w;
}

// P = operand with 128 rows per tile, Q = operand with BN rows per tile.
// SWAP == false: P = A (tokens), Q = W;  D[i, j] -> C[tile_p*128 + i, tile_q*BN + j]
// SWAP == true : P = W,          Q = A;  D[i, j] -> C[tile_q*BN + j, tile_p*128 + i]
//
// The kernel is persistent: CTA b works through items b, b + gridDim.x, ...  The shared-memory
// ring keeps running across items (the producer is already fetching the next item's operands
// while the last MMAs of the current one execute) and the accumulator is double-buffered in
// TMEM, so the epilogue of item i overlaps the main loop of item i + 1.
//
// EPI (SWAP == false only) fuses the projection's epilogue into the store of the tile:
//   EPI_SWIGLU  the Q tile is BN/2 up rows followed by the BN/2 matching gate rows of w1, so that a
//               thread finds up_j and gate_j of its token in the same accumulator row; it stores
//               silu(gate) * up to h [m, I] (lin.y, lin.n = I)
//   EPI_QKV     a thread rotates the 16 adjacent pairs of each 32-column chunk of its token with the
//               table row of the token's position and stores them to q_out / k-cache / v-cache
template <typename T, int BN, bool SWAP, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                    T* __restrict__ c, GemmShape shape, GemmGrid grid, int stages, const LinearParams lin) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t kTileP = kBM * kBK * 2;
  constexpr uint32_t kTileQ = BN * kBK * 2;
  constexpr uint32_t kStageBytes = kTileP + kTileQ;
  constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;  // TMEM columns of one accumulator buffer
  constexpr uint32_t kTmemCols = 2 * kAccCols;      // a power of two between 64 and 512

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  __shared__ uint64_t bars[2 * 8 + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kt = (shape.k + kBK - 1) / kBK;
  const int items = grid.tiles_p * grid.tiles_q;

  const uint32_t full0 = smem_u32(&bars[0]);
  const uint32_t empty0 = smem_u32(&bars[8]);
  const uint32_t acc_full0 = smem_u32(&bars[16]);   // MMA -> epilogue, one per accumulator buffer
  const uint32_t acc_empty0 = smem_u32(&bars[18]);  // epilogue -> MMA

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 128);  // every epilogue thread arrives
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
  // everything above overlaps the tail of the preceding kernel when launched as its programmatic dependent
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t g = 0;  // K tiles loaded so far, over all items: position in the ring
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const WorkItem w = work_item(item, grid);
        for (int kt = 0; kt < num_kt; ++kt, ++g) {
          const uint32_t s = g % static_cast<uint32_t>(stages);
          const uint32_t round = g / static_cast<uint32_t>(stages);
          // a fresh barrier passes a wait on parity 1, so the first round does not block
          ok = mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, &abort_flag, 1, &g_gemm_status);
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          const uint32_t dst = base + s * kStageBytes;
          const int kx = kt * kBK;
          tma_load_2d(dst, &tmap_p, full0 + 8 * s, kx, w.tile_p * kBM);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(dst + kTileP, &tmap_q, full0 + 8 * s, kx, w.tile_q * (BN / 2));
            tma_load_2d(dst + kTileP + kTileQ / 2, &tmap_q, full0 + 8 * s, kx, lin.n + w.tile_q * (BN / 2));
          } else {
            tma_load_2d(dst + kTileP, &tmap_q, full0 + 8 * s, kx, w.tile_q * BN);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // fp32 accumulate, A and B of type T, both K-major, N = BN, M = 128
      constexpr uint32_t kFmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                 (static_cast<uint32_t>(kBM >> 4) << 24);
      uint32_t g = 0;
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
        const WorkItem w = work_item(item, grid);
        const uint32_t a = it & 1;
        const uint32_t use = static_cast<uint32_t>(it) >> 1;
        // the epilogue must have drained this accumulator buffer (its first use does not block)
        ok = mbar_wait(acc_empty0 + 8 * a, (use & 1u) ^ 1u, &abort_flag, 4, &g_gemm_status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + a * kAccCols;
        for (int kt = 0; kt < num_kt; ++kt, ++g) {
          const uint32_t s = g % static_cast<uint32_t>(stages);
          const uint32_t round = g / static_cast<uint32_t>(stages);
          ok = mbar_wait(full0 + 8 * s, round & 1u, &abort_flag, 2, &g_gemm_status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t pa = base + s * kStageBytes;
          const uint64_t pdesc = smem_desc_sw128(pa);
          const uint64_t qdesc = smem_desc_sw128(pa + kTileP);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            // 16 K-elements = 32 bytes further along the swizzled row: +2 in 16-byte units
            umma_f16(d_tmem, pdesc + 2 * kk, qdesc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(acc_full0 + 8 * a);  // arrives when every MMA issued so far has completed
      }
    }
  } else {
    const int quarter = warp & 3;  // the TMEM lanes a warp may read are fixed by warp id mod 4
    const int i = quarter * 32 + lane;  // row of D held by this thread
    int it = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
      const WorkItem w = work_item(item, grid);
      const uint32_t a = it & 1;
      const uint32_t use = static_cast<uint32_t>(it) >> 1;
      // the tcgen05.ld below is warp-collective: the warp leaves together or not at all
      const bool ready = mbar_wait(acc_full0 + 8 * a, use & 1u, &abort_flag, 3, &g_gemm_status);
      if (!__all_sync(0xffffffffu, ready)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kAccCols;
      if (!SWAP && EPI == EPI_SWIGLU) {
        const int64_t row = static_cast<int64_t>(w.tile_p) * kBM + i;
#pragma unroll 1
        for (int cc = 0; cc < BN / 2; cc += 32) {
          uint32_t up[32], gate[32];
          tmem_ld32(tacc + cc, up);
          tmem_ld32(tacc + BN / 2 + cc, gate);
          const int64_t j0 = static_cast<int64_t>(w.tile_q) * (BN / 2) + cc;
          if (row >= shape.m || j0 >= lin.n) continue;
          T* dst = static_cast<T*>(lin.y) + row * lin.n + j0;
          __align__(16) T out[32];
#pragma unroll
          for (int e = 0; e < 32; ++e)
            out[e] = swiglu_rounded<T>(rnd<T>(__uint_as_float(up[e])), rnd<T>(__uint_as_float(gate[e])));
          if (j0 + 32 <= lin.n && (lin.n & 7) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(out)[v];
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (j0 + e < lin.n) dst[e] = out[e];
          }
        }
      } else if (!SWAP && EPI == EPI_QKV) {
        const int64_t row = static_cast<int64_t>(w.tile_p) * kBM + i;
        const int hd = lin.head_dim;
        const int64_t nq = static_cast<int64_t>(lin.n_head) * hd, nk = static_cast<int64_t>(lin.n_kv) * hd;
        const int64_t b = row / lin.S, sq = row - b * lin.S;
        int64_t pos = 0, trow = 0;
        bool live = row < shape.m;
        if (live) {
          pos = load_pos(lin.input_pos, lin.pos_is_i64, sq);
          trow = lin.table_gathered ? sq : pos;
          live = pos >= 0 && pos < lin.smax && trow < lin.table_rows;
        }
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t r[32];
          tmem_ld32(tacc + cc, r);
          const int64_t n = static_cast<int64_t>(w.tile_q) * BN + cc;  // a 32-column chunk never straddles a head
          if (!live || n >= shape.n) continue;
          float f[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) f[e] = rnd<T>(__uint_as_float(r[e]));
          T* dst;
          if (n < nq + nk) {
            const int64_t nn = n < nq ? n : n - nq;
            const int e0 = static_cast<int>(nn % hd);
            const uint4* cs = reinterpret_cast<const uint4*>(static_cast<const T*>(lin.rope_table) +
                                                             (trow * (hd >> 1) + (e0 >> 1)) * 2);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float t[8];
              unpack8<T>(cs[v], t);  // (cos, sin) of 4 pairs
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float o0, o1;
                rope_pair(f[v * 8 + 2 * q], f[v * 8 + 2 * q + 1], t[2 * q], t[2 * q + 1], o0, o1);
                f[v * 8 + 2 * q] = o0;
                f[v * 8 + 2 * q + 1] = o1;
              }
            }
            dst = n < nq ? static_cast<T*>(lin.q_out) + row * nq + n
                         : static_cast<T*>(lin.k_cache) + ((b * lin.n_kv + nn / hd) * lin.smax + pos) * hd + e0;
          } else {
            const int64_t nn = n - nq - nk;
            dst = static_cast<T*>(lin.v_cache) + ((b * lin.n_kv + nn / hd) * lin.smax + pos) * hd + nn % hd;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float g8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) g8[e] = f[v * 8 + e];
            reinterpret_cast<uint4*>(dst)[v] = pack8<T>(g8);
          }
        }
      } else
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 32) {
        uint32_t r[32];
        const uint32_t taddr = tacc + cc;
        tmem_ld32(taddr, r);  // BN == 16: only the first 16 columns are valid (32 are allocated)
        constexpr int kValid = BN < 32 ? BN : 32;
        if (!SWAP) {
          const int64_t row = static_cast<int64_t>(w.tile_p) * kBM + i;
          const int64_t col0 = static_cast<int64_t>(w.tile_q) * BN + cc;
          if (row < shape.m) {
            T* dst = c + row * shape.n + col0;
            if (col0 + kValid <= shape.n) {
#pragma unroll
              for (int v = 0; v < kValid / 8; ++v) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
                reinterpret_cast<uint4*>(dst)[v] = pack8<T>(f);
              }
            } else {
#pragma unroll
              for (int e = 0; e < kValid; ++e)
                if (col0 + e < shape.n) dst[e] = Num<T>::from_f(__uint_as_float(r[e]));
            }
          }
        } else {
          const int64_t n = static_cast<int64_t>(w.tile_p) * kBM + i;
          const int64_t tok0 = static_cast<int64_t>(w.tile_q) * BN + cc;
          if (n < shape.n) {
#pragma unroll
            for (int e = 0; e < kValid; ++e)
              if (tok0 + e < shape.m) c[(tok0 + e) * shape.n + n] = Num<T>::from_f(__uint_as_float(r[e]));
          }
        }
      }
      // this thread's reads of the buffer are complete (tcgen05.wait::ld in tmem_ld32): hand it back
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(acc_empty0 + 8 * a);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that were already issued time to land before the CTA's shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

// 2-D row-major [rows, k] tensor of 16-bit elements, box = 64 elements x box_rows rows.
int make_tmap(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(LRI_ERR_CUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype == LRI_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LRI_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LRI_OK;
}

int sm_count() { return device_sm_count(); }

namespace {

template <typename T, int BN, bool SWAP, int EPI = EPI_PLAIN>
int launch_tile(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st,
                const LinearParams* lin = nullptr) {
  CUtensorMap tp, tq;
  const void* p_ptr = SWAP ? w : a;
  const void* q_ptr = SWAP ? a : w;
  const int64_t p_rows = SWAP ? n : m;
  const int64_t q_rows = SWAP ? m : n;
  int rc = make_tmap(&tp, dtype, p_ptr, p_rows, k, kBM);
  if (rc != LRI_OK) return rc;
  rc = make_tmap(&tq, dtype, q_ptr, q_rows, k, EPI == EPI_SWIGLU ? BN / 2 : BN);
  if (rc != LRI_OK) return rc;
  constexpr int kStageBytes = (kBM + BN) * kBK * 2;
  int stages = kSmemBudget / kStageBytes;
  stages = stages > 8 ? 8 : stages;
  const int smem = stages * kStageBytes + 1024;
  auto kern = gemm_tcgen05_kernel<T, BN, SWAP, EPI>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  LRI_ONCE_PER_DEVICE(attr_set, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024));
  const int64_t tiles_p = (p_rows + kBM - 1) / kBM;
  // SWIGLU: a Q tile is BN/2 outputs (their up rows and their gate rows)
  const int64_t tiles_q = EPI == EPI_SWIGLU ? (lin->n + BN / 2 - 1) / (BN / 2) : (q_rows + BN - 1) / BN;
  const int64_t items = tiles_p * tiles_q;
  if (items >= (1ll << 31)) return fail(LRI_ERR_UNSUPPORTED, "gemm: %lld output tiles", (long long)items);
  // panel of P tiles: about 16 MB of the P operand, between 4 and 16 tiles (LRI_GEMM_GROUP overrides)
  const int forced_group = option(OPT_GEMM_GROUP);
  int64_t group = (16ll << 20) / (static_cast<int64_t>(kBM) * k * 2);
  group = group < 4 ? 4 : (group > 16 ? 16 : group);
  if (forced_group > 0) group = forced_group;
  group = group > tiles_p ? tiles_p : group;
  GemmGrid grid{static_cast<int>(tiles_p), static_cast<int>(tiles_q), static_cast<int>(group)};
  GemmShape shape{static_cast<int>(m), n, k};
  // one persistent CTA per SM, minus the SMs left to a collective that runs beside the GEMM (the all-reduce
  // of the previous sublayer in the ladder schedule: a kernel that owns every SM would keep it waiting)
  int usable = sm_count() - option(OPT_GEMM_RESERVE_SMS);
  usable = usable < 1 ? 1 : usable;
  const int ctas = static_cast<int>(items < usable ? items : usable);
  LRI_CUDA(launch_pdl(kern, dim3(static_cast<unsigned>(ctas)), dim3(kGemmThreads), static_cast<size_t>(smem), st, tp, tq,
                      static_cast<T*>(c), shape, grid, stages, lin ? *lin : LinearParams{}));
  LRI_LAUNCH_CHECK("gemm_tcgen05_kernel");
  return LRI_OK;
}

template <typename T>
int launch_typed(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st) {
  if (m <= 16) return launch_tile<T, 16, true>(dtype, a, w, c, m, n, k, st);
  if (m <= 32) return launch_tile<T, 32, true>(dtype, a, w, c, m, n, k, st);
  if (m <= 64) return launch_tile<T, 64, true>(dtype, a, w, c, m, n, k, st);
  // prefill: pick the N tile that leaves fewer idle SMs in the last wave
  const int sms = sm_count();
  const int64_t mt = (m + kBM - 1) / kBM;
  const int64_t t256 = mt * ((n + 255) / 256), t128 = mt * ((n + 127) / 128);
  // measured: a 128x256 tile takes about 1.1x the time of a 128x128 tile (1141 vs 623 TFLOP/s)
  const int64_t cost256 = ((t256 + sms - 1) / sms) * 110, cost128 = ((t128 + sms - 1) / sms) * 100;
  if (cost256 <= cost128) return launch_tile<T, 256, false>(dtype, a, w, c, m, n, k, st);
  return launch_tile<T, 128, false>(dtype, a, w, c, m, n, k, st);
}

// prefill with the epilogue fused: the same tile choice, counted in output tiles
template <typename T, int EPI>
int launch_fused(int dtype, const LinearParams& p, int64_t m, cudaStream_t st) {
  const int n_rows = EPI == EPI_SWIGLU ? 2 * p.n : p.n;       // rows of the weight
  const int64_t mt = (m + kBM - 1) / kBM;
  const int w256 = EPI == EPI_SWIGLU ? 128 : 256, w128 = EPI == EPI_SWIGLU ? 64 : 128;  // outputs per Q tile
  const int64_t t256 = mt * ((p.n + w256 - 1) / w256), t128 = mt * ((p.n + w128 - 1) / w128);
  const int sms = sm_count();
  const int64_t cost256 = ((t256 + sms - 1) / sms) * 110, cost128 = ((t128 + sms - 1) / sms) * 100;
  if (cost256 <= cost128) return launch_tile<T, 256, false, EPI>(dtype, p.x, p.w, nullptr, m, n_rows, p.k, st, &p);
  return launch_tile<T, 128, false, EPI>(dtype, p.x, p.w, nullptr, m, n_rows, p.k, st, &p);
}

}  // namespace

bool gemm_tcgen05_supports(int64_t m, int n, int k);

// Prefill-sized projections (more than 64 token rows) with the SwiGLU or the RoPE + KV-cache
// epilogue applied from the accumulator: p.m token rows, p.n outputs (SWIGLU: I), all epilogue fields set.
bool gemm_tcgen05_fused_supports(int epi, const LinearParams& p, int64_t m) {
  if (m <= 64 || !gemm_tcgen05_supports(m, epi == EPI_SWIGLU ? 2 * p.n : p.n, p.k)) return false;
  if (epi == EPI_SWIGLU) return aligned16(p.y);
  if (epi == EPI_QKV) return p.head_dim % 32 == 0 && aligned16(p.rope_table);
  return false;
}

int gemm_tcgen05_fused_launch(int dtype, int epi, const LinearParams& p, int64_t m, cudaStream_t st) {
  if (!gemm_tcgen05_fused_supports(epi, p, m)) return fail(LRI_ERR_ARG, "gemm: fused epilogue not available for this shape");
  if (epi == EPI_SWIGLU)
    return dtype == LRI_BF16 ? launch_fused<__nv_bfloat16, EPI_SWIGLU>(dtype, p, m, st)
                             : launch_fused<__half, EPI_SWIGLU>(dtype, p, m, st);
  return dtype == LRI_BF16 ? launch_fused<__nv_bfloat16, EPI_QKV>(dtype, p, m, st)
                           : launch_fused<__half, EPI_QKV>(dtype, p, m, st);
}

bool gemm_tcgen05_supports(int64_t m, int n, int k) {
  return m >= 1 && m < (1ll << 31) && n >= 8 && n % 8 == 0 && k >= 8 && k % 8 == 0;
}

int gemm_tcgen05_launch(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st) {
  return dtype == LRI_BF16 ? launch_typed<__nv_bfloat16>(dtype, a, w, c, m, n, k, st)
                           : launch_typed<__half>(dtype, a, w, c, m, n, k, st);
}

int gemm_tcgen05_status_read_and_clear(int* status_out) {
  int v = 0;
  LRI_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    LRI_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  }
  *status_out = v;
  return LRI_OK;
}

}  // namespace lri
