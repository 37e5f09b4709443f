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
#include <cuda.h>

#include <cstdlib>

#include <type_traits>

#include "linear.cuh"

namespace lri {
namespace {

constexpr int kBM = 128;            // rows of the UMMA M operand
constexpr int kBK = 64;             // K elements per stage (128 bytes)
constexpr int kUmmaK = 16;          // K elements per tcgen05.mma
constexpr int kGemmThreads = 192;   // 6 warps
constexpr uint32_t kPollBudget = 1u << 22;
constexpr int kSmemBudget = 200 * 1024;

__device__ int g_gemm_status = 0;  // 0 ok, else the code of the first wait that gave up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory; once any wait has given up, every later
// wait returns at once so the CTA drains quickly.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  for (uint32_t i = 0; i < kPollBudget; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_gemm_status, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// K-major operand tile in the 128-byte swizzle: rows 128 bytes apart, 8-row groups 1024 bytes
// apart (stride byte offset), leading byte offset unused for swizzled K-major layouts (1),
// descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct GemmShape {
  int m, n, k;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// One unit of work of a persistent CTA: an output tile and a slice of K.
struct WorkItem {
  int tile_p, tile_q, z, kt_begin, num_kt;
};
struct GemmGrid {
  int tiles_p, tiles_q, splits;
};
__device__ __forceinline__ WorkItem work_item(int item, const GemmGrid& g, int total_kt) {
  WorkItem w;
  const int per_slice = g.tiles_p * g.tiles_q;
  w.z = item / per_slice;
  const int rem = item - w.z * per_slice;
  w.tile_p = rem / g.tiles_q;  // neighbouring CTAs share the 128-row operand tile and stream different Q tiles
  w.tile_q = rem - w.tile_p * g.tiles_q;
  // slice z owns a contiguous range of K tiles, never empty (the host keeps splits <= number of K tiles)
  w.kt_begin = static_cast<int>(static_cast<int64_t>(total_kt) * w.z / g.splits);
  w.num_kt = static_cast<int>(static_cast<int64_t>(total_kt) * (w.z + 1) / g.splits) - w.kt_begin;
  return w;
}

// P = operand with 128 rows per tile, Q = operand with BN rows per tile.
// SWAP == false: P = A (tokens), Q = W;  D[i, j] -> C[tile_p*128 + i, tile_q*BN + j]
// SWAP == true : P = W,          Q = A;  D[i, j] -> C[tile_q*BN + j, tile_p*128 + i]
// With `partial` set (SWAP only) slice z of K writes fp32 partial[z][token][n] instead of C.
//
// The kernel is persistent: CTA b works through items b, b + gridDim.x, ...  The shared-memory
// ring keeps running across items (the producer is already fetching the next item's operands
// while the last MMAs of the current one execute) and the accumulator is double-buffered in
// TMEM, so the epilogue of item i overlaps the main loop of item i + 1.
template <typename T, int BN, bool SWAP>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                    T* __restrict__ c, float* __restrict__ partial, GemmShape shape, GemmGrid grid, int stages,
                    int rotate_k) {
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
  const int total_kt = (shape.k + kBK - 1) / kBK;
  const int items = grid.tiles_p * grid.tiles_q * grid.splits;

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
        const WorkItem w = work_item(item, grid, total_kt);
        const int rot = rotate_k ? item % w.num_kt : 0;
        for (int kt = 0; kt < w.num_kt; ++kt, ++g) {
          const uint32_t s = g % static_cast<uint32_t>(stages);
          const uint32_t round = g / static_cast<uint32_t>(stages);
          // a fresh barrier passes a wait on parity 1, so the first round does not block
          ok = mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, &abort_flag, 1);
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          const uint32_t dst = base + s * kStageBytes;
          // optional: items walk their K range from different starting points (the sum does not
          // care about the order)
          int kr = kt + rot;
          kr = kr >= w.num_kt ? kr - w.num_kt : kr;
          const int kx = (w.kt_begin + kr) * kBK;
          tma_load_2d(dst, &tmap_p, full0 + 8 * s, kx, w.tile_p * kBM);
          tma_load_2d(dst + kTileP, &tmap_q, full0 + 8 * s, kx, w.tile_q * BN);
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
        const WorkItem w = work_item(item, grid, total_kt);
        const uint32_t a = it & 1;
        const uint32_t use = static_cast<uint32_t>(it) >> 1;
        // the epilogue must have drained this accumulator buffer (its first use does not block)
        ok = mbar_wait(acc_empty0 + 8 * a, (use & 1u) ^ 1u, &abort_flag, 4);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + a * kAccCols;
        for (int kt = 0; kt < w.num_kt; ++kt, ++g) {
          const uint32_t s = g % static_cast<uint32_t>(stages);
          const uint32_t round = g / static_cast<uint32_t>(stages);
          ok = mbar_wait(full0 + 8 * s, round & 1u, &abort_flag, 2);
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
      const WorkItem w = work_item(item, grid, total_kt);
      const uint32_t a = it & 1;
      const uint32_t use = static_cast<uint32_t>(it) >> 1;
      if (!mbar_wait(acc_full0 + 8 * a, use & 1u, &abort_flag, 3)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kAccCols + cc;
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
            if (partial != nullptr) {
              float* dst = partial + static_cast<int64_t>(w.z) * shape.m * shape.n + n;
#pragma unroll
              for (int e = 0; e < kValid; ++e)
                if (tok0 + e < shape.m) dst[(tok0 + e) * shape.n] = __uint_as_float(r[e]);
            } else {
#pragma unroll
              for (int e = 0; e < kValid; ++e)
                if (tok0 + e < shape.m) c[(tok0 + e) * shape.n + n] = Num<T>::from_f(__uint_as_float(r[e]));
            }
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

// LRI_GEMM_ROTATE_K=1 makes work items start their walk over K at different tiles (tuning knob;
// measured neutral to slightly slower on B200, so off by default)
int rotate_k() {
  static const int on = [] {
    const char* e = getenv("LRI_GEMM_ROTATE_K");
    return (e && atoi(e) == 1) ? 1 : 0;
  }();
  return on;
}

int sm_count() {
  static const int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    return v;
  }();
  return n;
}

template <typename T, int BN, bool SWAP>
int launch_tile(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st,
                float* partial = nullptr, int splits = 1) {
  CUtensorMap tp, tq;
  const void* p_ptr = SWAP ? w : a;
  const void* q_ptr = SWAP ? a : w;
  const int64_t p_rows = SWAP ? n : m;
  const int64_t q_rows = SWAP ? m : n;
  int rc = make_tmap(&tp, dtype, p_ptr, p_rows, k, kBM);
  if (rc != LRI_OK) return rc;
  rc = make_tmap(&tq, dtype, q_ptr, q_rows, k, BN);
  if (rc != LRI_OK) return rc;
  constexpr int kStageBytes = (kBM + BN) * kBK * 2;
  int stages = kSmemBudget / kStageBytes;
  stages = stages > 8 ? 8 : stages;
  const int smem = stages * kStageBytes + 1024;
  auto kern = gemm_tcgen05_kernel<T, BN, SWAP>;
  static bool attr_set = false;  // per template instantiation
  if (!attr_set) {
    LRI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024));
    attr_set = true;
  }
  const int total_kt = (k + kBK - 1) / kBK;
  splits = splits < 1 ? 1 : (splits > total_kt ? total_kt : splits);
  if (!SWAP || partial == nullptr) splits = 1;
  const int64_t tiles_p = (p_rows + kBM - 1) / kBM, tiles_q = (q_rows + BN - 1) / BN;
  const int64_t items = tiles_p * tiles_q * splits;
  if (items >= (1ll << 31)) return fail(LRI_ERR_UNSUPPORTED, "gemm: %lld output tiles", (long long)items);
  GemmGrid grid{static_cast<int>(tiles_p), static_cast<int>(tiles_q), splits};
  GemmShape shape{static_cast<int>(m), n, k};
  const int ctas = static_cast<int>(items < sm_count() ? items : sm_count());
  LRI_CUDA(launch_pdl(kern, dim3(static_cast<unsigned>(ctas)), dim3(kGemmThreads), static_cast<size_t>(smem), st, tp, tq,
                      static_cast<T*>(c), partial, shape, grid, stages, rotate_k()));
  LRI_LAUNCH_CHECK("gemm_tcgen05_kernel");
  return LRI_OK;
}

template <typename T>
int launch_typed(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st,
                 float* partial = nullptr, int splits = 1) {
  if (m <= 16) return launch_tile<T, 16, true>(dtype, a, w, c, m, n, k, st, partial, splits);
  if (m <= 32) return launch_tile<T, 32, true>(dtype, a, w, c, m, n, k, st, partial, splits);
  if (m <= 64) return launch_tile<T, 64, true>(dtype, a, w, c, m, n, k, st, partial, splits);
  // prefill: pick the N tile that leaves fewer idle SMs in the last wave
  int sms = 148;
  const int64_t mt = (m + kBM - 1) / kBM;
  const int64_t t256 = mt * ((n + 255) / 256), t128 = mt * ((n + 127) / 128);
  // measured: a 128x256 tile takes about 1.1x the time of a 128x128 tile (1141 vs 623 TFLOP/s)
  const int64_t cost256 = ((t256 + sms - 1) / sms) * 110, cost128 = ((t128 + sms - 1) / sms) * 100;
  if (cost256 <= cost128) return launch_tile<T, 256, false>(dtype, a, w, c, m, n, k, st);
  return launch_tile<T, 128, false>(dtype, a, w, c, m, n, k, st);
}

}  // namespace

bool gemm_tcgen05_supports(int64_t m, int n, int k) {
  return m >= 1 && m < (1ll << 31) && n >= 8 && n % 8 == 0 && k >= 8 && k % 8 == 0;
}

int gemm_tcgen05_launch(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st) {
  return dtype == LRI_BF16 ? launch_typed<__nv_bfloat16>(dtype, a, w, c, m, n, k, st)
                           : launch_typed<__half>(dtype, a, w, c, m, n, k, st);
}

// Small-M (<= 64 token rows) weight-streaming form: W is the 128-row operand, K is cut into
// `splits` slices, slice z writes fp32 partial[z][m][n]; the caller sums the slices in its epilogue.
int gemm_tcgen05_splitk_launch(int dtype, const void* a, const void* w, float* partial, int64_t m, int n, int k,
                               int splits, cudaStream_t st) {
  if (m > 64 || partial == nullptr) return fail(LRI_ERR_ARG, "gemm split-K: m=%lld must be <= 64", (long long)m);
  return dtype == LRI_BF16 ? launch_typed<__nv_bfloat16>(dtype, a, w, nullptr, m, n, k, st, partial, splits)
                           : launch_typed<__half>(dtype, a, w, nullptr, m, n, k, st, partial, splits);
}

// Number of K slices for the small-M form: fill the 148 SMs (one CTA each) with as little idle
// tail as possible while every slice keeps at least 8 K tiles to amortise the pipeline fill.
int gemm_tcgen05_choose_splits(int n, int k) {
  const int64_t tiles = (n + kBM - 1) / kBM;
  const int total_kt = (k + kBK - 1) / kBK;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= kMaxSplitK; ++s) {
    if (s > 1 && total_kt / s < 8) break;
    const int64_t ctas = tiles * s;
    const int64_t waves = (ctas + 147) / 148;
    // idle tail of the last wave, plus a small charge per slice for the fp32 partials
    const double eff = static_cast<double>(ctas) / (148.0 * waves) - 0.01 * (s - 1);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
  }
  return best;
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
