// F4 on the fifth-generation tensor cores: causal GQA prefill attention with both products issued as
// tcgen05.mma and the accumulators in tensor memory.
//
// A CTA owns 128 consecutive queries of one (sequence, query head) and walks the visible keys in
// tiles of 64.  Per tile:
//   S = Q K^T      tcgen05.mma 128 x 64 x head_dim, Q and K tiles in shared memory (K-major, 128-byte
//                  swizzle, fetched by plain TMA loads), S in one of two TMEM buffers (64 fp32 columns)
//   softmax        4 warps, thread i owns query row i: tcgen05.ld of its 64 scores (a row lives in one
//                  TMEM lane, so max and sum need no shuffles), scale, causal mask, exp2 against the
//                  running reference maximum (ex2.approx, scale folded into one FMA), P rounded to the storage type and written back over S
//                  with tcgen05.st (32 columns of packed pairs)
//   O += P V       tcgen05.mma 128 x head_dim x 64 with P read from TMEM as the A operand and the V tile
//                  from shared memory as an MN-major B operand (V rows are keys, head_dim contiguous:
//                  exactly what the cache holds, no transpose), O in TMEM (head_dim fp32 columns)
// The output is rescaled lazily: the reference maximum of a row only moves (and O, l are multiplied by
// the correction, a TMEM load / store round trip) when the new maximum exceeds it by more than 2^8;
// until then P stays below 256, exact enough in the storage type.  One elected thread issues TMA, one
// issues the MMAs (S of tile j+1 is issued before P of tile j is awaited, so the tensor pipe works while
// the softmax warps do), K/V tiles go through a two-stage ring.  96 KB of shared memory and 256 TMEM
// columns per CTA let two CTAs share an SM: the softmax of one overlaps the MMAs of the other.
// Every mbarrier wait is bounded; on expiry a status word is set, TMEM is freed and the kernel returns.
//
// Rows of the KV cache past the newest position must hold finite values (they are multiplied by
// P = 0); the cache module zero-initialises them, as the reference's does (gpt_fast/utils.py:47-48).
#include "tcgen05.cuh"

namespace lri {
namespace {

using namespace tc;

constexpr int kFaM = 128;       // queries per CTA = rows of the UMMA
constexpr int kFaN = 64;        // keys per tile
constexpr int kFaStages = 2;
constexpr int kFaThreads = 192;  // TMA warp, MMA warp, 4 softmax warps
constexpr float kFaRescaleLog2 = 8.0f;

__device__ int g_attn_tc_status = 0;

struct FaParams {
  void* out;  // [B, S, n_head * HD]
  const void* input_pos;
  int pos_is_i64;
  int S, n_head, n_kv;
  int64_t smax;
  float scale_log2;
};

// MN-major operand tile in the 128-byte swizzle: 64 contiguous MN elements per 128-byte row, 8 K rows
// per 1024-byte atom; lbo = bytes between atoms along MN, sbo = bytes between atoms along K.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <typename T, int HD>
__global__ void __launch_bounds__(kFaThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  constexpr int kChunks = HD / 64;                        // 64-element (128-byte) column chunks of a row
  constexpr uint32_t kQChunkBytes = kFaM * 128;            // [128 rows][128 B]
  constexpr uint32_t kKvChunkBytes = kFaN * 128;           // [64 rows][128 B]
  constexpr uint32_t kQBytes = kChunks * kQChunkBytes;
  constexpr uint32_t kTileBytes = kChunks * kKvChunkBytes;  // one K or V tile
  constexpr uint32_t kStageBytes = 2 * kTileBytes;
  constexpr uint32_t kSCols = kFaN;                        // fp32 columns of one S buffer
  constexpr uint32_t kOCol = 2 * kSCols;                   // first column of O
  constexpr uint32_t kTmemCols = 256;                      // 2 * 64 + HD <= 256
  static_assert(HD == 64 || HD == 128, "head_dim 64 and 128 are built");

  extern __shared__ uint8_t fa_smem_raw[];
  const uint32_t base = (smem_u32(fa_smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + kQBytes;
  __shared__ uint64_t bars[1 + 2 * kFaStages + 6];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;  // long (late) tiles first
  const int q0 = q_tile * kFaM;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.n_head / p.n_kv);

  const uint32_t q_full = smem_u32(&bars[0]);
  const uint32_t kv_full0 = smem_u32(&bars[1]);
  const uint32_t kv_empty0 = smem_u32(&bars[1 + kFaStages]);
  const uint32_t s_full0 = smem_u32(&bars[1 + 2 * kFaStages]);      // MMA -> softmax, per S buffer
  const uint32_t p_full0 = smem_u32(&bars[1 + 2 * kFaStages + 2]);  // softmax -> MMA, per S buffer
  const uint32_t o_done0 = smem_u32(&bars[1 + 2 * kFaStages + 4]);  // P V of a tile complete, per parity of the tile

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kFaStages; ++s) {
      mbar_init(kv_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full0 + 8 * i, 1);
      mbar_init(p_full0 + 8 * i, 128);  // every softmax thread arrives
      mbar_init(o_done0 + 8 * i, 1);
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

  int64_t pos0 = load_pos(p.input_pos, p.pos_is_i64, 0);
  pos0 = pos0 < 0 ? 0 : pos0;
  const int q_end = (q0 + kFaM < p.S) ? q0 + kFaM : p.S;
  int64_t kv_end = pos0 + q_end;  // keys 0 .. pos0 + q_end - 1 are visible to the last row of the tile
  kv_end = kv_end > p.smax ? p.smax : kv_end;
  const int n_tiles = static_cast<int>((kv_end + kFaN - 1) / kFaN);  // >= 1
  const int kv_row0_hi = static_cast<int>((static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax);  // row of key 0 in the [rows, HD] view

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(q_smem + c * kQChunkBytes, &tmap_q, q_full, head * HD + c * 64, b * p.S + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t s = j % kFaStages, round = j / kFaStages;
        if (!mbar_wait(kv_empty0 + 8 * s, (round & 1u) ^ 1u, &abort_flag, 1, &g_attn_tc_status)) break;
        mbar_expect_tx(kv_full0 + 8 * s, kStageBytes);
        const uint32_t dst = kv_smem + s * kStageBytes;
        const int row = kv_row0_hi + j * kFaN;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          tma_load_2d(dst + c * kKvChunkBytes, &tmap_k, kv_full0 + 8 * s, c * 64, row);
          tma_load_2d(dst + kTileBytes + c * kKvChunkBytes, &tmap_v, kv_full0 + 8 * s, c * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      // S = Q K^T: both operands K-major, N = 64
      constexpr uint32_t idesc_qk = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (static_cast<uint32_t>(kFaN >> 3) << 17) |
                                    (static_cast<uint32_t>(kFaM >> 4) << 24);
      // O += P V: A from TMEM (K-major), B MN-major (bit 16), N = HD
      constexpr uint32_t idesc_pv = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (1u << 16) |
                                    (static_cast<uint32_t>(HD >> 3) << 17) | (static_cast<uint32_t>(kFaM >> 4) << 24);
      constexpr uint32_t v_lbo = kKvChunkBytes;  // between the 64-column chunks of head_dim
      constexpr uint32_t v_sbo = 1024u;           // between groups of 8 keys
      bool ok = mbar_wait(q_full, 0, &abort_flag, 2, &g_attn_tc_status);

      auto issue_qk = [&](int j) {
        const uint32_t s = j % kFaStages, round = j / kFaStages;
        if (!mbar_wait(kv_full0 + 8 * s, round & 1u, &abort_flag, 3, &g_attn_tc_status)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_smem = kv_smem + s * kStageBytes;
        const uint32_t d = tmem_base + static_cast<uint32_t>(j & 1) * kSCols;
#pragma unroll
        for (int kk = 0; kk < HD / kUmmaK; ++kk) {
          const uint64_t qd = smem_desc_sw128(q_smem + (kk / 4) * kQChunkBytes) + 2 * (kk % 4);
          const uint64_t kd = smem_desc_sw128(k_smem + (kk / 4) * kKvChunkBytes) + 2 * (kk % 4);
          umma_f16(d, qd, kd, idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full0 + 8 * (j & 1));
        return true;
      };
      auto issue_pv = [&](int j) {
        const uint32_t s = j % kFaStages;
        if (!mbar_wait(p_full0 + 8 * (j & 1), (static_cast<uint32_t>(j) >> 1) & 1u, &abort_flag, 4, &g_attn_tc_status))
          return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_smem = kv_smem + s * kStageBytes + kTileBytes;
        const uint32_t pa = tmem_base + static_cast<uint32_t>(j & 1) * kSCols;  // P over the first 32 columns of S
#pragma unroll
        for (int kk = 0; kk < kFaN / kUmmaK; ++kk) {
          // 16 keys further: 16 rows of 128 bytes in the V tile, 8 packed columns in P
          const uint64_t vd = smem_desc_mn_sw128(v_smem + kk * 2048u, v_lbo, v_sbo);
          umma_ts_f16(tmem_base + kOCol, pa + kk * 8, vd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty0 + 8 * s);      // K and V of this stage have been read
        umma_commit(o_done0 + 8 * (j & 1));  // O holds tiles 0..j
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (ok) ok = issue_pv(j);
      }
    }
  } else {
    const int quarter = warp & 3;       // TMEM lanes a warp may touch: 32 * (warp id mod 4)
    const int i = quarter * 32 + lane;  // query row of this thread
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int64_t qpos = pos0 + q0 + i;
    float m_ref = -INFINITY, l = 0.f;
    bool alive = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t sb = static_cast<uint32_t>(j & 1);
      const bool ready = mbar_wait(s_full0 + 8 * sb, (static_cast<uint32_t>(j) >> 1) & 1u, &abort_flag, 5, &g_attn_tc_status);
      if (!__all_sync(0xffffffffu, ready)) {
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t s_addr = tmem_base + lane_off + sb * kSCols;
      uint32_t r0[32], r1[32];
      tmem_ld32_issue(s_addr, r0);
      tmem_ld32_issue(s_addr + 32, r1);
      tmem_wait_ld();
      // raw scores; the softmax scale is folded into the exponent's multiply-add below
      float sv[kFaN];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        sv[e] = __uint_as_float(r0[e]);
        sv[32 + e] = __uint_as_float(r1[e]);
      }
      const int64_t key0 = static_cast<int64_t>(j) * kFaN;
      // tiles that reach past the first row's position or past the end of the visible keys need the mask
      if (key0 + kFaN - 1 > pos0 + q0 || key0 + kFaN > kv_end) {
#pragma unroll
        for (int e = 0; e < kFaN; ++e) {
          const int64_t kj = key0 + e;
          if (kj > qpos || kj >= kv_end) sv[e] = -INFINITY;
        }
      }
      // four independent chains: a 64-long dependent max (or sum) would cost 64 instruction latencies
      float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int e = 4; e < kFaN; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], sv[e]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;  // in log2 units
      if (j == 0) {
        m_ref = mx;  // tile 0 holds key 0, which every query sees: finite
      } else {
        const bool need = mx > m_ref + kFaRescaleLog2;
        if (__any_sync(0xffffffffu, need)) {
          // O holds tiles 0..j-1 once the P V product of tile j-1 has completed
          const uint32_t ob = static_cast<uint32_t>((j - 1) & 1);
          const bool done = mbar_wait(o_done0 + 8 * ob, (static_cast<uint32_t>(j - 1) >> 1) & 1u, &abort_flag, 6,
                                      &g_attn_tc_status);
          if (!__all_sync(0xffffffffu, done)) {
            alive = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const float corr = need ? exp2f(m_ref - mx) : 1.0f;
#pragma unroll 1
          for (int cc = 0; cc < HD; cc += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_off + kOCol + cc, o);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(tmem_base + lane_off + kOCol + cc, o);
          }
          tmem_wait_st();
          l *= corr;
          if (need) m_ref = mx;
        }
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      uint32_t pk[32];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        // (evaluating a share of the exponentials as a polynomial on the FMA pipe, to unload the special-function
        // unit, was measured slower on B200: 89 and 96 us against 84 us with a quarter and a half of them moved)
        const float p0 = exp2_approx(fmaf(sv[2 * e], p.scale_log2, neg_m));
        const float p1 = exp2_approx(fmaf(sv[2 * e + 1], p.scale_log2, neg_m));
        sum4[e & 3] += p0 + p1;
        pk[e] = pack2<T>(p0, p1);  // key 2e in the low half of column e
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l += sum;
      tmem_st32(s_addr, pk);  // P over the first 32 columns of this S buffer
      tmem_wait_st();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_full0 + 8 * sb);
    }
    if (alive) {
      const uint32_t ob = static_cast<uint32_t>((n_tiles - 1) & 1);
      const bool done = mbar_wait(o_done0 + 8 * ob, (static_cast<uint32_t>(n_tiles - 1) >> 1) & 1u, &abort_flag, 7,
                                  &g_attn_tc_status);
      if (__all_sync(0xffffffffu, done)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        const int s_idx = q0 + i;
        T* dst = static_cast<T*>(p.out) + ((static_cast<int64_t>(b) * p.S + s_idx) * p.n_head + head) * HD;
#pragma unroll 1
        for (int cc = 0; cc < HD; cc += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_off + kOCol + cc, o);
          if (s_idx < p.S) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[v * 8 + e]) * inv;
              reinterpret_cast<uint4*>(dst + cc)[v] = pack8<T>(f);
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that were already issued time to land before the CTA's shared memory is released
    for (int w = 0; w < 2000; ++w) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename T, int HD>
int launch_fa(int dtype, const void* q, const void* k_cache, const void* v_cache, const FaParams& p, int B,
              cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  int rc = make_tmap(&tq, dtype, q, static_cast<int64_t>(B) * p.S, static_cast<int64_t>(p.n_head) * HD, kFaM);
  if (rc != LRI_OK) return rc;
  const int64_t kv_rows = static_cast<int64_t>(B) * p.n_kv * p.smax;
  rc = make_tmap(&tk, dtype, k_cache, kv_rows, HD, kFaN);
  if (rc != LRI_OK) return rc;
  rc = make_tmap(&tv, dtype, v_cache, kv_rows, HD, kFaN);
  if (rc != LRI_OK) return rc;
  constexpr int kChunks = HD / 64;
  constexpr int smem = kChunks * kFaM * 128 + kFaStages * 2 * kChunks * kFaN * 128 + 1024;
  auto kern = attn_prefill_tc_kernel<T, HD>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  LRI_ONCE_PER_DEVICE(attr_set, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.S + kFaM - 1) / kFaM, p.n_head, B);
  kern<<<grid, kFaThreads, smem, st>>>(tq, tk, tv, p);
  LRI_LAUNCH_CHECK("attn_prefill_tc_kernel");
  return LRI_OK;
}

}  // namespace

// Shapes the tensor-memory kernel takes: the row coordinates of its tensor maps are 32-bit.
bool attn_prefill_tc_supports(int B, int S, int n_head, int n_kv, int head_dim, int64_t smax) {
  if (head_dim != 64 && head_dim != 128) return false;
  const int64_t kv_rows = static_cast<int64_t>(B) * n_kv * smax + kFaN;
  const int64_t q_rows = static_cast<int64_t>(B) * S + kFaM;
  return kv_rows < (1ll << 31) && q_rows < (1ll << 31) && static_cast<int64_t>(n_head) * head_dim < (1ll << 31);
}

int attn_prefill_tc_launch(int dtype, const void* q, const void* k_cache, const void* v_cache, const void* input_pos,
                           int pos_is_i64, void* out, int B, int S, int n_head, int n_kv, int head_dim, int64_t smax,
                           float scale_log2, cudaStream_t st) {
  FaParams p{};
  p.out = out, p.input_pos = input_pos, p.pos_is_i64 = pos_is_i64;
  p.S = S, p.n_head = n_head, p.n_kv = n_kv, p.smax = smax, p.scale_log2 = scale_log2;
  if (dtype == LRI_BF16)
    return head_dim == 128 ? launch_fa<__nv_bfloat16, 128>(dtype, q, k_cache, v_cache, p, B, st)
                           : launch_fa<__nv_bfloat16, 64>(dtype, q, k_cache, v_cache, p, B, st);
  return head_dim == 128 ? launch_fa<__half, 128>(dtype, q, k_cache, v_cache, p, B, st)
                         : launch_fa<__half, 64>(dtype, q, k_cache, v_cache, p, B, st);
}

int attn_prefill_tc_status_read_and_clear(int* status_out) {
  int v = 0;
  LRI_CUDA(cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    LRI_CUDA(cudaMemcpyToSymbol(g_attn_tc_status, &zero, sizeof(int)));
  }
  *status_out = v;
  return LRI_OK;
}

}  // namespace lri
