// F3: GQA decode attention split over the sequence (one query token per sequence), and
// F4: causal GQA prefill attention (flash-attention style, tensor-core tiles via mma.sync).
//
// Both read the dense KV cache [B_max, n_kv, smax, head_dim] and the current position from
// device memory, use fp32 softmax state, and round the output once to the storage type.
#include <cstdlib>

#include "common.cuh"

namespace lri {
// cluster form of the decode kernel (attention_cluster.cu)
bool attn_decode_cluster_supports(int num_splits);
int attn_decode_cluster_head_tile(int B, int n_kv, int g);
int attn_decode_cluster_launch(int dtype, const void* q, const void* k_cache, const void* v_cache,
                               const void* input_pos, int pos_is_i64, void* out, int B, int n_head, int n_kv,
                               int head_dim, int64_t smax, int num_splits, float scale_log2, cudaStream_t st);
// tcgen05 / TMEM form of the prefill kernel (attention_tc.cu)
bool attn_prefill_tc_supports(int B, int S, int n_head, int n_kv, int head_dim, int64_t smax);
int attn_prefill_tc_launch(int dtype, const void* q, const void* k_cache, const void* v_cache, const void* input_pos,
                           int pos_is_i64, void* out, int B, int S, int n_head, int n_kv, int head_dim, int64_t smax,
                           float scale_log2, cudaStream_t st);
namespace {

constexpr float kLog2e = 1.4426950408889634f;

// =====================================================================================================
// F3 decode
// =====================================================================================================
constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecUnroll = 4;  // positions per row group and loop iteration
constexpr int kMaxSplits = 64;

struct DecodeParams {
  const void* q;        // [B, n_head, HD]
  const void* k_cache;  // [B_max, n_kv, smax, HD]
  const void* v_cache;
  const void* input_pos;
  int pos_is_i64;
  void* out;  // [B, n_head * HD]
  int n_head, n_kv;
  int64_t smax;
  int num_splits;
  float scale_log2;  // log2(e) / sqrt(HD)
  unsigned int* counters;  // [B * n_head] (one per (batch, head tile) is used)
  float* part_ml;          // [B, n_head, num_splits, 2]
  float* part_o;           // [B, n_head, num_splits, HD]
};

// Grid (num_splits, n_kv * tiles_per_kv, B); a CTA handles GT query heads that share one kv head
// over one range of positions.  LPR lanes hold one cache row (8 elements each); the 32 / LPR row
// groups of a warp and the warps of the CTA take interleaved positions.
template <typename T, int HD, int GT>
__global__ void __launch_bounds__(kDecThreads) attn_decode_kernel(const DecodeParams p) {
  constexpr int LPR = HD / 8;        // lanes per row
  constexpr int RPW = 32 / LPR;      // row groups per warp
  constexpr int NRG = RPW * kDecWarps;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sl = lane % LPR;         // which 8 elements of the row
  const int rg = warp * RPW + lane / LPR;  // row group: takes positions p0 + rg, p0 + rg + NRG, ...
  const int split = blockIdx.x;
  const int g = p.n_head / p.n_kv;
  const int tiles_per_kv = g / GT;
  const int kvh = blockIdx.y / tiles_per_kv;
  const int head0 = kvh * g + (blockIdx.y % tiles_per_kv) * GT;
  const int b = blockIdx.z;

  pdl_launch_dependents();
  pdl_wait();  // q and the newest cache row were written by the preceding kernel
  int64_t ctx = load_pos(p.input_pos, p.pos_is_i64, 0) + 1;
  ctx = ctx < 0 ? 0 : (ctx > p.smax ? p.smax : ctx);
  const int64_t chunk = (ctx + p.num_splits - 1) / p.num_splits;
  const int64_t p0 = split * chunk;
  const int64_t p1 = (p0 + chunk < ctx) ? p0 + chunk : ctx;

  const T* kbase = static_cast<const T*>(p.k_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;
  const T* vbase = static_cast<const T*>(p.v_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;

  float qf[GT][8];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    const T* qp = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + sl * 8;
    unpack8<T>(*reinterpret_cast<const uint4*>(qp), qf[h]);
#pragma unroll
    for (int e = 0; e < 8; ++e) qf[h][e] *= p.scale_log2;
  }

  float m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
  }

  // The trip count depends on the warp only: every lane of a warp runs the same iterations, so the
  // full-mask shuffles below are executed by all 32 lanes (row groups past the end compute on a
  // clamped row and are masked out).
  for (int64_t jb = p0 + warp * RPW; jb < p1; jb += static_cast<int64_t>(NRG) * kDecUnroll) {
    uint4 kv[kDecUnroll], vv[kDecUnroll];
    bool valid[kDecUnroll];
#pragma unroll
    for (int t = 0; t < kDecUnroll; ++t) {
      const int64_t j = jb + lane / LPR + static_cast<int64_t>(t) * NRG;
      valid[t] = j < p1;
      const int64_t jc = valid[t] ? j : p1 - 1;
      kv[t] = ld_stream16(kbase + jc * HD);
      vv[t] = ld_stream16(vbase + jc * HD);
    }
    float s[kDecUnroll][GT];
#pragma unroll
    for (int t = 0; t < kDecUnroll; ++t) {
      float kf[8];
      unpack8<T>(kv[t], kf);
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qf[h][e], kf[e], d);
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[t][h] = valid[t] ? d : -INFINITY;
      }
    }
#pragma unroll
    for (int h = 0; h < GT; ++h) {
      float mx = s[0][h];
#pragma unroll
      for (int t = 1; t < kDecUnroll; ++t) mx = fmaxf(mx, s[t][h]);
      const float m_new = fmaxf(m[h], mx);
      // a row group that has seen no valid position yet keeps m = -inf; exponentials are then
      // taken against 0 so that they evaluate to 0 instead of NaN
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m[h] - m_use);
      l[h] *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
      m[h] = m_new;
#pragma unroll
      for (int t = 0; t < kDecUnroll; ++t) s[t][h] = exp2f(s[t][h] - m_use);
    }
#pragma unroll
    for (int t = 0; t < kDecUnroll; ++t) {
      float vf[8];
      unpack8<T>(vv[t], vf);
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        l[h] += s[t][h];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(s[t][h], vf[e], acc[h][e]);
      }
    }
  }

  // ---- merge the row groups of the CTA ---------------------------------------------------------
  __shared__ float sm_m[NRG][GT];
  __shared__ float sm_l[NRG][GT];
  __shared__ float sm_o[NRG][GT][HD];
  __shared__ unsigned int ticket_s;
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    if (sl == 0) {
      sm_m[rg][h] = m[h];
      sm_l[rg][h] = l[h];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sm_o[rg][h][sl * 8 + e] = acc[h][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * HD; idx += kDecThreads) {
    const int h = idx / HD, e = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < NRG; ++r) mm = fmaxf(mm, sm_m[r][h]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int r = 0; r < NRG; ++r) {
        const float w = exp2f(sm_m[r][h] - mm);  // 0 for groups that saw no position
        ll += sm_l[r][h] * w;
        oo += sm_o[r][h][e] * w;
      }
    }
    const int64_t slot = (static_cast<int64_t>(b) * p.n_head + head0 + h) * p.num_splits + split;
    p.part_o[slot * HD + e] = oo;
    if (e == 0) {
      p.part_ml[slot * 2] = mm;
      p.part_ml[slot * 2 + 1] = ll;
    }
  }

  // ---- the last CTA of this (batch, head tile) merges the splits ---------------------------------
  __threadfence();
  __syncthreads();
  unsigned int* counter = p.counters + static_cast<int64_t>(b) * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) ticket_s = atomicAdd(counter, 1u);
  __syncthreads();
  if (ticket_s != static_cast<unsigned int>(p.num_splits - 1)) return;
  __threadfence();
  // Weights of the splits: one warp per head, lanes over splits, so the (m, l) pairs arrive in one
  // round trip to L2 instead of one per split.  sm_o is free again and holds the weights.
  float* wgt = &sm_o[0][0][0];        // [GT][kMaxSplits]
  float* inv = wgt + GT * kMaxSplits;  // [GT]
  const int ns = p.num_splits;
  if (warp < GT) {
    const int h = warp;
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml) +
                       (static_cast<int64_t>(b) * p.n_head + head0 + h) * ns;
    float2 v[kMaxSplits / 32];
    float mm = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int sp = lane + 32 * i;
      v[i] = sp < ns ? __ldcg(ml + sp) : make_float2(-INFINITY, 0.f);
      mm = fmaxf(mm, v[i].x);
    }
    mm = warp_max(mm);
    float ll = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int sp = lane + 32 * i;
      const float w = mm == -INFINITY ? 0.f : exp2f(v[i].x - mm);
      ll += v[i].y * w;
      if (sp < ns) wgt[h * kMaxSplits + sp] = w;
    }
    ll = warp_sum(ll);
    if (lane == 0) inv[h] = ll > 0.f ? 1.f / ll : 0.f;
  }
  __syncthreads();
  // Outputs: a thread owns 4 consecutive elements of one head and walks the splits with
  // independent 16-byte loads (unrolled, so several are in flight).
  for (int idx = threadIdx.x; idx < GT * (HD / 4); idx += kDecThreads) {
    const int h = idx / (HD / 4), e4 = idx % (HD / 4);
    const float4* po = reinterpret_cast<const float4*>(p.part_o) +
                       ((static_cast<int64_t>(b) * p.n_head + head0 + h) * ns) * (HD / 4) + e4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < ns; ++sp) {
      const float4 o = __ldcg(po + static_cast<int64_t>(sp) * (HD / 4));
      const float w = wgt[h * kMaxSplits + sp];
      acc.x = fmaf(o.x, w, acc.x);
      acc.y = fmaf(o.y, w, acc.y);
      acc.z = fmaf(o.z, w, acc.z);
      acc.w = fmaf(o.w, w, acc.w);
    }
    const float s = inv[h];
    T* dst = static_cast<T*>(p.out) + (static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + e4 * 4;
    uint2 packed;
    packed.x = pack2<T>(acc.x * s, acc.y * s);
    packed.y = pack2<T>(acc.z * s, acc.w * s);
    *reinterpret_cast<uint2*>(dst) = packed;
  }
  if (threadIdx.x == 0) *counter = 0u;  // ready for the next call
}

// =====================================================================================================
// F4 prefill
// =====================================================================================================
constexpr int kPfBlockM = 64, kPfBlockN = 64, kPfThreads = 128;

struct PrefillParams {
  const void* q;  // [B, S, n_head, HD]
  const void* k_cache;
  const void* v_cache;
  const void* input_pos;
  int pos_is_i64;
  void* out;  // [B, S, n_head * HD]
  int S, n_head, n_kv;
  int64_t smax;
  float scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 zero-fills the 16 destination bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Grid (ceil(S / 64), n_head, B).  Each of the 4 warps owns 16 query rows; K and V tiles of 64
// positions are staged in shared memory with padded rows (HD + 8 elements) so that ldmatrix
// reads are bank-conflict free.
template <typename T, int HD>
__global__ void __launch_bounds__(kPfThreads) attn_prefill_kernel(const PrefillParams p) {
  constexpr int LDS = HD + 8;          // padded row length in elements
  constexpr int KB = HD / 16;          // k blocks of the QK^T product
  constexpr int NB = kPfBlockN / 8;    // n blocks (key columns) of a score tile
  constexpr int OB = HD / 8;           // n blocks of the output
  constexpr int CPR = HD / 8;          // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t pf_smem[];
  T* sq = reinterpret_cast<T*>(pf_smem);
  T* sk = sq + kPfBlockM * LDS;
  T* sv = sk + kPfBlockN * LDS;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q0 = blockIdx.x * kPfBlockM;
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = head / (p.n_head / p.n_kv);
  int64_t pos0 = load_pos(p.input_pos, p.pos_is_i64, 0);
  pos0 = pos0 < 0 ? 0 : pos0;
  const int q_end = (q0 + kPfBlockM < p.S) ? q0 + kPfBlockM : p.S;
  int64_t kv_end = pos0 + q_end;  // keys 0 .. pos0 + q_end - 1 are visible to the last row
  kv_end = kv_end > p.smax ? p.smax : kv_end;

  const T* qg = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.S * p.n_head + head) * HD;
  const T* kg = static_cast<const T*>(p.k_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD;
  const T* vg = static_cast<const T*>(p.v_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD;

  // ---- Q tile -> shared -> A fragments ---------------------------------------------------------------
  for (int c = threadIdx.x; c < kPfBlockM * CPR; c += kPfThreads) {
    const int r = c / CPR, cc = c % CPR;
    const int s = q0 + r;
    const bool ok = s < p.S;
    const T* src = qg + static_cast<int64_t>(ok ? s : 0) * p.n_head * HD + cc * 8;
    cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(sq + r * LDS + cc * 8)), src, ok);
  }
  cp_async_wait_all();
  __syncthreads();
  uint32_t qa[KB][4];
  {
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int col = (lane >> 4) * 8;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb)
      ldmatrix_x4(static_cast<uint32_t>(__cvta_generic_to_shared(sq + row * LDS + kb * 16 + col)), qa[kb]);
  }

  float o[OB][4];
#pragma unroll
  for (int i = 0; i < OB; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // absolute positions of the two query rows this thread holds scores for
  const int64_t qpos0 = pos0 + q0 + warp * 16 + (lane >> 2);
  const int64_t qpos1 = qpos0 + 8;

  const int n_tiles = static_cast<int>((kv_end + kPfBlockN - 1) / kPfBlockN);
  for (int t = 0; t < n_tiles; ++t) {
    const int64_t kv0 = static_cast<int64_t>(t) * kPfBlockN;
    __syncthreads();  // everyone is done with the previous K/V tiles
    for (int c = threadIdx.x; c < kPfBlockN * CPR; c += kPfThreads) {
      const int r = c / CPR, cc = c % CPR;
      const int64_t j = kv0 + r;
      const bool ok = j < kv_end;
      const int64_t jc = ok ? j : 0;
      cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(sk + r * LDS + cc * 8)), kg + jc * HD + cc * 8, ok);
      cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(sv + r * LDS + cc * 8)), vg + jc * HD + cc * 8, ok);
    }
    cp_async_wait_all();
    __syncthreads();

    // ---- scores: 16 x 64 per warp ------------------------------------------------------------------
    float sc[NB][4];
#pragma unroll
    for (int i = 0; i < NB; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[i][e] = 0.f;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
      for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
        // two key blocks (16 keys) x 16 k-elements per ldmatrix.x4
        const int krow = nb2 * 16 + (lane & 7) + (lane >> 4) * 8;
        const int kcol = kb * 16 + ((lane >> 3) & 1) * 8;
        uint32_t bf[4];
        ldmatrix_x4(static_cast<uint32_t>(__cvta_generic_to_shared(sk + krow * LDS + kcol)), bf);
        mma16816<T>(sc[2 * nb2], qa[kb], bf[0], bf[1]);
        mma16816<T>(sc[2 * nb2 + 1], qa[kb], bf[2], bf[3]);
      }
    }

    // ---- scale, causal mask, online softmax -----------------------------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int64_t key = kv0 + nb * 8 + (lane & 3) * 2;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t kj = key + (e & 1);
        const int64_t qp = (e < 2) ? qpos0 : qpos1;
        const float v = (kj <= qp && kj < kv_end) ? sc[nb][e] * p.scale_log2 : -INFINITY;
        sc[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      // a row with no visible key yet keeps m = -inf; use 0 as the reference so exp2 stays finite
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use);
      m_run[r] = m_new;
      mx[r] = m_use;
      l_run[r] *= corr[r];
    }
    uint32_t pa[NB / 2][4];
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[e] = exp2f(sc[nb][e] - mx[e >> 1]);
        rs[e >> 1] += pv[e];
      }
      pa[nb >> 1][(nb & 1) * 2 + 0] = pack2<T>(pv[0], pv[1]);
      pa[nb >> 1][(nb & 1) * 2 + 1] = pack2<T>(pv[2], pv[3]);
    }
    l_run[0] += rs[0];
    l_run[1] += rs[1];
#pragma unroll
    for (int i = 0; i < OB; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }

    // ---- O += P V ----------------------------------------------------------------------------------------
#pragma unroll
    for (int jb = 0; jb < kPfBlockN / 16; ++jb) {
#pragma unroll
      for (int ob2 = 0; ob2 < OB / 2; ++ob2) {
        const int vrow = jb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int vcol = ob2 * 16 + (lane >> 4) * 8;
        uint32_t bf[4];
        ldmatrix_x4_trans(static_cast<uint32_t>(__cvta_generic_to_shared(sv + vrow * LDS + vcol)), bf);
        mma16816<T>(o[2 * ob2], pa[jb], bf[0], bf[1]);
        mma16816<T>(o[2 * ob2 + 1], pa[jb], bf[2], bf[3]);
      }
    }
  }

  // ---- finalize: row sums across the 4 lanes of a row, normalise, store ---------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  const int s0 = q0 + warp * 16 + (lane >> 2), s1 = s0 + 8;
  T* og = static_cast<T*>(p.out) + (static_cast<int64_t>(b) * p.S * p.n_head + head) * HD;
#pragma unroll
  for (int i = 0; i < OB; ++i) {
    const int e = i * 8 + (lane & 3) * 2;
    if (s0 < p.S)
      *reinterpret_cast<uint32_t*>(og + static_cast<int64_t>(s0) * p.n_head * HD + e) = pack2<T>(o[i][0] * inv0, o[i][1] * inv0);
    if (s1 < p.S)
      *reinterpret_cast<uint32_t*>(og + static_cast<int64_t>(s1) * p.n_head * HD + e) = pack2<T>(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// =====================================================================================================
// F3, large batches: the query heads of one KV head as the rows of tensor-core tiles
// =====================================================================================================
// With 16 or more sequences the K/V bytes of a layer are tens to hundreds of MB and the kernel
// above, built for the latency of a single sequence (every K row costs shuffle-reduced dot
// products for each query head), cannot issue fast enough to stream them.  Here a CTA takes one
// (sequence, KV head, range of positions) and treats the g <= 16 query heads that share the KV head
// as the 16 rows of mma.sync tiles: S = Q K^T and O += P V run on the tensor cores exactly as in
// the prefill kernel, with a "query tile" that is the head group instead of 16 positions.  Each of
// the 4 warps walks its own tiles of 16 positions (tile w, w + 4, ...) through a private 3-stage
// cp.async ring (8.5 KB per stage: about 100 KB in flight per CTA, two CTAs per SM), keeps its
// own online-softmax state, and the warps, then the ranges, are merged as in the kernel above.
constexpr int kMmaDecWarps = 4;
constexpr int kMmaDecThreads = kMmaDecWarps * 32;
constexpr int kMmaDecStages = 3;
constexpr int kMmaDecTile = 16;   // positions per warp tile
constexpr int kMmaDecMaxGroup = 16;

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int HD>
__global__ void __launch_bounds__(kMmaDecThreads, 2) attn_decode_mma_kernel(const DecodeParams p) {
  constexpr int LDS = HD + 8;  // padded row length in elements (bank-conflict-free ldmatrix)
  constexpr int KB = HD / 16;  // k blocks of Q K^T
  constexpr int OB = HD / 8;   // 8-column blocks of the output
  constexpr int CPR = HD / 8;  // 16-byte chunks per row
  constexpr int kTileElems = kMmaDecTile * LDS;
  constexpr int kStageElems = 2 * kTileElems;  // K tile, V tile
  extern __shared__ __align__(16) uint8_t dm_smem[];
  T* sq = reinterpret_cast<T*>(dm_smem);                      // [16][LDS]
  T* ring = sq + kMmaDecTile * LDS;                            // [warps][stages][K | V]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int g = p.n_head / p.n_kv;
  const int head0 = kvh * g;

  pdl_launch_dependents();
  pdl_wait();  // q and the newest cache row were written by the preceding kernel
  int64_t ctx = load_pos(p.input_pos, p.pos_is_i64, 0) + 1;
  ctx = ctx < 0 ? 0 : (ctx > p.smax ? p.smax : ctx);
  const int64_t chunk = (ctx + p.num_splits - 1) / p.num_splits;
  const int64_t p0 = split * chunk;
  const int64_t p1 = (p0 + chunk < ctx) ? p0 + chunk : ctx;
  const int n_tiles = p1 > p0 ? static_cast<int>((p1 - p0 + kMmaDecTile - 1) / kMmaDecTile) : 0;

  const T* kg = static_cast<const T*>(p.k_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD;
  const T* vg = static_cast<const T*>(p.v_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD;
  T* my_ring = ring + warp * (kMmaDecStages * kStageElems);

  // tile `t` (positions p0 + 16 t ...) of this range into stage `st` of the warp's ring
  auto issue = [&](int t, int st) {
    if (t < n_tiles) {
      T* dk = my_ring + st * kStageElems;
      T* dv = dk + kTileElems;
      const int64_t j0 = p0 + static_cast<int64_t>(t) * kMmaDecTile;
#pragma unroll
      for (int c = lane; c < kMmaDecTile * CPR; c += 32) {
        const int r = c / CPR, cc = c % CPR;
        const int64_t j = j0 + r;
        const bool ok = j < p1;
        const int64_t jc = ok ? j : 0;
        cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(dk + r * LDS + cc * 8)), kg + jc * HD + cc * 8, ok);
        cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(dv + r * LDS + cc * 8)), vg + jc * HD + cc * 8, ok);
      }
    }
    cp_async_commit();  // always: the group count per thread stays the same on every path
  };
  // start the K/V stream, then fetch Q behind it
#pragma unroll
  for (int s = 0; s < kMmaDecStages - 1; ++s) issue(warp + s * kMmaDecWarps, s);

  // ---- Q: head h of the group is row h; rows from g up are zero -----------------------------------
  const T* qg = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.n_head + head0) * HD;
  for (int c = threadIdx.x; c < kMmaDecTile * CPR; c += kMmaDecThreads) {
    const int r = c / CPR, cc = c % CPR;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < g) v = *reinterpret_cast<const uint4*>(qg + static_cast<int64_t>(r) * HD + cc * 8);
    *reinterpret_cast<uint4*>(sq + r * LDS + cc * 8) = v;
  }
  __syncthreads();
  uint32_t qa[KB][4];
  {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int col = (lane >> 4) * 8;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb)
      ldmatrix_x4(static_cast<uint32_t>(__cvta_generic_to_shared(sq + row * LDS + kb * 16 + col)), qa[kb]);
  }

  float o[OB][4];
#pragma unroll
  for (int i = 0; i < OB; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  int it = 0;
  for (int t = warp; t < n_tiles; t += kMmaDecWarps, ++it) {
    // keep kMmaDecStages - 1 tiles in flight beyond the one being consumed
    issue(t + (kMmaDecStages - 1) * kMmaDecWarps, (it + kMmaDecStages - 1) % kMmaDecStages);
    cp_async_wait_group<kMmaDecStages - 1>();
    __syncwarp();
    const T* sk = my_ring + (it % kMmaDecStages) * kStageElems;
    const T* sv = sk + kTileElems;
    const int64_t kv0 = p0 + static_cast<int64_t>(t) * kMmaDecTile;

    // ---- scores 16 heads x 16 positions -----------------------------------------------------------
    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[i][e] = 0.f;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      const int krow = (lane & 7) + (lane >> 4) * 8;
      const int kcol = kb * 16 + ((lane >> 3) & 1) * 8;
      uint32_t bf[4];
      ldmatrix_x4(static_cast<uint32_t>(__cvta_generic_to_shared(sk + krow * LDS + kcol)), bf);
      mma16816<T>(sc[0], qa[kb], bf[0], bf[1]);
      mma16816<T>(sc[1], qa[kb], bf[2], bf[3]);
    }
    // ---- scale, mask the positions past the range, online softmax ------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int64_t key = kv0 + nb * 8 + (lane & 3) * 2;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = (key + (e & 1) < p1) ? sc[nb][e] * p.scale_log2 : -INFINITY;
        sc[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use);
      m_run[r] = m_new;
      mx[r] = m_use;
      l_run[r] *= corr[r];
    }
    uint32_t pa[4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[e] = exp2f(sc[nb][e] - mx[e >> 1]);
        l_run[e >> 1] += pv[e];
      }
      pa[nb * 2 + 0] = pack2<T>(pv[0], pv[1]);
      pa[nb * 2 + 1] = pack2<T>(pv[2], pv[3]);
    }
#pragma unroll
    for (int i = 0; i < OB; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // ---- O += P V (16 positions = one k block) ------------------------------------------------------------
#pragma unroll
    for (int ob2 = 0; ob2 < OB / 2; ++ob2) {
      const int vrow = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int vcol = ob2 * 16 + (lane >> 4) * 8;
      uint32_t bf[4];
      ldmatrix_x4_trans(static_cast<uint32_t>(__cvta_generic_to_shared(sv + vrow * LDS + vcol)), bf);
      mma16816<T>(o[2 * ob2], pa, bf[0], bf[1]);
      mma16816<T>(o[2 * ob2 + 1], pa, bf[2], bf[3]);
    }
    __syncwarp();  // every lane is done with this stage before a later issue() overwrites it
  }
  cp_async_wait_all();
  __syncthreads();  // the rings are free: they now hold the warps' results

  // ---- the warps' (max, sum, values) per head, then the CTA's ---------------------------------------------
  float* sm_o = reinterpret_cast<float*>(ring);                       // [warps][16][HD]
  float* sm_m = sm_o + kMmaDecWarps * kMmaDecTile * HD;               // [warps][16]
  float* sm_l = sm_m + kMmaDecWarps * kMmaDecTile;                    // [warps][16]
  __shared__ unsigned int ticket_s;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    if ((lane & 3) == 0) {
      sm_m[warp * kMmaDecTile + r0] = m_run[0];
      sm_m[warp * kMmaDecTile + r1] = m_run[1];
      sm_l[warp * kMmaDecTile + r0] = l_run[0];
      sm_l[warp * kMmaDecTile + r1] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < OB; ++i) {
      const int e = i * 8 + (lane & 3) * 2;
      float* d0 = sm_o + (warp * kMmaDecTile + r0) * HD + e;
      float* d1 = sm_o + (warp * kMmaDecTile + r1) * HD + e;
      d0[0] = o[i][0];
      d0[1] = o[i][1];
      d1[0] = o[i][2];
      d1[1] = o[i][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < g * HD; idx += kMmaDecThreads) {
    const int h = idx / HD, e = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaDecWarps; ++w) mm = fmaxf(mm, sm_m[w * kMmaDecTile + h]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kMmaDecWarps; ++w) {
        const float wt = exp2f(sm_m[w * kMmaDecTile + h] - mm);  // 0 for warps that saw no position
        ll += sm_l[w * kMmaDecTile + h] * wt;
        oo += sm_o[(w * kMmaDecTile + h) * HD + e] * wt;
      }
    }
    const int64_t slot = (static_cast<int64_t>(b) * p.n_head + head0 + h) * p.num_splits + split;
    p.part_o[slot * HD + e] = oo;
    if (e == 0) {
      p.part_ml[slot * 2] = mm;
      p.part_ml[slot * 2 + 1] = ll;
    }
  }

  // ---- the last CTA of this (sequence, KV head) merges the ranges ---------------------------------------------
  __threadfence();
  __syncthreads();
  unsigned int* counter = p.counters + static_cast<int64_t>(b) * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) ticket_s = atomicAdd(counter, 1u);
  __syncthreads();
  if (ticket_s != static_cast<unsigned int>(p.num_splits - 1)) return;
  __threadfence();
  float* wgt = sm_o;                                  // [g][kMaxSplits]
  float* inv = wgt + kMmaDecMaxGroup * kMaxSplits;    // [g]
  const int ns = p.num_splits;
  for (int h = warp; h < g; h += kMmaDecWarps) {
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + (static_cast<int64_t>(b) * p.n_head + head0 + h) * ns;
    float2 v[kMaxSplits / 32];
    float mm = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int sp = lane + 32 * i;
      v[i] = sp < ns ? __ldcg(ml + sp) : make_float2(-INFINITY, 0.f);
      mm = fmaxf(mm, v[i].x);
    }
    mm = warp_max(mm);
    float ll = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxSplits / 32; ++i) {
      const int sp = lane + 32 * i;
      const float w = mm == -INFINITY ? 0.f : exp2f(v[i].x - mm);
      ll += v[i].y * w;
      if (sp < ns) wgt[h * kMaxSplits + sp] = w;
    }
    ll = warp_sum(ll);
    if (lane == 0) inv[h] = ll > 0.f ? 1.f / ll : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < g * (HD / 4); idx += kMmaDecThreads) {
    const int h = idx / (HD / 4), e4 = idx % (HD / 4);
    const float4* po = reinterpret_cast<const float4*>(p.part_o) +
                       ((static_cast<int64_t>(b) * p.n_head + head0 + h) * ns) * (HD / 4) + e4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < ns; ++sp) {
      const float4 ov = __ldcg(po + static_cast<int64_t>(sp) * (HD / 4));
      const float w = wgt[h * kMaxSplits + sp];
      acc.x = fmaf(ov.x, w, acc.x);
      acc.y = fmaf(ov.y, w, acc.y);
      acc.z = fmaf(ov.z, w, acc.z);
      acc.w = fmaf(ov.w, w, acc.w);
    }
    const float s = inv[h];
    T* dst = static_cast<T*>(p.out) + (static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + e4 * 4;
    uint2 packed;
    packed.x = pack2<T>(acc.x * s, acc.y * s);
    packed.y = pack2<T>(acc.z * s, acc.w * s);
    *reinterpret_cast<uint2*>(dst) = packed;
  }
  if (threadIdx.x == 0) *counter = 0u;  // ready for the next call
}

template <int HD>
constexpr int mma_decode_smem() {
  return (kMmaDecTile + kMmaDecWarps * kMmaDecStages * 2 * kMmaDecTile) * (HD + 8) * 2;
}

template <typename T, int HD>
int launch_decode_mma(const DecodeParams& p, int B, cudaStream_t st) {
  constexpr int smem = mma_decode_smem<HD>();
  static_assert(kMmaDecWarps * kMmaDecTile * HD * 4 + 2 * kMmaDecWarps * kMmaDecTile * 4 <= smem - kMmaDecTile * (HD + 8) * 2,
                "the merge arrays must fit in the rings");
  static_assert((kMmaDecMaxGroup * kMaxSplits + kMmaDecMaxGroup) * 4 <= kMmaDecWarps * kMmaDecTile * HD * 4,
                "the split weights must fit in the value array");
  auto kern = attn_decode_mma_kernel<T, HD>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  LRI_ONCE_PER_DEVICE(attr_set, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.num_splits, p.n_kv, B);
  LRI_CUDA(launch_pdl(kern, grid, dim3(kMmaDecThreads), static_cast<size_t>(smem), st, p));
  LRI_LAUNCH_CHECK("attn_decode_mma_kernel");
  return LRI_OK;
}

template <typename T, int HD>
int launch_decode(const DecodeParams& p, int B, cudaStream_t st) {
  const int g = p.n_head / p.n_kv;
  const int gt = (g % 4 == 0) ? 4 : ((g % 2 == 0) ? 2 : 1);
  dim3 grid(p.num_splits, p.n_kv * (g / gt), B);
  if (gt == 4)
    LRI_CUDA(launch_pdl(attn_decode_kernel<T, HD, 4>, grid, dim3(kDecThreads), 0, st, p));
  else if (gt == 2)
    LRI_CUDA(launch_pdl(attn_decode_kernel<T, HD, 2>, grid, dim3(kDecThreads), 0, st, p));
  else
    LRI_CUDA(launch_pdl(attn_decode_kernel<T, HD, 1>, grid, dim3(kDecThreads), 0, st, p));
  LRI_LAUNCH_CHECK("attn_decode_kernel");
  return LRI_OK;
}

template <typename T, int HD>
int launch_prefill(const PrefillParams& p, int B, cudaStream_t st) {
  constexpr int smem = (kPfBlockM + 2 * kPfBlockN) * (HD + 8) * 2;
  auto kern = attn_prefill_kernel<T, HD>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  LRI_ONCE_PER_DEVICE(attr_set, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.S + kPfBlockM - 1) / kPfBlockM, p.n_head, B);
  kern<<<grid, kPfThreads, smem, st>>>(p);
  LRI_LAUNCH_CHECK("attn_prefill_kernel");
  return LRI_OK;
}

// Which decode kernel: the tensor-core kernel from 128 (sequence, KV head) pairs on (measured on
// B200 at 8 KV heads, context 1152: batch 16 20.0 vs 24.0 us, batch 64 59 vs 82 us per layer),
// the latency kernels below that.  LRI_ATTN_MMA=1 / 0 forces / forbids it.
bool attn_mma_wanted(int B, int n_kv) {
  const int mode = option(OPT_ATTN_MMA);
  return mode == 1 || (mode == -1 && static_cast<int64_t>(B) * n_kv >= 128);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
// The arrival counters take a fixed region at the start of the scratch buffer, so that calls
// with different batch sizes can share one zero-initialised buffer.
constexpr size_t kCounterBytes = 32768;
constexpr size_t kMaxCounterRows = kCounterBytes / 4;

int check_attn(const char* who, int dtype, int B, int n_head, int n_kv, int head_dim, int64_t smax) {
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "%s: dtype %d", who, dtype);
  LRI_REQUIRE(B >= 0 && B <= 65535, LRI_ERR_ARG, "%s: B=%d", who, B);
  LRI_REQUIRE(n_head > 0 && n_kv > 0 && n_head % n_kv == 0 && n_head <= 65535, LRI_ERR_ARG,
              "%s: n_head=%d must be a positive multiple of n_kv=%d", who, n_head, n_kv);
  LRI_REQUIRE(head_dim == 64 || head_dim == 128, LRI_ERR_UNSUPPORTED, "%s: head_dim=%d (64 and 128 are built)", who,
              head_dim);
  LRI_REQUIRE(smax > 0, LRI_ERR_ARG, "%s: smax=%lld", who, (long long)smax);
  return LRI_OK;
}

}  // namespace
}  // namespace lri

using namespace lri;

extern "C" size_t lri_attn_decode_scratch_bytes(int B, int n_head, int n_kv, int head_dim, int num_splits) {
  (void)n_kv;
  if (B <= 0 || n_head <= 0 || head_dim <= 0 || num_splits <= 0) return 0;
  const size_t rows = static_cast<size_t>(B) * n_head;
  return kCounterBytes + align_up(rows * num_splits * 2 * 4, 16) + rows * num_splits * head_dim * 4;
}

// Number of sequence ranges, fixed per cache geometry so that the launch grid never depends on the
// current position.  Up to 8 ranges (a power of two; 16 for a one- or two-cluster launch) run as one
// thread-block cluster and merge through shared memory; that form is kept as long as a CTA then streams at most ~1 MB of K/V.
// Longer caches take more ranges (up to 64, at least 64 positions each) and merge through the scratch
// buffer.  The tensor-core kernel (from 128 (sequence, KV head) pairs on) takes one range per pair,
// two only while one per pair would leave SMs without work.
extern "C" int lri_attn_decode_plan(int B, int n_head, int n_kv, int head_dim, int64_t smax, int* num_splits) {
  LRI_REQUIRE(num_splits != nullptr, LRI_ERR_ARG, "attn_decode_plan: NULL output");
  LRI_REQUIRE(B >= 1 && n_head >= 1 && n_kv >= 1 && n_head % n_kv == 0 && head_dim >= 1 && smax >= 1, LRI_ERR_ARG,
              "attn_decode_plan: B=%d n_head=%d n_kv=%d head_dim=%d smax=%lld", B, n_head, n_kv, head_dim, (long long)smax);
  const int64_t sms = device_sm_count();
  const int forced = option(OPT_DECODE_SPLITS);
  if (forced > 0) {
    const int64_t cap = smax / 32 > 1 ? smax / 32 : 1;
    *num_splits = static_cast<int>(forced < cap ? forced : cap);
    return LRI_OK;
  }
  const int g = n_head / n_kv;
  if (g <= kMmaDecMaxGroup && attn_mma_wanted(B, n_kv)) {
    *num_splits = (static_cast<int64_t>(B) * n_kv < 2 * sms && smax >= 256) ? 2 : 1;
    return LRI_OK;
  }
  const int gt = attn_decode_cluster_head_tile(B, n_kv, g);
  const int64_t base = static_cast<int64_t>(B) * n_kv * (g / gt);
  const int64_t want = (2 * sms + base - 1) / base;
  const int64_t bytes_per_cta_at_8 = smax * head_dim * 2 * 2 / 8;
  if (want <= 8 || bytes_per_cta_at_8 <= (1 << 20)) {
    // clusters of 16 (the opt-in maximum) only for up to four clusters, i.e. a shard of one or two KV heads of
    // a single sequence with its query heads spread over the clusters (measured on B200, context 1152, one
    // cluster: 5.4 vs 6.7 us); with 8 clusters they are slower than 8 both alone (10.0 vs 8.3 us) and next to
    // the MLP chain they share the SMs with
    const int64_t cap = (base <= 4 && attn_decode_cluster_supports(16)) ? 16 : 8;
    int n = 1;
    const int64_t lim = want < cap ? want : cap;
    while (n * 2 <= lim && smax / (n * 2) >= 32) n *= 2;
    *num_splits = n;
    return LRI_OK;
  }
  int64_t n = want < 64 ? want : 64;
  const int64_t by_len = smax / 64 > 1 ? smax / 64 : 1;
  n = n < by_len ? n : by_len;
  *num_splits = static_cast<int>(n < 1 ? 1 : n);
  return LRI_OK;
}

extern "C" int lri_attn_decode(int dtype, const void* q, const void* k_cache, const void* v_cache,
                               const void* input_pos, int pos_is_i64, void* out, int B, int n_head, int n_kv,
                               int head_dim, int64_t smax, int num_splits, void* scratch, size_t scratch_bytes,
                               lri_stream_t stream) {
  int rc = check_attn("attn_decode", dtype, B, n_head, n_kv, head_dim, smax);
  if (rc != LRI_OK) return rc;
  LRI_REQUIRE(q && k_cache && v_cache && input_pos && out, LRI_ERR_ARG, "attn_decode: NULL pointer");
  LRI_REQUIRE(num_splits >= 1 && num_splits <= kMaxSplits, LRI_ERR_ARG, "attn_decode: num_splits=%d outside 1..%d",
              num_splits, kMaxSplits);
  LRI_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && aligned16(out), LRI_ERR_ALIGN,
              "attn_decode: pointers must be 16-byte aligned");
  const bool mma = attn_mma_wanted(B, n_kv) && n_head / n_kv <= kMmaDecMaxGroup && scratch != nullptr;
  if (!mma && attn_decode_cluster_supports(num_splits)) {
    // 1, 2, 4, 8 or 16 splits: the splits are the CTAs of one cluster and merge through distributed
    // shared memory; the scratch buffer is not touched
    if (B == 0) return LRI_OK;
    return attn_decode_cluster_launch(dtype, q, k_cache, v_cache, input_pos, pos_is_i64, out, B, n_head, n_kv,
                                      head_dim, smax, num_splits, kLog2e / sqrtf(static_cast<float>(head_dim)),
                                      static_cast<cudaStream_t>(stream));
  }
  LRI_REQUIRE(scratch && aligned16(scratch) &&
                  scratch_bytes >= lri_attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits),
              LRI_ERR_WORKSPACE, "attn_decode: scratch of %zu bytes (16-byte aligned) required",
              lri_attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits));
  if (B == 0) return LRI_OK;
  const size_t rows = static_cast<size_t>(B) * n_head;
  LRI_REQUIRE(rows <= kMaxCounterRows, LRI_ERR_UNSUPPORTED, "attn_decode: B*n_head=%zu exceeds %zu", rows,
              kMaxCounterRows);
  DecodeParams p{};
  p.q = q, p.k_cache = k_cache, p.v_cache = v_cache, p.input_pos = input_pos, p.pos_is_i64 = pos_is_i64, p.out = out;
  p.n_head = n_head, p.n_kv = n_kv, p.smax = smax, p.num_splits = num_splits;
  p.scale_log2 = kLog2e / sqrtf(static_cast<float>(head_dim));
  uint8_t* s = static_cast<uint8_t*>(scratch);
  p.counters = reinterpret_cast<unsigned int*>(s);
  p.part_ml = reinterpret_cast<float*>(s + kCounterBytes);
  p.part_o = reinterpret_cast<float*>(s + kCounterBytes + align_up(rows * num_splits * 2 * 4, 16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mma) {
    if (dtype == LRI_BF16)
      return head_dim == 128 ? launch_decode_mma<__nv_bfloat16, 128>(p, B, st)
                             : launch_decode_mma<__nv_bfloat16, 64>(p, B, st);
    return head_dim == 128 ? launch_decode_mma<__half, 128>(p, B, st) : launch_decode_mma<__half, 64>(p, B, st);
  }
  if (dtype == LRI_BF16)
    return head_dim == 128 ? launch_decode<__nv_bfloat16, 128>(p, B, st) : launch_decode<__nv_bfloat16, 64>(p, B, st);
  return head_dim == 128 ? launch_decode<__half, 128>(p, B, st) : launch_decode<__half, 64>(p, B, st);
}

extern "C" int lri_attn_prefill(int dtype, const void* q, const void* k_cache, const void* v_cache,
                                const void* input_pos, int pos_is_i64, void* out, int B, int S, int n_head, int n_kv,
                                int head_dim, int64_t smax, lri_stream_t stream) {
  int rc = check_attn("attn_prefill", dtype, B, n_head, n_kv, head_dim, smax);
  if (rc != LRI_OK) return rc;
  LRI_REQUIRE(q && k_cache && v_cache && input_pos && out, LRI_ERR_ARG, "attn_prefill: NULL pointer");
  LRI_REQUIRE(S >= 0 && S <= (1 << 22), LRI_ERR_ARG, "attn_prefill: S=%d", S);
  LRI_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && aligned16(out), LRI_ERR_ALIGN,
              "attn_prefill: pointers must be 16-byte aligned");
  if (B == 0 || S == 0) return LRI_OK;
  // option attn_prefill_tc: 1 = the tcgen05 / TMEM kernel (default), 0 = the mma.sync kernel below
  if (option(OPT_ATTN_PREFILL_TC) != 0 && attn_prefill_tc_supports(B, S, n_head, n_kv, head_dim, smax))
    return attn_prefill_tc_launch(dtype, q, k_cache, v_cache, input_pos, pos_is_i64, out, B, S, n_head, n_kv, head_dim,
                                  smax, kLog2e / sqrtf(static_cast<float>(head_dim)), static_cast<cudaStream_t>(stream));
  PrefillParams p{};
  p.q = q, p.k_cache = k_cache, p.v_cache = v_cache, p.input_pos = input_pos, p.pos_is_i64 = pos_is_i64, p.out = out;
  p.S = S, p.n_head = n_head, p.n_kv = n_kv, p.smax = smax;
  p.scale_log2 = kLog2e / sqrtf(static_cast<float>(head_dim));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == LRI_BF16)
    return head_dim == 128 ? launch_prefill<__nv_bfloat16, 128>(p, B, st) : launch_prefill<__nv_bfloat16, 64>(p, B, st);
  return head_dim == 128 ? launch_prefill<__half, 128>(p, B, st) : launch_prefill<__half, 64>(p, B, st);
}

// =====================================================================================================
// Decode attention for callers that cannot hand over scratch memory
// =====================================================================================================
// Some callers of this library own no allocator they may use on the hot path: a plug-in that is
// given only tensors and a stream by its host framework, or a serving process whose device
// memory was planned up front and in which a cudaMalloc (which synchronises the whole device)
// is forbidden once traffic flows.  For them the split partials and arrival counters of the
// decode-attention kernel live in the fixed array below, which every GPU that loads this library
// keeps until the process exits.
namespace lri {
namespace {
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB per GPU
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
}  // namespace
}  // namespace lri

extern "C" size_t lri_attn_decode_static_scratch_capacity(void) { return lri::kStaticScratchBytes; }

extern "C" int lri_attn_decode_static(int dtype, const void* q, const void* k_cache, const void* v_cache,
                                      const void* input_pos, int pos_is_i64, void* out, int B, int n_head,
                                      int n_kv, int head_dim, int64_t smax, int num_splits, lri_stream_t stream) {
  const size_t need = lri_attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits);
  LRI_REQUIRE(need <= kStaticScratchBytes, LRI_ERR_WORKSPACE,
              "attn_decode_static: B=%d n_head=%d head_dim=%d num_splits=%d needs %zu bytes of scratch, the built-in "
              "array holds %zu; lower num_splits or use lri_attn_decode with caller-owned scratch",
              B, n_head, head_dim, num_splits, need, kStaticScratchBytes);
  int dev = -1;
  LRI_CUDA(cudaGetDevice(&dev));
  LRI_REQUIRE(dev >= 0 && dev < kMaxDevices, LRI_ERR_UNSUPPORTED, "attn_decode_static: device ordinal %d", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {
    // In host code the array's name is only a handle; the address the kernel must get comes from
    // the runtime, for the device that is current now.  Done on the first call per device.
    void* p = nullptr;
    LRI_CUDA(cudaGetSymbolAddress(&p, g_static_decode_scratch));
    LRI_REQUIRE(p != nullptr, LRI_ERR_CUDA, "attn_decode_static: no device address for the scratch array");
    g_static_scratch_ptr[dev] = p;
  }
  return lri_attn_decode(dtype, q, k_cache, v_cache, input_pos, pos_is_i64, out, B, n_head, n_kv, head_dim, smax,
                         num_splits, g_static_scratch_ptr[dev], kStaticScratchBytes, stream);
}
