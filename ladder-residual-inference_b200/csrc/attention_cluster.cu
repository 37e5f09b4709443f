// F3, low-latency form: GQA decode attention whose sequence splits are the CTAs of one
// thread-block cluster and are merged through distributed shared memory.
//
// At decode batch sizes the K/V bytes of one layer are a few MB, so the kernel is a chain of
// memory round trips, not a bandwidth problem.  The split-K form that goes through global
// scratch pays for: partial store, fence, atomic ticket, two rounds of partial loads.  Here the
// num_splits (1, 2, 4, 8 or 16) CTAs that share a (batch, kv-head tile) form a cluster.  A CTA
// issues the loads of its whole range at once when the range is short enough (U positions per row
// group in flight, chosen from the cache length at launch, so a 1 K context costs one DRAM round
// trip instead of three), merges its row groups in shared memory and stores its (max, sum, weighted
// values) straight into the shared memory of the cluster's first CTA (remote stores are fire and
// forget, remote loads are a round trip).  After ONE cluster barrier the first CTA merges the splits
// and writes the output; the others exit.  No scratch memory, no counters, and the grid still does
// not depend on the position.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace lri {
int attn_decode_cluster_head_tile(int B, int n_kv, int g);

namespace {

constexpr int kClWarps = 8;
constexpr int kClThreads = kClWarps * 32;
constexpr int kClMaxSplits = 16;

struct ClusterDecodeParams {
  const void* q;        // [B, n_head, HD]
  const void* k_cache;  // [B_max, n_kv, smax, HD]
  const void* v_cache;
  const void* input_pos;
  int pos_is_i64;
  void* out;  // [B, n_head * HD]
  int n_head, n_kv;
  int64_t smax;
  float scale_log2;
};

// dynamic shared memory: [NRG][GT] max, [NRG][GT] sum, [NRG][GT][HD] values (this CTA's row groups), then the
// splits' results as gathered in the cluster's first CTA: [16][GT][HD] values, [16][GT] max, [16][GT] sum
template <int HD, int GT>
constexpr int cluster_smem_bytes() {
  constexpr int NRG = (32 / (HD / 8)) * kClWarps;
  return (NRG * GT * (2 + HD) + kClMaxSplits * GT * (HD + 2)) * 4;
}

template <typename T, int HD, int GT, int U>
__global__ void __launch_bounds__(kClThreads) attn_decode_cluster_kernel(const ClusterDecodeParams p) {
  constexpr int LPR = HD / 8;    // lanes per cache row
  constexpr int RPW = 32 / LPR;  // row groups per warp
  constexpr int NRG = RPW * kClWarps;
  cg::cluster_group cluster = cg::this_cluster();
  const int ns = static_cast<int>(cluster.num_blocks());  // == gridDim.x
  const int split = static_cast<int>(cluster.block_rank());
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sl = lane % LPR;
  const int rg = warp * RPW + lane / LPR;
  const int g = p.n_head / p.n_kv;
  const int tiles_per_kv = g / GT;
  const int kvh = blockIdx.y / tiles_per_kv;
  const int head0 = kvh * g + (blockIdx.y % tiles_per_kv) * GT;
  const int b = blockIdx.z;

  extern __shared__ __align__(16) float cl_smem[];
  float* sm_m = cl_smem;                  // [NRG][GT]
  float* sm_l = sm_m + NRG * GT;          // [NRG][GT]
  float* sm_o = sm_l + NRG * GT;          // [NRG][GT][HD]
  float* g_o = sm_o + NRG * GT * HD;      // [16][GT][HD]   (used in the cluster's first CTA)
  float* g_m = g_o + kClMaxSplits * GT * HD;  // [16][GT]
  float* g_l = g_m + kClMaxSplits * GT;       // [16][GT]

  const T* kbase = static_cast<const T*>(p.k_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;
  const T* vbase = static_cast<const T*>(p.v_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;
  {
    // While the preceding kernel (the QKV projection) still runs: ask the L2 for this CTA's share of the
    // cache, so that the loads below cost an L2 round trip instead of a DRAM one.  All rows but the newest
    // were written by earlier steps.  The position read here may still be the previous step's; it only
    // steers a hint (clamped to the cache), and the L2 is shared, so it does not matter which CTA asks.
    int64_t hint = (p.pos_is_i64 ? *reinterpret_cast<const volatile int64_t*>(p.input_pos)
                                 : static_cast<int64_t>(*reinterpret_cast<const volatile int32_t*>(p.input_pos))) + 2;
    hint = hint < 0 ? 0 : (hint > p.smax ? p.smax : hint);
    const int64_t hchunk = (hint + ns - 1) / ns;
    const int64_t h0 = split * hchunk;
    const int64_t h1 = (h0 + hchunk < hint) ? h0 + hchunk : hint;
    if ((sl & 7) == 0) {  // one request per 128-byte line
      for (int64_t j = h0 + rg; j < h1; j += NRG) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kbase + j * HD));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vbase + j * HD));
      }
    }
  }
  pdl_launch_dependents();
  pdl_wait();  // q and the newest cache row come from the preceding kernel
  int64_t ctx = load_pos(p.input_pos, p.pos_is_i64, 0) + 1;
  float qf[GT][8];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    const T* qp = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + sl * 8;
    unpack8<T>(*reinterpret_cast<const uint4*>(qp), qf[h]);
#pragma unroll
    for (int e = 0; e < 8; ++e) qf[h][e] *= p.scale_log2;
  }
  ctx = ctx < 0 ? 0 : (ctx > p.smax ? p.smax : ctx);
  const int64_t chunk = (ctx + ns - 1) / ns;
  const int64_t p0 = split * chunk;
  const int64_t p1 = (p0 + chunk < ctx) ? p0 + chunk : ctx;

  float m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
  }

  // Warp-uniform trip count (all 32 lanes run the shuffles); rows past the end are clamped and masked.
  // With U chosen at launch so that NRG * U covers the longest possible range, the loop body runs once.
  for (int64_t jb = p0 + warp * RPW; jb < p1; jb += static_cast<int64_t>(NRG) * U) {
    uint4 kv[U], vv[U];
    bool valid[U];
#pragma unroll
    for (int t = 0; t < U; ++t) {
      const int64_t j = jb + lane / LPR + static_cast<int64_t>(t) * NRG;
      valid[t] = j < p1;
      const int64_t jc = valid[t] ? j : p1 - 1;
      kv[t] = ld_stream16(kbase + jc * HD);
      vv[t] = ld_stream16(vbase + jc * HD);
    }
    float s[U][GT];
#pragma unroll
    for (int t = 0; t < U; ++t) {
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
      for (int t = 1; t < U; ++t) mx = fmaxf(mx, s[t][h]);
      const float m_new = fmaxf(m[h], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;  // no valid position yet: exponentials give 0
      const float corr = exp2f(m[h] - m_use);
      l[h] *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
      m[h] = m_new;
#pragma unroll
      for (int t = 0; t < U; ++t) s[t][h] = exp2f(s[t][h] - m_use);
    }
#pragma unroll
    for (int t = 0; t < U; ++t) {
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

  // ---- merge the row groups of this CTA, result straight into the first CTA's gather arrays ------------
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    if (sl == 0) {
      sm_m[rg * GT + h] = m[h];
      sm_l[rg * GT + h] = l[h];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sm_o[(rg * GT + h) * HD + sl * 8 + e] = acc[h][e];
  }
  __syncthreads();
  float* r_o = cluster.map_shared_rank(g_o, 0);
  float* r_m = cluster.map_shared_rank(g_m, 0);
  float* r_l = cluster.map_shared_rank(g_l, 0);
  for (int idx = threadIdx.x; idx < GT * HD; idx += kClThreads) {
    const int h = idx / HD, e = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < NRG; ++r) mm = fmaxf(mm, sm_m[r * GT + h]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int r = 0; r < NRG; ++r) {
        const float w = exp2f(sm_m[r * GT + h] - mm);
        ll += sm_l[r * GT + h] * w;
        oo += sm_o[(r * GT + h) * HD + e] * w;
      }
    }
    r_o[(split * GT + h) * HD + e] = oo;
    if (e == 0) {
      r_m[split * GT + h] = mm;
      r_l[split * GT + h] = ll;
    }
  }
  cluster.sync();  // every split's result has landed in the first CTA's shared memory
  if (split != 0) return;

  // ---- the first CTA merges the splits -----------------------------------------------------------------
  for (int idx = threadIdx.x; idx < GT * HD; idx += kClThreads) {
    const int h = idx / HD, e = idx % HD;
    float mm = -INFINITY;
    for (int r = 0; r < ns; ++r) mm = fmaxf(mm, g_m[r * GT + h]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
      for (int r = 0; r < ns; ++r) {
        const float w = exp2f(g_m[r * GT + h] - mm);
        ll += g_l[r * GT + h] * w;
        oo += g_o[(r * GT + h) * HD + e] * w;
      }
    }
    const float res = ll > 0.f ? oo / ll : 0.f;
    static_cast<T*>(p.out)[(static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + e] = Num<T>::from_f(res);
  }
}

template <typename T, int HD, int GT, int U>
int launch_one(const ClusterDecodeParams& p, int B, int ns, int tiles, cudaStream_t st) {
  constexpr int smem = cluster_smem_bytes<HD, GT>();
  auto kern = attn_decode_cluster_kernel<T, HD, GT, U>;
  static std::atomic<unsigned long long> attr_set{0};  // per template instantiation, one bit per device
  if (device_setup_needed(attr_set)) {
    LRI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    LRI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    device_setup_done(attr_set);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ns, tiles, B);
  cfg.blockDim = dim3(kClThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ns;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  LRI_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  LRI_LAUNCH_CHECK("attn_decode_cluster_kernel");
  return LRI_OK;
}

// U = positions per row group kept in flight: enough to cover the longest range a CTA can get
// (ceil(smax / ns) positions over NRG row groups) in one pass when that takes at most 12, else 4 per pass.
template <typename T, int HD, int GT>
int launch_u(const ClusterDecodeParams& p, int B, int ns, int tiles, cudaStream_t st) {
  constexpr int NRG = (32 / (HD / 8)) * kClWarps;
  const int64_t longest = (p.smax + ns - 1) / ns;
  const int64_t need = (longest + NRG - 1) / NRG;
  if (need <= 2) return launch_one<T, HD, GT, 2>(p, B, ns, tiles, st);
  if (need <= 4) return launch_one<T, HD, GT, 4>(p, B, ns, tiles, st);
  if (need <= 6) return launch_one<T, HD, GT, 6>(p, B, ns, tiles, st);
  if (need <= 8 && GT <= 2) return launch_one<T, HD, GT, 8>(p, B, ns, tiles, st);
  return launch_one<T, HD, GT, 4>(p, B, ns, tiles, st);
}

template <typename T, int HD>
int launch_hd(const ClusterDecodeParams& p, int B, int ns, cudaStream_t st) {
  const int g = p.n_head / p.n_kv;
  const int gt = attn_decode_cluster_head_tile(B, p.n_kv, g);
  const int tiles = p.n_kv * (g / gt);
  if (gt == 4) return launch_u<T, HD, 4>(p, B, ns, tiles, st);
  if (gt == 2) return launch_u<T, HD, 2>(p, B, ns, tiles, st);
  return launch_u<T, HD, 1>(p, B, ns, tiles, st);
}

}  // namespace

// Query heads of a KV group that one CTA serves (the CTAs of a group's tiles read the same cache rows).
// A thread's time goes into its dot products and their shuffles, GT of each per cache row, so with few
// clusters in the grid (a small shard of one or two sequences) the heads are spread over more clusters
// while at most 4 result: on the 8B shard of 1/8 (one KV head, 4 query heads, context 1152) 16-CTA
// clusters take 5.40 us with 4 heads per CTA, 4.00 us with 2, 3.35 us with 1; on the 1/4 shard 5.41,
// 4.13 and 4.19 us.  LRI_ATTN_HEAD_TILE=1|2|4 overrides.
int attn_decode_cluster_head_tile(int B, int n_kv, int g) {
  const int forced = option(OPT_ATTN_HEAD_TILE);
  if (forced > 0 && g % forced == 0) return forced;
  int gt = (g % 4 == 0) ? 4 : ((g % 2 == 0) ? 2 : 1);
  while (gt > 1 && static_cast<int64_t>(B) * n_kv * (g / (gt / 2)) <= 4) gt /= 2;
  return gt;
}

bool attn_decode_cluster_supports(int num_splits) {
  return option(OPT_ATTN_CLUSTER) != 0 &&
         (num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8 || num_splits == 16);
}

int attn_decode_cluster_launch(int dtype, const void* q, const void* k_cache, const void* v_cache,
                               const void* input_pos, int pos_is_i64, void* out, int B, int n_head, int n_kv,
                               int head_dim, int64_t smax, int num_splits, float scale_log2, cudaStream_t st) {
  ClusterDecodeParams p{};
  p.q = q, p.k_cache = k_cache, p.v_cache = v_cache, p.input_pos = input_pos, p.pos_is_i64 = pos_is_i64, p.out = out;
  p.n_head = n_head, p.n_kv = n_kv, p.smax = smax, p.scale_log2 = scale_log2;
  if (dtype == LRI_BF16)
    return head_dim == 128 ? launch_hd<__nv_bfloat16, 128>(p, B, num_splits, st)
                           : launch_hd<__nv_bfloat16, 64>(p, B, num_splits, st);
  return head_dim == 128 ? launch_hd<__half, 128>(p, B, num_splits, st) : launch_hd<__half, 64>(p, B, num_splits, st);
}

}  // namespace lri
