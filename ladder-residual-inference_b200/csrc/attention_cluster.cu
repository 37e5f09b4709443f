// F3, low-latency form: GQA decode attention whose sequence splits are the CTAs of one
// thread-block cluster and are merged through distributed shared memory.
//
// At decode batch sizes the K/V bytes of one layer are a few MB, so the kernel is a chain of
// memory round trips, not a bandwidth problem.  The split-K form that goes through global
// scratch pays for: partial store, fence, atomic ticket, two rounds of partial loads.  Here the
// num_splits (1, 2, 4 or 8) CTAs that share a (batch, kv-head tile) form a cluster; each leaves
// its (max, sum, weighted values) in its own shared memory, the cluster synchronises once, and
// every CTA merges one slice of the output elements by reading its peers' shared memory.
// No scratch memory, no counters, and the grid still does not depend on the position.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace lri {
namespace {

constexpr int kClWarps = 8;
constexpr int kClThreads = kClWarps * 32;
constexpr int kClUnroll = 4;

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

template <typename T, int HD, int GT>
__global__ void __launch_bounds__(kClThreads, 2) attn_decode_cluster_kernel(const ClusterDecodeParams p) {
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

  __shared__ float sm_m[NRG][GT];
  __shared__ float sm_l[NRG][GT];
  __shared__ float sm_o[NRG][GT][HD];
  // this CTA's merged result, read by the peers of the cluster
  __shared__ __align__(16) float c_o[GT][HD];
  __shared__ float c_m[GT];
  __shared__ float c_l[GT];

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
  const T* kbase = static_cast<const T*>(p.k_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;
  const T* vbase = static_cast<const T*>(p.v_cache) + (static_cast<int64_t>(b) * p.n_kv + kvh) * p.smax * HD + sl * 8;

  float m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
  }

  // Warp-uniform trip count (all 32 lanes run the shuffles); rows past the end are clamped and masked.
  for (int64_t jb = p0 + warp * RPW; jb < p1; jb += static_cast<int64_t>(NRG) * kClUnroll) {
    uint4 kv[kClUnroll], vv[kClUnroll];
    bool valid[kClUnroll];
#pragma unroll
    for (int t = 0; t < kClUnroll; ++t) {
      const int64_t j = jb + lane / LPR + static_cast<int64_t>(t) * NRG;
      valid[t] = j < p1;
      const int64_t jc = valid[t] ? j : p1 - 1;
      kv[t] = ld_stream16(kbase + jc * HD);
      vv[t] = ld_stream16(vbase + jc * HD);
    }
    float s[kClUnroll][GT];
#pragma unroll
    for (int t = 0; t < kClUnroll; ++t) {
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
      for (int t = 1; t < kClUnroll; ++t) mx = fmaxf(mx, s[t][h]);
      const float m_new = fmaxf(m[h], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;  // no valid position yet: exponentials give 0
      const float corr = exp2f(m[h] - m_use);
      l[h] *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
      m[h] = m_new;
#pragma unroll
      for (int t = 0; t < kClUnroll; ++t) s[t][h] = exp2f(s[t][h] - m_use);
    }
#pragma unroll
    for (int t = 0; t < kClUnroll; ++t) {
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

  // ---- merge the row groups of this CTA into c_m / c_l / c_o -----------------------------------------
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
  for (int idx = threadIdx.x; idx < GT * HD; idx += kClThreads) {
    const int h = idx / HD, e = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < NRG; ++r) mm = fmaxf(mm, sm_m[r][h]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int r = 0; r < NRG; ++r) {
        const float w = exp2f(sm_m[r][h] - mm);
        ll += sm_l[r][h] * w;
        oo += sm_o[r][h][e] * w;
      }
    }
    c_o[h][e] = oo;
    if (e == 0) {
      c_m[h] = mm;
      c_l[h] = ll;
    }
  }
  cluster.sync();  // every CTA's result is in its shared memory and visible to the cluster

  // ---- each CTA merges one slice of the GT*HD output elements over all splits -------------------------
  const int per_cta = GT * HD / ns;  // ns is 1, 2, 4 or 8 and divides GT*HD
  for (int i = threadIdx.x; i < per_cta; i += kClThreads) {
    const int idx = split * per_cta + i;
    const int h = idx / HD, e = idx % HD;
    float pm[8], pl[8], po[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < ns) {
        pm[r] = *cluster.map_shared_rank(&c_m[h], r);
        pl[r] = *cluster.map_shared_rank(&c_l[h], r);
        po[r] = *cluster.map_shared_rank(&c_o[h][e], r);
      } else {
        pm[r] = -INFINITY;
        pl[r] = 0.f;
        po[r] = 0.f;
      }
    }
    float mm = pm[0];
#pragma unroll
    for (int r = 1; r < 8; ++r) mm = fmaxf(mm, pm[r]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float w = exp2f(pm[r] - mm);
        ll += pl[r] * w;
        oo += po[r] * w;
      }
    }
    const float res = ll > 0.f ? oo / ll : 0.f;
    static_cast<T*>(p.out)[(static_cast<int64_t>(b) * p.n_head + head0 + h) * HD + e] = Num<T>::from_f(res);
  }
  cluster.sync();  // keep this CTA's shared memory alive until every peer has read it
}

template <typename T, int HD, int GT>
int launch_one(const ClusterDecodeParams& p, int B, int ns, int tiles, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ns, tiles, B);
  cfg.blockDim = dim3(kClThreads);
  cfg.dynamicSmemBytes = 0;
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
  LRI_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel<T, HD, GT>, p));
  LRI_LAUNCH_CHECK("attn_decode_cluster_kernel");
  return LRI_OK;
}

template <typename T, int HD>
int launch_hd(const ClusterDecodeParams& p, int B, int ns, cudaStream_t st) {
  const int g = p.n_head / p.n_kv;
  const int gt = (g % 4 == 0) ? 4 : ((g % 2 == 0) ? 2 : 1);
  const int tiles = p.n_kv * (g / gt);
  if (gt == 4) return launch_one<T, HD, 4>(p, B, ns, tiles, st);
  if (gt == 2) return launch_one<T, HD, 2>(p, B, ns, tiles, st);
  return launch_one<T, HD, 1>(p, B, ns, tiles, st);
}

}  // namespace

bool attn_decode_cluster_supports(int num_splits) {
  return option(OPT_ATTN_CLUSTER) != 0 && (num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8);
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
