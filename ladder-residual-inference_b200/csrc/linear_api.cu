// C entry points of the linear-layer family (F2, F5, F6, F7): argument checks, the choice
// between the decode GEMV and the prefill GEMM, the elementwise epilogues that follow the
// GEMM (RoPE + cache scatter, SwiGLU, addend), and a plain SIMT GEMM kept as a selectable
// back end for shapes the tcgen05 kernel does not take.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "linear.cuh"

namespace lri {

bool gemm_tcgen05_supports(int64_t m, int n, int k);
int gemm_tcgen05_launch(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st);
int gemm_tcgen05_status_read_and_clear(int* status_out);
int attn_prefill_tc_status_read_and_clear(int* status_out);
bool gemm_tcgen05_fused_supports(int epi, const LinearParams& p, int64_t m);
int gemm_tcgen05_fused_launch(int dtype, int epi, const LinearParams& p, int64_t m, cudaStream_t st);

// ---- error text, launch counter, options --------------------------------------------------------
namespace {
thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};

struct OptionSpec {
  const char* name;  // as given to lri_set_option / lri_get_option
  const char* env;   // environment variable that supplies the initial value
  int def, lo, hi;
};
// order = enum Option (common.cuh)
const OptionSpec kOptionSpecs[OPT_COUNT] = {
    {"stream_rows", "LRI_STREAM_ROWS", 8, 1, kGemvMmaMaxRows},
    {"gemv_simt", "LRI_GEMV_SMALL", 0, 0, 1},
    {"gemv_rows_per_cta", "LRI_GEMV_R", 0, 0, 8},
    {"gemv_depth", "LRI_GEMV_U", 0, 0, 2},
    {"gemv_mma_tiles", "LRI_GEMV_MT", 0, 0, 4},
    {"gemm_group", "LRI_GEMM_GROUP", 0, 0, 1024},
    {"fused_prefill", "LRI_FUSED_PREFILL", 1, 0, 1},
    {"pdl", "LRI_PDL", 1, 0, 1},
    {"attn_cluster", "LRI_ATTN_CLUSTER", 1, 0, 1},
    {"attn_mma", "LRI_ATTN_MMA", -1, -1, 1},
    {"decode_splits", "LRI_DECODE_SPLITS", 0, 0, 64},
    {"attn_prefill_tc", "LRI_ATTN_PREFILL_TC", 1, 0, 1},
    {"gemm_reserve_sms", "LRI_GEMM_RESERVE_SMS", 0, 0, 64},
    {"attn_head_tile", "LRI_ATTN_HEAD_TILE", 0, 0, 4},
};

bool option_value_ok(int which, int v) {
  const OptionSpec& s = kOptionSpecs[which];
  if (v < s.lo || v > s.hi) return false;
  if (which == OPT_GEMV_R) return v == 0 || v == 2 || v == 4 || v == 8;
  if (which == OPT_GEMV_U) return v == 0 || v == 2;
  if (which == OPT_GEMV_MT) return v == 0 || v == 1 || v == 2 || v == 4;
  if (which == OPT_ATTN_HEAD_TILE) return v == 0 || v == 1 || v == 2 || v == 4;
  return true;
}

struct OptionTable {
  std::atomic<int> v[OPT_COUNT];
  OptionTable() {
    for (int i = 0; i < OPT_COUNT; ++i) {
      int val = kOptionSpecs[i].def;
      const char* e = getenv(kOptionSpecs[i].env);
      if (e && *e) {
        const int parsed = (i == OPT_GEMV_SIMT) ? (strcmp(e, "simt") == 0 ? 1 : 0) : atoi(e);
        // out-of-range numbers are clamped (what the variables did before they became options)
        int c = parsed < kOptionSpecs[i].lo ? kOptionSpecs[i].lo : (parsed > kOptionSpecs[i].hi ? kOptionSpecs[i].hi : parsed);
        if (option_value_ok(i, c)) val = c;
      }
      v[i].store(val);
    }
  }
};
OptionTable& options() {
  static OptionTable t;
  return t;
}

// LRI_GEMM_BACKEND=simt|tcgen05 in the environment sets the initial choice (debugging aid).
int backend_from_env() {
  const char* e = getenv("LRI_GEMM_BACKEND");
  if (e && strcmp(e, "simt") == 0) return LRI_GEMM_SIMT;
  if (e && strcmp(e, "tcgen05") == 0) return LRI_GEMM_TCGEN05;
  return LRI_GEMM_AUTO;
}
std::atomic<int> g_backend{backend_from_env()};
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int option(int which) { return (which >= 0 && which < OPT_COUNT) ? options().v[which].load(std::memory_order_relaxed) : 0; }
bool pdl_enabled() { return option(OPT_PDL) != 0; }

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}
int device_sm_count() {
  static std::atomic<int> cache[64];
  const int dev = current_device();
  if (dev >= 0 && dev < 64) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int v = 0;
  if (dev < 0 || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
    cudaGetLastError();
    return 148;
  }
  if (dev < 64) cache[dev].store(v, std::memory_order_relaxed);
  return v;
}

// Token rows up to which the weight-streaming kernels (no workspace) are used; more rows go to the
// tcgen05 GEMM (measured cross-over on B200: the streaming kernels win up to 8 rows).
int streaming_rows() { return option(OPT_STREAM_ROWS); }
// Option fused_prefill = 0 keeps the prefill projections on the plain GEMM followed by an elementwise
// kernel (debugging aid; also what runs for shapes the fused epilogues do not take).
bool fused_prefill_epilogues() { return option(OPT_FUSED_PREFILL) != 0; }
bool prefer_simt_gemv() { return option(OPT_GEMV_SIMT) != 0; }
int current_gemm_backend() { return g_backend.load(); }

namespace {

// ---- SIMT GEMM: 64x64 tile, 256 threads, 4x4 outputs per thread, fp32 accumulation --------------
constexpr int kST = 64, kSK = 32, kSLd = kST + 4;

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ w,
                                                        T* __restrict__ c, int m, int n, int k) {
  __shared__ float as[kSK][kSLd];
  __shared__ float ws[kSK][kSLd];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kST, n0 = static_cast<int64_t>(blockIdx.x) * kST;
  const int lrow = tid >> 2, lk = (tid & 3) * 8;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += kSK) {
    float fa[8] = {}, fw[8] = {};
    if (m0 + lrow < m && k0 + lk < k) unpack8<T>(*reinterpret_cast<const uint4*>(a + (m0 + lrow) * k + k0 + lk), fa);
    if (n0 + lrow < n && k0 + lk < k) unpack8<T>(*reinterpret_cast<const uint4*>(w + (n0 + lrow) * k + k0 + lk), fw);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      as[lk + e][lrow] = fa[e];
      ws[lk + e][lrow] = fw[e];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&as[kk][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t r = m0 + ty * 4 + i, col = n0 + tx * 4 + j;
      if (r < m && col < n) c[r * n + col] = Num<T>::from_f(acc[i][j]);
    }
}

template <typename T>
int launch_simt(const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st) {
  dim3 grid(static_cast<unsigned>((n + kST - 1) / kST), static_cast<unsigned>((m + kST - 1) / kST));
  gemm_simt_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(w), static_cast<T*>(c),
                                            static_cast<int>(m), n, k);
  LRI_LAUNCH_CHECK("gemm_simt_kernel");
  return LRI_OK;
}

// ---- elementwise epilogues after the GEMM -----------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const T* __restrict__ ug, T* __restrict__ h, int64_t m,
                                                          int n) {
  // one thread per 8 outputs; ug row = [up (n) | gate (n)]
  const int64_t vec_per_row = n >> 3;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= m * vec_per_row) return;
  const int64_t row = i / vec_per_row, v = i - row * vec_per_row;
  const uint4* src = reinterpret_cast<const uint4*>(ug + row * 2 * n);
  float u[8], g[8], o[8];
  unpack8<T>(src[v], u);
  unpack8<T>(src[vec_per_row + v], g);
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = rnd<T>(silu_f(g[e])) * u[e];
  reinterpret_cast<uint4*>(h + row * n)[v] = pack8<T>(o);
}

template <typename T>
__global__ void __launch_bounds__(256) qkv_scatter_kernel(const T* __restrict__ qkv, const LinearParams p) {
  // one thread per adjacent pair of the projection output
  const int64_t width = static_cast<int64_t>(p.n_head + 2 * p.n_kv) * p.head_dim;
  const int64_t pairs_per_row = width >> 1;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(p.m) * pairs_per_row) return;
  const int64_t row = i / pairs_per_row, n = (i - row * pairs_per_row) * 2;
  float v0, v1;
  Num<T>::unpack2(*reinterpret_cast<const uint32_t*>(qkv + row * width + n), v0, v1);
  qkv_epilogue_pair<T>(p, row, n, v0, v1);
}

template <typename T>
__global__ void __launch_bounds__(256) add_rows_kernel(T* __restrict__ y, const T* __restrict__ addend,
                                                       int64_t nvec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  float a[8], b[8];
  unpack8<T>(reinterpret_cast<const uint4*>(y)[i], a);
  unpack8<T>(reinterpret_cast<const uint4*>(addend)[i], b);
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] += b[e];
  reinterpret_cast<uint4*>(y)[i] = pack8<T>(a);
}

unsigned blocks_for(int64_t items, int threads) { return static_cast<unsigned>((items + threads - 1) / threads); }

}  // namespace

int gemm_launch(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st) {
  const int backend = current_gemm_backend();
  const bool tc_ok = gemm_tcgen05_supports(m, n, k) && aligned16(a) && aligned16(w) && aligned16(c);
  if (backend == LRI_GEMM_TCGEN05 && !tc_ok)
    return fail(LRI_ERR_UNSUPPORTED, "gemm: tcgen05 back end needs n %% 8 == 0, k %% 8 == 0 and 16-byte aligned pointers");
  if (backend != LRI_GEMM_SIMT && tc_ok) return gemm_tcgen05_launch(dtype, a, w, c, m, n, k, st);
  return dtype == LRI_BF16 ? launch_simt<__nv_bfloat16>(a, w, c, m, n, k, st)
                           : launch_simt<__half>(a, w, c, m, n, k, st);
}

// The stream-K path serves token rows above the streaming kernels and up to kSplitKMaxRows.
static bool streamk_rows(int64_t M) {
  return M > streaming_rows() && M <= kSplitKMaxRows && current_gemm_backend() != LRI_GEMM_SIMT;
}
static size_t streamk_bytes(int epi, int64_t M, int64_t n) {
  return (M > streaming_rows() && M <= kSplitKMaxRows && n < (1ll << 31)) ? gemm_streamk_workspace_bytes(epi, M, static_cast<int>(n)) : 0;
}
static size_t max_size(size_t a, size_t b) { return a > b ? a : b; }

int swiglu_rows_launch(int dtype, const void* ug, void* h, int64_t m, int n, cudaStream_t st) {
  const int64_t items = m * (n >> 3);
  if (dtype == LRI_BF16)
    swiglu_rows_kernel<__nv_bfloat16><<<blocks_for(items, 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(ug), static_cast<__nv_bfloat16*>(h), m, n);
  else
    swiglu_rows_kernel<__half><<<blocks_for(items, 256), 256, 0, st>>>(static_cast<const __half*>(ug),
                                                                        static_cast<__half*>(h), m, n);
  LRI_LAUNCH_CHECK("swiglu_rows_kernel");
  return LRI_OK;
}

int qkv_scatter_launch(int dtype, const void* qkv, const LinearParams& p, cudaStream_t st) {
  const int64_t items = static_cast<int64_t>(p.m) * ((static_cast<int64_t>(p.n_head + 2 * p.n_kv) * p.head_dim) >> 1);
  if (dtype == LRI_BF16)
    qkv_scatter_kernel<__nv_bfloat16><<<blocks_for(items, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(qkv), p);
  else
    qkv_scatter_kernel<__half><<<blocks_for(items, 256), 256, 0, st>>>(static_cast<const __half*>(qkv), p);
  LRI_LAUNCH_CHECK("qkv_scatter_kernel");
  return LRI_OK;
}

int add_rows_launch(int dtype, void* y, const void* addend, int64_t count, cudaStream_t st) {
  const int64_t nvec = count >> 3;
  if (dtype == LRI_BF16)
    add_rows_kernel<__nv_bfloat16><<<blocks_for(nvec, 256), 256, 0, st>>>(
        static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(addend), nvec);
  else
    add_rows_kernel<__half><<<blocks_for(nvec, 256), 256, 0, st>>>(static_cast<__half*>(y),
                                                                    static_cast<const __half*>(addend), nvec);
  LRI_LAUNCH_CHECK("add_rows_kernel");
  return LRI_OK;
}

}  // namespace lri

// ---- C ABI ----------------------------------------------------------------------------------------
using namespace lri;

extern "C" const char* lri_last_error(void) { return g_err; }
extern "C" int lri_version(void) { return 100; }
extern "C" int64_t lri_launch_count(void) { return g_launches.load(); }
extern "C" int lri_set_gemm_backend(int backend) {
  LRI_REQUIRE(backend >= LRI_GEMM_AUTO && backend <= LRI_GEMM_SIMT, LRI_ERR_ARG, "set_gemm_backend: %d", backend);
  g_backend.store(backend);
  return LRI_OK;
}
extern "C" int lri_set_option(const char* name, int value) {
  LRI_REQUIRE(name != nullptr, LRI_ERR_ARG, "set_option: NULL name");
  for (int i = 0; i < OPT_COUNT; ++i)
    if (strcmp(name, kOptionSpecs[i].name) == 0) {
      LRI_REQUIRE(option_value_ok(i, value), LRI_ERR_ARG, "set_option: %s=%d is outside %d..%d (or not a value it takes)",
                  name, value, kOptionSpecs[i].lo, kOptionSpecs[i].hi);
      options().v[i].store(value);
      return LRI_OK;
    }
  return fail(LRI_ERR_ARG, "set_option: unknown option '%s'", name);
}
extern "C" int lri_get_option(const char* name, int* value_out) {
  LRI_REQUIRE(name != nullptr && value_out != nullptr, LRI_ERR_ARG, "get_option: NULL argument");
  for (int i = 0; i < OPT_COUNT; ++i)
    if (strcmp(name, kOptionSpecs[i].name) == 0) {
      *value_out = option(i);
      return LRI_OK;
    }
  return fail(LRI_ERR_ARG, "get_option: unknown option '%s'", name);
}
extern "C" int lri_gemm_status(void) {
  int v = 0, v2 = 0, v3 = 0;
  int rc = gemm_tcgen05_status_read_and_clear(&v);
  if (rc != LRI_OK) return rc;
  rc = gemm_streamk_status_read_and_clear(&v2);
  if (rc != LRI_OK) return rc;
  rc = attn_prefill_tc_status_read_and_clear(&v3);
  if (rc != LRI_OK) return rc;
  if (v != 0 || v2 != 0)
    return fail(LRI_ERR_TIMEOUT, "tcgen05 GEMM: a bounded mbarrier wait gave up (site %d)", v != 0 ? v : v2);
  if (v3 != 0) return fail(LRI_ERR_TIMEOUT, "tcgen05 prefill attention: a bounded mbarrier wait gave up (site %d)", v3);
  return LRI_OK;
}

static int check_common(const char* who, int dtype, const void* x, const void* w, int64_t M, int K) {
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "%s: dtype %d", who, dtype);
  LRI_REQUIRE(x && w, LRI_ERR_ARG, "%s: NULL input", who);
  LRI_REQUIRE(M >= 0 && M < (1ll << 31), LRI_ERR_ARG, "%s: M=%lld", who, (long long)M);
  LRI_REQUIRE(K > 0 && K % 8 == 0, LRI_ERR_UNSUPPORTED, "%s: K=%d must be a positive multiple of 8", who, K);
  LRI_REQUIRE(aligned16(x) && aligned16(w), LRI_ERR_ALIGN, "%s: x and w must be 16-byte aligned", who);
  return LRI_OK;
}

extern "C" int lri_linear(int dtype, const void* x, const void* w, const void* addend, void* y, int64_t M, int N,
                          int K, void* workspace, size_t workspace_bytes, lri_stream_t stream) {
  int rc = check_common("linear", dtype, x, w, M, K);
  if (rc != LRI_OK) return rc;
  LRI_REQUIRE(y != nullptr && N > 0, LRI_ERR_ARG, "linear: y is NULL or N=%d", N);
  if (M == 0) return LRI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M <= streaming_rows()) {
    LinearParams p{};
    p.x = x, p.w = w, p.y = y, p.addend = addend, p.m = static_cast<int>(M), p.n = N, p.k = K;
    return streaming_launch(dtype, EPI_PLAIN, p, st, prefer_simt_gemv());
  }
  if (streamk_rows(M)) {
    LinearParams p{};
    p.x = x, p.w = w, p.y = y, p.addend = addend, p.m = static_cast<int>(M), p.n = N, p.k = K;
    if (gemm_streamk_supports(EPI_PLAIN, p, workspace, workspace_bytes))
      return gemm_streamk_launch(dtype, EPI_PLAIN, p, workspace, workspace_bytes, st);
  }
  if (M <= kGemvMmaMaxRows) {  // no usable workspace: the streaming kernel takes up to 16 rows
    LinearParams p{};
    p.x = x, p.w = w, p.y = y, p.addend = addend, p.m = static_cast<int>(M), p.n = N, p.k = K;
    return streaming_launch(dtype, EPI_PLAIN, p, st, prefer_simt_gemv());
  }
  rc = gemm_launch(dtype, x, w, y, M, N, K, st);
  if (rc != LRI_OK || addend == nullptr) return rc;
  LRI_REQUIRE((M * N) % 8 == 0 && aligned16(y) && aligned16(addend), LRI_ERR_ALIGN,
              "linear: addend path needs M*N %% 8 == 0 and 16-byte aligned y, addend");
  return add_rows_launch(dtype, y, addend, M * N, st);
}

extern "C" int lri_streamk_plan(int64_t M, int N, int K, int* tiles, int* k_tiles, int* max_segments, int* ctas,
                                int* token_tile) {
  LRI_REQUIRE(M >= 1 && M <= kSplitKMaxRows && N >= 1 && K >= 1, LRI_ERR_ARG, "streamk_plan: M=%lld N=%d K=%d",
              (long long)M, N, K);
  LRI_REQUIRE(tiles && k_tiles && max_segments && ctas && token_tile, LRI_ERR_ARG, "streamk_plan: NULL output");
  gemm_streamk_plan(EPI_PLAIN, M, N, K, tiles, k_tiles, max_segments, ctas, token_tile);
  return LRI_OK;
}

extern "C" size_t lri_linear_workspace_bytes(int64_t M, int N) { return M < 0 || N <= 0 ? 0 : streamk_bytes(EPI_PLAIN, M, N); }

static size_t gateup_raw_bytes(int64_t M, int I) {
  return M <= kGemvMmaMaxRows ? 0 : static_cast<size_t>(M) * 2 * static_cast<size_t>(I) * 2;
}
extern "C" size_t lri_gateup_workspace_bytes(int64_t M, int I) {
  return max_size(gateup_raw_bytes(M, I), streamk_bytes(EPI_SWIGLU, M, I));
}

extern "C" int lri_gateup_swiglu(int dtype, const void* x, const void* w1, void* h, int64_t M, int I, int K,
                                 void* workspace, size_t workspace_bytes, lri_stream_t stream) {
  int rc = check_common("gateup_swiglu", dtype, x, w1, M, K);
  if (rc != LRI_OK) return rc;
  LRI_REQUIRE(h != nullptr && I > 0, LRI_ERR_ARG, "gateup_swiglu: h is NULL or I=%d", I);
  if (M == 0) return LRI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LinearParams p{};
  p.x = x, p.w = w1, p.y = h, p.m = static_cast<int>(M), p.n = I, p.k = K;
  if (M <= streaming_rows()) return streaming_launch(dtype, EPI_SWIGLU, p, st, prefer_simt_gemv());
  if (streamk_rows(M) && gemm_streamk_supports(EPI_SWIGLU, p, workspace, workspace_bytes))
    return gemm_streamk_launch(dtype, EPI_SWIGLU, p, workspace, workspace_bytes, st);
  // no usable workspace: the streaming kernel takes up to 16 rows
  if (M <= kGemvMmaMaxRows) return streaming_launch(dtype, EPI_SWIGLU, p, st, prefer_simt_gemv());
  LRI_REQUIRE(I % 8 == 0, LRI_ERR_UNSUPPORTED, "gateup_swiglu: I=%d must be a multiple of 8 for M > %d", I, kGemvMmaMaxRows);
  // prefill: SwiGLU applied from the accumulator, no workspace needed
  if (M > kSplitKMaxRows && current_gemm_backend() != LRI_GEMM_SIMT && fused_prefill_epilogues() &&
      gemm_tcgen05_fused_supports(EPI_SWIGLU, p, M))
    return gemm_tcgen05_fused_launch(dtype, EPI_SWIGLU, p, M, st);
  LRI_REQUIRE(workspace && workspace_bytes >= gateup_raw_bytes(M, I) && aligned16(workspace) && aligned16(h),
              LRI_ERR_WORKSPACE, "gateup_swiglu: workspace of %zu bytes (16-byte aligned) required",
              lri_gateup_workspace_bytes(M, I));
  rc = gemm_launch(dtype, x, w1, workspace, M, 2 * I, K, st);
  if (rc != LRI_OK) return rc;
  return swiglu_rows_launch(dtype, workspace, h, M, I, st);
}

static size_t qkv_raw_bytes(int64_t M, int n_head, int n_kv, int head_dim) {
  return M <= kGemvMmaMaxRows ? 0 : static_cast<size_t>(M) * static_cast<size_t>(n_head + 2 * n_kv) * head_dim * 2;
}
extern "C" size_t lri_qkv_workspace_bytes(int64_t M, int n_head, int n_kv, int head_dim) {
  return max_size(qkv_raw_bytes(M, n_head, n_kv, head_dim),
                  streamk_bytes(EPI_QKV, M, static_cast<int64_t>(n_head + 2 * n_kv) * head_dim));
}

extern "C" int lri_qkv_rope_kvcache(int dtype, const void* x, const void* wqkv, const void* rope_table,
                                    const void* input_pos, int pos_is_i64, void* q_out, void* k_cache, void* v_cache,
                                    int B, int S, int K, int n_head, int n_kv, int head_dim, int64_t smax,
                                    int64_t table_rows, int table_gathered, void* workspace,
                                    size_t workspace_bytes, lri_stream_t stream) {
  LRI_REQUIRE(B >= 0 && S >= 0, LRI_ERR_ARG, "qkv_rope_kvcache: B=%d S=%d", B, S);
  const int64_t M = static_cast<int64_t>(B) * S;
  int rc = check_common("qkv_rope_kvcache", dtype, x, wqkv, M, K);
  if (rc != LRI_OK) return rc;
  LRI_REQUIRE(rope_table && input_pos && q_out && k_cache && v_cache, LRI_ERR_ARG, "qkv_rope_kvcache: NULL pointer");
  LRI_REQUIRE(n_head > 0 && n_kv > 0 && head_dim > 0 && head_dim % 8 == 0, LRI_ERR_UNSUPPORTED,
              "qkv_rope_kvcache: n_head=%d n_kv=%d head_dim=%d (head_dim must be a multiple of 8)", n_head, n_kv,
              head_dim);
  LRI_REQUIRE(smax > 0 && table_rows > 0, LRI_ERR_ARG, "qkv_rope_kvcache: smax=%lld table_rows=%lld", (long long)smax,
              (long long)table_rows);
  LRI_REQUIRE(aligned16(q_out) && aligned16(k_cache) && aligned16(v_cache) && aligned16(rope_table), LRI_ERR_ALIGN,
              "qkv_rope_kvcache: outputs and table must be 16-byte aligned");
  if (M == 0) return LRI_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LinearParams p{};
  p.x = x, p.w = wqkv, p.m = static_cast<int>(M), p.n = (n_head + 2 * n_kv) * head_dim, p.k = K;
  p.rope_table = rope_table, p.input_pos = input_pos, p.pos_is_i64 = pos_is_i64;
  p.q_out = q_out, p.k_cache = k_cache, p.v_cache = v_cache;
  p.S = S, p.n_head = n_head, p.n_kv = n_kv, p.head_dim = head_dim, p.smax = smax, p.table_rows = table_rows, p.table_gathered = table_gathered;
  if (M <= streaming_rows()) return streaming_launch(dtype, EPI_QKV, p, st, prefer_simt_gemv());
  if (streamk_rows(M) && gemm_streamk_supports(EPI_QKV, p, workspace, workspace_bytes))
    return gemm_streamk_launch(dtype, EPI_QKV, p, workspace, workspace_bytes, st);
  // no usable workspace: the streaming kernel takes up to 16 rows
  if (M <= kGemvMmaMaxRows) return streaming_launch(dtype, EPI_QKV, p, st, prefer_simt_gemv());
  // prefill: RoPE + cache write from the accumulator
  if (M > kSplitKMaxRows && current_gemm_backend() != LRI_GEMM_SIMT && fused_prefill_epilogues() &&
      gemm_tcgen05_fused_supports(EPI_QKV, p, M))
    return gemm_tcgen05_fused_launch(dtype, EPI_QKV, p, M, st);
  LRI_REQUIRE(workspace && workspace_bytes >= qkv_raw_bytes(M, n_head, n_kv, head_dim) && aligned16(workspace),
              LRI_ERR_WORKSPACE, "qkv_rope_kvcache: workspace of %zu bytes (16-byte aligned) required",
              lri_qkv_workspace_bytes(M, n_head, n_kv, head_dim));
  rc = gemm_launch(dtype, x, wqkv, workspace, M, p.n, K, st);
  if (rc != LRI_OK) return rc;
  return qkv_scatter_launch(dtype, workspace, p, st);
}
