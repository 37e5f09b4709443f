// Shared device/host helpers for the sm_100a kernels: dtype traits, 16-byte vector access,
// error reporting of the C ABI, launch counting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "lri_b200.h"

namespace lri {

// ---- host side ---------------------------------------------------------------------------
// Formats the calling thread's error message and returns `code`.
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);

#define LRI_REQUIRE(cond, code, ...)                  \
  do {                                                \
    if (!(cond)) return ::lri::fail(code, __VA_ARGS__); \
  } while (0)

#define LRI_CUDA(expr)                                                                        \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess)                                                                    \
      return ::lri::fail(LRI_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                         __FILE__, __LINE__);                                                 \
  } while (0)

// After a kernel launch: reports a launch-configuration error without synchronising.
#define LRI_LAUNCH_CHECK(what)                                                                 \
  do {                                                                                         \
    cudaError_t e_ = cudaPeekAtLastError();                                                    \
    if (e_ != cudaSuccess) {                                                                   \
      cudaGetLastError();                                                                      \
      return ::lri::fail(LRI_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e_)); \
    }                                                                                          \
    ::lri::count_launch();                                                                     \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- tuning options ----------------------------------------------------------------------------
// One table per process.  Every entry starts from its LRI_* environment variable (read once, at the
// first use of any option) and can be changed at run time through lri_set_option(); the kernels'
// launch code reads the table on every call, so a change takes effect on the next launch.
enum Option {
  OPT_STREAM_ROWS = 0,  // LRI_STREAM_ROWS    token rows up to which the weight-streaming kernels run (1..16, default 8)
  OPT_GEMV_SIMT,        // LRI_GEMV_SMALL=simt  keep the SIMT streaming kernel for 2..8 rows (default 0)
  OPT_GEMV_R,           // LRI_GEMV_R         weight rows per CTA of the SIMT streaming kernel: 2, 4 or 8 (0 = choose)
  OPT_GEMV_U,           // LRI_GEMV_U         2 halves the loads in flight per thread of that kernel (0 = default)
  OPT_GEMV_MT,          // LRI_GEMV_MT        row tiles per CTA of the tensor-core streaming kernel: 1, 2, 4 (0 = choose)
  OPT_GEMM_GROUP,       // LRI_GEMM_GROUP     token tiles per panel of the prefill GEMM's tile walk (0 = choose)
  OPT_FUSED_PREFILL,    // LRI_FUSED_PREFILL  0: prefill projections run the plain GEMM + an elementwise epilogue
  OPT_PDL,              // LRI_PDL            0: no programmatic dependent launch
  OPT_ATTN_CLUSTER,     // LRI_ATTN_CLUSTER   0: decode attention never takes the thread-block-cluster kernel
  OPT_ATTN_MMA,         // LRI_ATTN_MMA       1 / 0 forces / forbids the tensor-core decode-attention kernel (-1 = choose)
  OPT_DECODE_SPLITS,    // LRI_DECODE_SPLITS  fixed number of sequence ranges for decode attention (0 = choose)
  OPT_ATTN_PREFILL_TC,  // LRI_ATTN_PREFILL_TC  0: prefill attention on the mma.sync kernel; 1: tcgen05 / TMEM kernel (default)
  OPT_GEMM_RESERVE_SMS, // LRI_GEMM_RESERVE_SMS  SMs the persistent prefill GEMM leaves free (for a collective running beside it)
  OPT_ATTN_HEAD_TILE,   // LRI_ATTN_HEAD_TILE  query heads per CTA of the cluster decode-attention kernel: 1, 2, 4 (0 = choose)
  OPT_COUNT
};
int option(int which);

// ---- per-device state -------------------------------------------------------------------------------
// Function attributes (dynamic shared memory size) and the SM count belong to a device, not to the
// process: one-time set-up is keyed by the ordinal of the device that is current at the call.
int current_device();    // ordinal of the current device, -1 when the runtime cannot tell
int device_sm_count();   // multiprocessors of the current device (148 when the runtime cannot tell)
// LRI_ONCE_PER_DEVICE(seen, call): runs a CUDA runtime call the first time the enclosing launch code
// is used on the current device (and again after a failure); `seen` is a static atomic bit set with one
// bit per device ordinal.  Ordinals outside 0..63 repeat the call every time, which is harmless.
inline bool device_setup_needed(const std::atomic<unsigned long long>& seen) {
  const int dev = current_device();
  return dev < 0 || dev >= 64 || (seen.load(std::memory_order_acquire) & (1ull << dev)) == 0;
}
inline void device_setup_done(std::atomic<unsigned long long>& seen) {
  const int dev = current_device();
  if (dev >= 0 && dev < 64) seen.fetch_or(1ull << dev, std::memory_order_release);
}
#define LRI_ONCE_PER_DEVICE(seen, call)      \
  do {                                       \
    if (::lri::device_setup_needed(seen)) {  \
      LRI_CUDA(call);                        \
      ::lri::device_setup_done(seen);        \
    }                                        \
  } while (0)

// Programmatic dependent launch.  Kernels of the decode step are launched with the
// programmatic-stream-serialization attribute: a kernel may start while its predecessor in the
// stream is still draining, runs the part of its prologue that does not depend on the
// predecessor (address set-up, streaming the first weight vectors) and then blocks in
// pdl_wait() until the predecessor has completed and its writes are visible.  Every kernel
// launched this way calls pdl_wait() before it reads or writes anything another kernel touches.
// LRI_PDL=0 in the environment turns the attribute off (the device-side calls become no-ops).
bool pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- dtype traits ------------------------------------------------------------------------
template <typename T>
struct Num;

template <>
struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float f) { return __float2bfloat16_rn(f); }
  // two packed elements (low half first) to two floats
  static __device__ __forceinline__ void unpack2(uint32_t u, float& lo, float& hi) {
    lo = __uint_as_float(u << 16);
    hi = __uint_as_float(u & 0xffff0000u);
  }
};

template <>
struct Num<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float f) { return __float2half_rn(f); }
  static __device__ __forceinline__ void unpack2(uint32_t u, float& lo, float& hi) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
  }
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  Num<T>::unpack2(v.x, f[0], f[1]);
  Num<T>::unpack2(v.y, f[2], f[3]);
  Num<T>::unpack2(v.z, f[4], f[5]);
  Num<T>::unpack2(v.w, f[6], f[7]);
}

// two floats rounded (to nearest even) to T and packed, `lo` in the low half: one paired conversion
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack2<T>(f[0], f[1]);
  v.y = pack2<T>(f[2], f[3]);
  v.z = pack2<T>(f[4], f[5]);
  v.w = pack2<T>(f[6], f[7]);
  return v;
}

// round-trip through the storage type: the value an op's output has after it is stored
template <typename T>
__device__ __forceinline__ float rnd(float f) {
  return Num<T>::to_f(Num<T>::from_f(f));
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 16-byte streaming load that does not allocate in L1 (weights are read exactly once)
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ int64_t load_pos(const void* input_pos, int pos_is_i64, int64_t i) {
  return pos_is_i64 ? reinterpret_cast<const int64_t*>(input_pos)[i]
                    : static_cast<int64_t>(reinterpret_cast<const int32_t*>(input_pos)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 2^x by the special-function unit alone (no range fix-up: arguments here are <= 8, and results below
// the smallest normal number may flush to zero)
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// SiLU as torch evaluates it in fp32: x / (1 + exp(-x))
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// silu(gate) rounded to T, times up (both already rounded to T), rounded to T.
template <typename T>
__device__ __forceinline__ T swiglu_rounded(float up_rounded, float gate_rounded) {
  float s = rnd<T>(silu_f(gate_rounded));
  return Num<T>::from_f(s * up_rounded);
}

// Rotation of one adjacent pair in fp32 with separately rounded products (no FMA
// contraction), from values and table entries already rounded to T.
__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, float& o0, float& o1) {
  o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
  o1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
}

}  // namespace lri
