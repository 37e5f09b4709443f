// Greedy decoding head: LM-head projection of this rank's vocabulary rows fused with the arg-max
// over rows (argmax.cuh), followed by one warp that exchanges the ranks' candidates over NVLink and
// writes the token.  Up to 8 sequences the weight-streaming GEMV folds the candidates in its
// epilogue and no logits are written; for more sequences the logits of the rank's slice come from
// the stream-K projection and a small kernel folds them.
#include <cstddef>

#include "linear.cuh"
#include "p2p_comm.cuh"

namespace lri {
namespace {

constexpr int kRowThreads = 256;
constexpr int kRowChunk = kRowThreads * 8;  // logits per CTA

// Grid (chunks, rows): CTA (c, m) folds logits [c * kRowChunk, ...) of sequence m.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) argmax_rows_kernel(const T* __restrict__ logits, int n, const ArgmaxArgs a) {
  pdl_launch_dependents();
  pdl_wait();  // the logits come from the preceding kernel
  const int m = blockIdx.y;
  const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kRowChunk + threadIdx.x * 8;
  unsigned long long k = 0ull;
  if (i0 < n) {
    const T* row = logits + static_cast<int64_t>(m) * n;
    if (i0 + 8 <= n && (n & 7) == 0) {
      float f[8];
      unpack8<T>(*reinterpret_cast<const uint4*>(row + i0), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const unsigned long long c = argmax_key(f[e], a.index_offset + i0 + e);
        k = c > k ? c : k;
      }
    } else {
      for (int e = 0; e < 8 && i0 + e < n; ++e) {
        const unsigned long long c = argmax_key(Num<T>::to_f(row[i0 + e]), a.index_offset + i0 + e);
        k = c > k ? c : k;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
    k = other > k ? other : k;
  }
  __shared__ unsigned long long part[kRowThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = k;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < kRowThreads / 32; ++w) k = part[w] > k ? part[w] : k;
    argmax_offer(a, m, k);
  }
}

// One warp: the rank's keys are final (every producing CTA has completed); exchange and write the tokens.
__global__ void __launch_bounds__(32) argmax_finish_kernel(const ArgmaxArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  argmax_finish(a);
}

int fill_args(lri_comm* c, int64_t M, int64_t index_offset, int32_t* token_out, void* scratch, size_t scratch_bytes,
              int timeout_ms, ArgmaxArgs* a) {
  LRI_REQUIRE(M >= 1 && M <= kArgmaxMaxRows, LRI_ERR_UNSUPPORTED, "lm_head_argmax: M=%lld outside 1..%d", (long long)M,
              kArgmaxMaxRows);
  LRI_REQUIRE(token_out != nullptr, LRI_ERR_ARG, "lm_head_argmax: token_out is NULL");
  LRI_REQUIRE(scratch != nullptr && aligned16(scratch) && scratch_bytes >= kArgmaxScratchBytes, LRI_ERR_WORKSPACE,
              "lm_head_argmax: scratch of %zu zero-initialised bytes (16-byte aligned) required", kArgmaxScratchBytes);
  LRI_REQUIRE(index_offset >= 0 && index_offset < (1ll << 31), LRI_ERR_ARG, "lm_head_argmax: index_offset=%lld",
              (long long)index_offset);
  *a = ArgmaxArgs{};
  a->keys = static_cast<unsigned long long*>(scratch);
  a->token_out = token_out;
  a->index_offset = index_offset;
  a->rows = static_cast<int>(M);
  a->world = 1;
  if (c != nullptr && c->world > 1) {
    for (int r = 0; r < c->world; ++r) {
      LRI_REQUIRE(c->peer[r] != nullptr, LRI_ERR_ARG, "lm_head_argmax: peer %d is not connected", r);
      a->inbox[r] = c->peer[r];
    }
    uint8_t* ctl = c->local + control_offset(c->world, c->max_bytes);
    a->region_off = ll_region(c->world, c->max_bytes, kHeadRegion);
    a->slot_bytes = kLlSlotBytes;
    a->epoch_ptr = reinterpret_cast<unsigned int*>(ctl + offsetof(Control, chan_epoch)) + kHeadRegion;
    a->status_ptr = reinterpret_cast<int*>(ctl + offsetof(Control, status));
    a->timeout_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull;
    a->world = c->world, a->rank = c->rank;
  }
  return LRI_OK;
}

}  // namespace
}  // namespace lri

using namespace lri;

extern "C" size_t lri_lm_head_argmax_scratch_bytes(void) { return kArgmaxScratchBytes; }

extern "C" int lri_lm_head_argmax(lri_comm* comm, int dtype, const void* x, const void* w, int64_t M, int N, int K,
                                  int64_t index_offset, int32_t* token_out, void* scratch, size_t scratch_bytes,
                                  void* logits_ws, size_t logits_ws_bytes, void* workspace, size_t workspace_bytes,
                                  int timeout_ms, lri_stream_t stream) {
  LRI_REQUIRE(dtype == LRI_BF16 || dtype == LRI_FP16, LRI_ERR_UNSUPPORTED, "lm_head_argmax: dtype %d", dtype);
  LRI_REQUIRE(x != nullptr && (w != nullptr || N == 0), LRI_ERR_ARG, "lm_head_argmax: NULL input");
  LRI_REQUIRE(N >= 0 && K > 0 && K % 8 == 0, LRI_ERR_UNSUPPORTED, "lm_head_argmax: N=%d K=%d (K a positive multiple of 8)", N, K);
  LRI_REQUIRE(aligned16(x) && aligned16(w), LRI_ERR_ALIGN, "lm_head_argmax: x and w must be 16-byte aligned");
  ArgmaxArgs a;
  int rc = fill_args(comm, M, index_offset, token_out, scratch, scratch_bytes, timeout_ms, &a);
  if (rc != LRI_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (N > 0 && M <= kGemvMaxRows) {
    LinearParams p{};
    p.x = x, p.w = w, p.m = static_cast<int>(M), p.n = N, p.k = K;
    p.am = a;
    rc = gemv_launch(dtype, EPI_ARGMAX, p, st);
    if (rc != LRI_OK) return rc;
    LRI_CUDA(launch_pdl(argmax_finish_kernel, dim3(1), dim3(32), 0, st, a));
    LRI_LAUNCH_CHECK("argmax_finish_kernel");
    return LRI_OK;
  }
  // more sequences than the streaming kernel takes (or an empty slice): the logits of the slice first
  if (N > 0) {
    LRI_REQUIRE(logits_ws != nullptr && aligned16(logits_ws) && logits_ws_bytes >= static_cast<size_t>(M) * N * 2,
                LRI_ERR_WORKSPACE, "lm_head_argmax: M=%lld > %d needs a logits buffer of %zu bytes (16-byte aligned)",
                (long long)M, kGemvMaxRows, static_cast<size_t>(M) * N * 2);
    rc = lri_linear(dtype, x, w, nullptr, logits_ws, M, N, K, workspace, workspace_bytes, stream);
    if (rc != LRI_OK) return rc;
  }
  const dim3 grid(static_cast<unsigned>(N > 0 ? (N + kRowChunk - 1) / kRowChunk : 1), static_cast<unsigned>(M));
  if (dtype == LRI_BF16)
    LRI_CUDA(launch_pdl(argmax_rows_kernel<__nv_bfloat16>, grid, dim3(kRowThreads), 0, st,
                        static_cast<const __nv_bfloat16*>(logits_ws), N, a));
  else
    LRI_CUDA(launch_pdl(argmax_rows_kernel<__half>, grid, dim3(kRowThreads), 0, st, static_cast<const __half*>(logits_ws),
                        N, a));
  LRI_LAUNCH_CHECK("argmax_rows_kernel");
  LRI_CUDA(launch_pdl(argmax_finish_kernel, dim3(1), dim3(32), 0, st, a));
  LRI_LAUNCH_CHECK("argmax_finish_kernel");
  return LRI_OK;
}
