// Parameters and epilogue code shared by the GEMV (decode) and GEMM (prefill) linear kernels.
#pragma once

#include "argmax.cuh"
#include "common.cuh"

namespace lri {

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_QKV = 2, EPI_ARGMAX = 3 };
constexpr int kGemvMaxRows = 8;

// Producer side of the split all-reduce, fused into the epilogue of a row-parallel projection:
// every finished output pair is also stored, as an 8-byte half line {2 elements, epoch}, into slot
// `rank` of every peer's inbox on a push channel.  The epoch is the channel's count of consumed
// messages plus one; the consumer (the gathering add + RMSNorm) advances the count.
struct PushArgs {
  uint8_t* inbox[8];              // every rank's inbox as mapped by this rank
  const unsigned int* epoch_ptr;  // this rank's counter of consumed messages on the channel
  size_t region_off;              // offset of the channel's line region inside an inbox
  int64_t slot_bytes;             // bytes of one (buffer, source rank) slot
  int world, rank, enabled;
};

struct LinearParams {
  const void* x;  // [m, k]
  const void* w;  // PLAIN/QKV: [n, k]; SWIGLU: [2n, k] = [up rows | gate rows]
  void* y;        // PLAIN: [m, n]; SWIGLU: [m, n]; QKV: unused
  const void* addend;
  int m, n, k;
  // QKV epilogue
  const void* rope_table;  // [table_rows, head_dim/2, 2]
  const void* input_pos;   // [S]
  int pos_is_i64;
  void* q_out;    // [B, S, n_head, head_dim]
  void* k_cache;  // [B_max, n_kv, smax, head_dim]
  void* v_cache;
  int S, n_head, n_kv, head_dim;
  int64_t smax, table_rows;
  int table_gathered;  // rope_table row s belongs to token s (rows already gathered by position)
  PushArgs push;       // PLAIN epilogue of the SIMT kernel only
  ArgmaxArgs am;       // ARGMAX epilogue of the SIMT kernel: greedy choice instead of stored logits
};

// Epilogue of the QKV projection for token row `m` and the adjacent output pair (n, n+1),
// n even, values already rounded to T: rotate q / k pairs with the table row of the token's
// position and scatter to q_out / k_cache / v_cache.
template <typename T>
__device__ __forceinline__ void qkv_epilogue_pair(const LinearParams& p, int64_t m, int64_t n, float v0, float v1) {
  const int hd = p.head_dim;
  const int64_t nq = static_cast<int64_t>(p.n_head) * hd;
  const int64_t nk = static_cast<int64_t>(p.n_kv) * hd;
  const int64_t b = m / p.S;
  const int64_t s = m - b * p.S;
  const int64_t pos = load_pos(p.input_pos, p.pos_is_i64, s);
  const int64_t trow = p.table_gathered ? s : pos;
  if (pos < 0 || pos >= p.smax || trow >= p.table_rows) return;
  const T* table = static_cast<const T*>(p.rope_table);
  if (n < nq + nk) {
    const int64_t nn = n < nq ? n : n - nq;
    const int e = static_cast<int>(nn % hd);
    const T* cs = table + (trow * (hd >> 1) + (e >> 1)) * 2;
    float o0, o1;
    rope_pair(v0, v1, Num<T>::to_f(cs[0]), Num<T>::to_f(cs[1]), o0, o1);
    T* dst;
    if (n < nq) {
      dst = static_cast<T*>(p.q_out) + m * nq + n;
    } else {
      const int64_t h = nn / hd;
      dst = static_cast<T*>(p.k_cache) + ((b * p.n_kv + h) * p.smax + pos) * hd + e;
    }
    *reinterpret_cast<uint32_t*>(dst) = pack2<T>(o0, o1);
  } else {
    const int64_t nn = n - nq - nk;
    const int64_t h = nn / hd;
    const int e = static_cast<int>(nn % hd);
    T* dst = static_cast<T*>(p.v_cache) + ((b * p.n_kv + h) * p.smax + pos) * hd + e;
    *reinterpret_cast<uint32_t*>(dst) = pack2<T>(v0, v1);
  }
}

// decode path, 1 <= p.m <= 8 (SIMT FMA)
int gemv_launch(int dtype, int epi, const LinearParams& p, cudaStream_t st);
// decode path, 1 <= p.m <= 16 (same streaming, tensor-core FMA)
constexpr int kGemvMmaMaxRows = 16;
int gemv_mma_launch(int dtype, int epi, const LinearParams& p, cudaStream_t st);
// Rows up to which the streaming kernels (no workspace) are used, and which of the two runs:
// one row -> SIMT kernel, 2..16 rows -> tensor-core kernel (LRI_GEMV_SMALL=simt keeps the SIMT
// kernel up to 8 rows).
inline int streaming_launch(int dtype, int epi, const LinearParams& p, cudaStream_t st, bool prefer_simt) {
  if (p.m == 1 || (prefer_simt && p.m <= kGemvMaxRows)) return gemv_launch(dtype, epi, p, st);
  return gemv_mma_launch(dtype, epi, p, st);
}
bool prefer_simt_gemv();

// C[m, n] = A[m, k] * W[n, k]^T, C in `dtype`, any m.  backend: lri_gemm_backend.
int gemm_launch(int dtype, const void* a, const void* w, void* c, int64_t m, int n, int k, cudaStream_t st);

// Small-batch decode above the streaming kernels (up to kSplitKMaxRows token rows): a tcgen05
// stream-K GEMM with the weights as the 128-row operand, fp32 partial tiles in a workspace and
// the projection's epilogue applied by the CTA that completes a tile (gemm_streamk.cu).
// lin.n counts outputs (SWIGLU: the weight has 2 * lin.n rows).
constexpr int kMaxSplitK = 8;
constexpr int kSplitKMaxRows = 64;
size_t gemm_streamk_workspace_bytes(int epi, int64_t m, int n);
bool gemm_streamk_supports(int epi, const LinearParams& lin, const void* workspace, size_t workspace_bytes);
int gemm_streamk_launch(int dtype, int epi, const LinearParams& lin, void* workspace, size_t workspace_bytes,
                        cudaStream_t st);
int gemm_streamk_status_read_and_clear(int* status_out);
void gemm_streamk_plan(int epi, int64_t m, int n, int k, int* tiles, int* k_tiles, int* max_seg, int* ctas,
                       int* token_tile_out);

// elementwise epilogues used after the GEMM on the prefill path
int swiglu_rows_launch(int dtype, const void* ug /*[m, 2n]*/, void* h /*[m, n]*/, int64_t m, int n, cudaStream_t st);
int qkv_scatter_launch(int dtype, const void* qkv /*[m, (nh+2nkv)*hd]*/, const LinearParams& p, cudaStream_t st);
int add_rows_launch(int dtype, void* y, const void* addend, int64_t count, cudaStream_t st);

int current_gemm_backend();

}  // namespace lri
