/*
 * lri_b200.h - C ABI of the B200 (sm_100a) kernels behind the tensor-parallel decode/prefill step.
 *
 * The reference project is pure Python (its kernels are library calls and one Triton kernel),
 * so it has no FFI of its own; each entry point below names the reference code it replaces
 * (paths relative to the reference repository root).  A Python binding (ctypes) passes
 * `tensor.data_ptr()` values and the raw handle of the current CUDA stream.
 *
 * Conventions
 *   - Plain pointers and sizes only.  Every pointer is a DEVICE pointer unless it says "host".
 *   - The caller owns all memory.  No entry point allocates device memory or synchronises the
 *     device unless its comment says so; work is enqueued on `stream`.
 *   - `dtype` is LRI_BF16 or LRI_FP16 (activations, weights and caches share it); all
 *     accumulation is fp32 and results are rounded once to `dtype` where the reference's
 *     nn.Linear / elementwise op would round.
 *   - Matrices are row-major.  Weights have the nn.Linear layout [out_features, in_features].
 *   - Positions are read on the device from `input_pos` (int32 when pos_is_i64 == 0, int64
 *     otherwise), never from a host scalar, so a captured CUDA graph stays valid when the caller
 *     advances the position tensor in place (benchmark.py:209-217).
 *   - Return value: LRI_OK or a negative lri_status; lri_last_error() gives the message of the
 *     calling thread's last failure.  The reference's convention is a Python assert/exception
 *     (gpt_fast/utils.py:52, 155-162); the binding raises RuntimeError on a negative status.
 */
#ifndef LRI_B200_H_
#define LRI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* lri_stream_t; /* a cudaStream_t */

enum lri_dtype { LRI_BF16 = 0, LRI_FP16 = 1 };

enum lri_status {
  LRI_OK = 0,
  LRI_ERR_ARG = -1,         /* null pointer, non-positive extent, inconsistent sizes */
  LRI_ERR_ALIGN = -2,       /* pointer or row pitch not aligned as the kernel needs */
  LRI_ERR_UNSUPPORTED = -3, /* shape or dtype outside what the kernels are built for */
  LRI_ERR_CUDA = -4,        /* a CUDA runtime/driver call failed (message has the CUDA text) */
  LRI_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  LRI_ERR_TIMEOUT = -6,     /* a bounded device-side wait gave up (peer flag, mbarrier) */
  LRI_ERR_NO_DEVICE = -7    /* no usable sm_100 device */
};

/* GEMM back end for M > 8 rows.  AUTO picks tcgen05 when the shape allows it. */
enum lri_gemm_backend { LRI_GEMM_AUTO = 0, LRI_GEMM_TCGEN05 = 1, LRI_GEMM_SIMT = 2 };

const char* lri_last_error(void);
int lri_version(void);
/* Selects the GEMM back end used by the linear-layer entry points (process-wide). */
int lri_set_gemm_backend(int backend);
/* Tuning options: one table per process, each entry initialised from an LRI_* environment variable
 * at first use and changeable at run time; a change applies from the next launch on.  Names (initial
 * value from): stream_rows (LRI_STREAM_ROWS, 1..16, token rows up to which the weight-streaming
 * kernels run), gemv_simt (LRI_GEMV_SMALL=simt), gemv_rows_per_cta (LRI_GEMV_R: 0, 2, 4, 8),
 * gemv_depth (LRI_GEMV_U: 0, 2), gemv_mma_tiles (LRI_GEMV_MT: 0, 1, 2, 4), gemm_group
 * (LRI_GEMM_GROUP), fused_prefill (LRI_FUSED_PREFILL: 0, 1), pdl (LRI_PDL: 0, 1), attn_cluster
 * (LRI_ATTN_CLUSTER: 0, 1), attn_mma (LRI_ATTN_MMA: -1 choose, 0, 1), decode_splits
 * (LRI_DECODE_SPLITS: 0 choose, 1..64), attn_prefill_tc (LRI_ATTN_PREFILL_TC: 0 mma.sync kernel, 1 tcgen05
 * kernel), gemm_reserve_sms (LRI_GEMM_RESERVE_SMS: SMs
 * the persistent prefill GEMM leaves free for a collective running beside it, 0..64), attn_head_tile
 * (LRI_ATTN_HEAD_TILE: query heads of a KV group per CTA of the cluster decode attention, 0 choose, 1, 2, 4).  Unknown
 * names and values an option does not take return LRI_ERR_ARG.  No counterpart in the reference
 * (its only switches are benchmark.py's command-line flags). */
int lri_set_option(const char* name, int value);
int lri_get_option(const char* name, int* value_out);
/* Number of kernels this library has launched from the calling process so far. */
int64_t lri_launch_count(void);
/* The tcgen05 GEMM bounds every mbarrier wait; a wait that gives up records its site in a
 * device status word.  Reads and clears it (synchronous copy): LRI_OK or LRI_ERR_TIMEOUT. */
int lri_gemm_status(void);

/* ---- F1: residual add + RMSNorm -------------------------------------------------------
 * residual_out = round(round(residual * residual_scale) + add1) [+ add2, rounded again];
 * normed_out   = round(residual_out * rsqrt(mean(residual_out^2) + eps)) * weight.
 * add1, add2 may be NULL (no add); weight/normed_out may be NULL (add only); residual_out may
 * be NULL (norm only) or alias residual.  residual_scale != 1 is the desync block's x / tp.
 * Replaces: the Triton add kernel gpt_fast/gpt_ladder_TP.py:364-377 (launched :331, :348),
 * the final three-way add gpt_ladder_TP.py:280, RMSNorm.forward gpt_fast/utils.py:62-78 and
 * the `y + x / tp_world_size` of gpt_fast/gpt_desync_TP.py:366-382. */
int lri_add_rmsnorm(int dtype, const void* residual, const void* add1, const void* add2,
                    float residual_scale, const void* weight, float eps, void* residual_out,
                    void* normed_out, int64_t rows, int dim, lri_stream_t stream);

/* ---- embedding gather ------------------------------------------------------------------
 * out[i, :] = table[idx[i], :].  idx is int64 when idx_is_i64 != 0, else int32.
 * Replaces: self.tok_embeddings(idx), gpt_fast/gpt_ladder_TP.py:256. */
int lri_embedding(int dtype, const void* table, const void* idx, int idx_is_i64, void* out,
                  int64_t n_tokens, int dim, int64_t vocab, lri_stream_t stream);

/* ---- F5 / F7: linear layer y = x W^T (+ addend) ------------------------------------------
 * x [M, K], w [N, K], y [M, N].  addend (may be NULL) is added after y's own rounding and the
 * sum rounded again (the parallel block's `w2(...) + y`, gpt_fast/utils.py:385).  M <= 8 runs
 * the weight-streaming kernels (SIMT for one row, mma.sync for 2..8); larger M the tcgen05 GEMM.
 * For 8 < M <= 64 a workspace of lri_linear_workspace_bytes(M, N) bytes (16-byte aligned) selects
 * the tcgen05 stream-K kernel: all SMs stream equal shares of the weight, fp32 partial tiles go
 * to the workspace and the CTA that completes a tile sums them and applies the addend.  With
 * NULL or a smaller workspace the plain GEMM runs.  Two calls that may run at the same time on
 * different streams need different workspaces; at most 16 stream-K kernels (this entry point,
 * lri_qkv_rope_kvcache, lri_gateup_swiglu) may be in flight at once.  Replaces: self.wo / self.w2 / self.output nn.Linear calls, gpt_fast/utils.py:148,
 * 258, 384-385 and gpt_fast/gpt_ladder_TP.py:283. */
size_t lri_linear_workspace_bytes(int64_t M, int N);
/* How the stream-K kernel would cut a projection with N outputs (for lri_gateup_swiglu: N = I) and
 * depth K at 1 <= M <= 64 token rows: 128-output tiles, 64-element K tiles, the number of
 * persistent CTAs, the most segments one tile may be cut into (the workspace holds that many
 * fp32 partial tiles of token_tile x 128 per tile) and the token tile 16 / 32 / 64.  Host
 * arithmetic only, usable without a GPU.  No counterpart in the reference. */
int lri_streamk_plan(int64_t M, int N, int K, int* tiles, int* k_tiles, int* max_segments, int* ctas,
                     int* token_tile);
int lri_linear(int dtype, const void* x, const void* w, const void* addend, void* y, int64_t M,
               int N, int K, void* workspace, size_t workspace_bytes, lri_stream_t stream);

/* ---- F2: QKV projection + RoPE + KV-cache write ----------------------------------------
 * x [B*S, K]; wqkv [(n_head + 2 n_kv) * head_dim, K] with rows [q heads | k heads | v heads];
 * rope_table [table_rows, head_dim/2, 2] = (cos, sin) in `dtype`; input_pos [S].  The table row
 * of token s is input_pos[s], or s itself when table_gathered != 0 (the caller already indexed
 * the table by position, as the reference's forward does: freqs_cis[input_pos]).
 * q_out [B, S, n_head, head_dim] receives the rotated queries; rotated keys and the values are
 * written to k_cache / v_cache [B_max, n_kv, smax, head_dim] at [b, h, input_pos[s], :].
 * Rotation is over adjacent pairs in fp32 from the rounded projection, as the reference does.
 * A position outside [0, min(smax, table_rows)) is skipped (nothing is written for it).
 * M = B*S > 8 needs workspace of lri_qkv_workspace_bytes(M, n_head, n_kv, head_dim) bytes.
 * Replaces: gpt_fast/utils.py:187-198 (wqkv, split, apply_rotary_emb) and KVCache.update
 * utils.py:50-59, 249-250. */
size_t lri_qkv_workspace_bytes(int64_t M, int n_head, int n_kv, int head_dim);
int lri_qkv_rope_kvcache(int dtype, const void* x, const void* wqkv, const void* rope_table,
                         const void* input_pos, int pos_is_i64, void* q_out, void* k_cache,
                         void* v_cache, int B, int S, int K, int n_head, int n_kv, int head_dim,
                         int64_t smax, int64_t table_rows, int table_gathered, void* workspace,
                         size_t workspace_bytes, lri_stream_t stream);

/* ---- F6: gate/up projection + SwiGLU -----------------------------------------------------
 * w1 [2*I, K] with rows [up (I rows) | gate (I rows)]; h[m, j] = round(silu(gate_j)) * up_j.
 * M > 8 needs workspace of lri_gateup_workspace_bytes(M, I) bytes.
 * Replaces: FeedForward.forward's w1 / chunk / silu*mul, gpt_fast/utils.py:145-148 (and the
 * u, g part of FuseAttentionMLP, utils.py:311-313, 385). */
size_t lri_gateup_workspace_bytes(int64_t M, int I);
int lri_gateup_swiglu(int dtype, const void* x, const void* w1, void* h, int64_t M, int I, int K,
                      void* workspace, size_t workspace_bytes, lri_stream_t stream);

/* ---- F3: GQA decode attention, split over the sequence --------------------------------------
 * One query token per sequence.  q [B, n_head, head_dim]; caches [B_max, n_kv, smax, head_dim];
 * context = positions 0..input_pos[0] inclusive (the new key is already in the cache); query
 * head h reads kv head h / (n_head / n_kv); scale 1/sqrt(head_dim); out [B, n_head*head_dim].
 * The sequence is cut into num_splits ranges handled by different CTAs and merged by the last
 * CTA to finish, so the grid does not depend on the position.  scratch: at least
 * lri_attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits) bytes, 16-byte aligned;
 * its first 32768 bytes are arrival counters that must be zero before the first call
 * (each call leaves them zero).  Calls sharing one scratch must not overlap on the device.
 * Three kernels serve this entry point: with 1, 2, 4, 8 or 16 ranges and fewer than 128 (sequence,
 * KV head) pairs the ranges are the CTAs of one thread-block cluster and merge through
 * distributed shared memory (scratch untouched); from 128 pairs on (and n_head / n_kv <= 16) a
 * tensor-core kernel takes the query heads of a KV head as the rows of mma tiles and merges the
 * ranges through the scratch; other range counts use the SIMT scratch kernel.
 * Replaces: the decode case of gpt_fast/utils.py:252-255 (repeat_interleave + SDPA over the
 * whole cache under mask = causal_mask[input_pos]). */
size_t lri_attn_decode_scratch_bytes(int B, int n_head, int n_kv, int head_dim, int num_splits);
/* The num_splits the library recommends for a cache geometry (host arithmetic on the SM count of the
 * current device, 148 without one; honours the decode_splits and attn_mma options): fixed per
 * geometry so that a captured graph stays valid as the position grows. */
int lri_attn_decode_plan(int B, int n_head, int n_kv, int head_dim, int64_t smax, int* num_splits);
int lri_attn_decode(int dtype, const void* q, const void* k_cache, const void* v_cache,
                    const void* input_pos, int pos_is_i64, void* out, int B, int n_head, int n_kv,
                    int head_dim, int64_t smax, int num_splits, void* scratch,
                    size_t scratch_bytes, lri_stream_t stream);

/* lri_attn_decode_static: the same kernel and arguments as lri_attn_decode, minus the scratch
 * pointer.  (No counterpart in the reference: it exists for callers of THIS library that may not
 * allocate - a plug-in that receives only tensors and a stream from its host framework, or a
 * server whose device memory is fixed before traffic starts and where a cudaMalloc, which
 * synchronises the device, must never happen while requests are in flight.)  The split partials
 * and counters live in an 8 MiB array built into the library
 * (lri_attn_decode_static_scratch_capacity()), held by every GPU that loads it until the process
 * ends.  A configuration needing more (lri_attn_decode_scratch_bytes(...) > capacity) is refused
 * with LRI_ERR_WORKSPACE.  Nothing is allocated or freed, here or in anything it calls.
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  All calls on a device share the one array:
 * two calls that overlap on the GPU (different streams) corrupt each other; calls in one stream
 * are fine, and each call leaves the counters at zero for the next. */
size_t lri_attn_decode_static_scratch_capacity(void);
int lri_attn_decode_static(int dtype, const void* q, const void* k_cache, const void* v_cache,
                           const void* input_pos, int pos_is_i64, void* out, int B, int n_head,
                           int n_kv, int head_dim, int64_t smax, int num_splits,
                           lri_stream_t stream);

/* ---- F4: causal GQA prefill attention --------------------------------------------------------
 * q [B, S, n_head, head_dim]; query s has position input_pos[0] + s (positions must be
 * consecutive, as in the reference's only caller, benchmark.py:138) and attends cache positions
 * 0..input_pos[0]+s.  out [B, S, n_head*head_dim].
 * Replaces: the prefill case of gpt_fast/utils.py:252-257. */
int lri_attn_prefill(int dtype, const void* q, const void* k_cache, const void* v_cache,
                     const void* input_pos, int pos_is_i64, void* out, int B, int S, int n_head,
                     int n_kv, int head_dim, int64_t smax, lri_stream_t stream);

/* ---- F8: all-reduce over peer memory (one process per GPU) -----------------------------------
 * A communicator owns, on every rank, one inbox buffer that all peers can write.  One-shot
 * all-reduce: every rank stores its partial into slot `rank` of each peer's inbox, then raises
 * a per-peer flag; the consumer waits (bounded) for all flags of the current epoch and sums
 * the slots in fp32.  The wait gives up after `timeout_ms` and records LRI_ERR_TIMEOUT
 * in a device status word that lri_comm_status() reads; it never traps and never spins forever.
 *
 * lri_comm_create: allocates the local inbox with cudaMalloc (the one allocation this library
 *   makes; it synchronises) and returns an opaque handle plus a 64-byte IPC handle to send
 *   to the peers.  max_elems = largest message in elements; slots are double buffered.
 * lri_comm_connect: `ipc_handles` = world*64 bytes gathered from all ranks (host memory).
 * lri_allreduce: in-place-capable SUM of `count` elements of `dtype`; out = sum over ranks of
 *   their `in`.  Epochs advance from a device-resident counter, so graph replays stay correct.
 * Replaces: all_reduce_func / dist.all_reduce, gpt_fast/utils.py:390-397. */
typedef struct lri_comm lri_comm;
int lri_comm_create(int rank, int world, int64_t max_elems, lri_comm** comm_out,
                    unsigned char ipc_handle_out[64]);
int lri_comm_connect(lri_comm* comm, const unsigned char* ipc_handles /* host, world*64 */);
int lri_allreduce(lri_comm* comm, int dtype, const void* in, void* out, int64_t count,
                  int timeout_ms, lri_stream_t stream);
/* Split form of the all-reduce for small messages (up to lri_comm_push_max_elems() elements): the
 * producer pushes its partial into the peers' inboxes right after the row-parallel projection
 * (lri_comm_push, channel 1 or 2, each with its own device-resident epoch), and the reduction
 * happens inside the consumer: lri_add_rmsnorm_gather is lri_add_rmsnorm whose addend k is, when
 * channel_k > 0, the SUM over ranks of the message last pushed on that channel (add_k then points
 * to this rank's own partial; rank-order fp32 sum, rounded once, bit-identical on all ranks) and,
 * when channel_k == 0, a plain addend pointer or NULL.  No reduce kernel and no stream fork: an
 * all-reduce costs one small push kernel.  A rank must consume message n of a channel before it
 * pushes message n+1 on it (the consumer advances the channel's epoch; two buffers per channel),
 * which every schedule here does; all ranks push the same sequence.  The consumer's wait is bounded by timeout_ms (status word as above).
 * Replaces: all_reduce_func + the residual add + RMSNorm that follow it,
 * gpt_fast/gpt_ladder_TP.py:323-356, gpt_fast/gpt_dense_TP.py:281-282.
 * lri_linear_push is lri_linear (decode, M <= 8) whose epilogue also pushes: every finished
 * output pair goes to the peers as an 8-byte {2 elements, epoch} half line, so the transfer
 * overlaps the tail of the projection and no push kernel is launched (the fused
 * compute + collective form of the row-parallel projections wo / w2). */
int64_t lri_comm_push_max_elems(void);
int lri_linear_push(lri_comm* comm, int channel, int dtype, const void* x, const void* w,
                    const void* addend, void* y, int64_t M, int N, int K, lri_stream_t stream);
int lri_comm_push(lri_comm* comm, int channel, int dtype, const void* in, int64_t count,
                  lri_stream_t stream);
int lri_add_rmsnorm_gather(lri_comm* comm, int dtype, const void* residual, int channel1,
                           const void* add1, int channel2, const void* add2, float residual_scale,
                           const void* weight, float eps, void* residual_out, void* normed_out,
                           int64_t rows, int dim, int timeout_ms, lri_stream_t stream);
/* lri_add_rmsnorm_allreduce: the whole all-reduce inside the consumer.  Same arguments and result as
 * lri_add_rmsnorm_gather, but nothing is pushed beforehand: every thread of the kernel first stores
 * the elements of this rank's partial(s) it is about to sum into the peers' inboxes and then polls
 * for theirs, so all-reduce + residual add + RMSNorm cost one launch on the consuming stream (no
 * all-reduce kernel, no communication stream, no event hop).  Channels, epochs, message limit and
 * ordering rule are those of the push channels; a channel carries either pushed or self-pushed
 * messages, all ranks alike.
 * Replaces: all_reduce_func + residual add + RMSNorm, gpt_fast/gpt_ladder_TP.py:323-356. */
int lri_add_rmsnorm_allreduce(lri_comm* comm, int dtype, const void* residual, int channel1,
                              const void* add1, int channel2, const void* add2, float residual_scale,
                              const void* weight, float eps, void* residual_out, void* normed_out,
                              int64_t rows, int dim, int timeout_ms, lri_stream_t stream);
/* ---- greedy decoding head: LM-head projection + arg-max over vocabulary rows and ranks ---------
 * token_out[m] (int32) = index of the largest logit of sequence m over the whole vocabulary, lowest
 * index on ties, where this rank holds rows [index_offset, index_offset + N) of the output projection
 * (w [N, K]) and the other ranks of `comm` hold the rest; comm == NULL: one rank.  Logits are compared
 * as the projection would store them (fp32 sums rounded to `dtype`).  M <= 8: the weight-streaming
 * kernel folds its candidates in its epilogue (one 64-bit key per sequence in `scratch`) and writes no
 * logits.  8 < M <= 64: the slice's logits go to logits_ws (M*N elements) through lri_linear (workspace
 * as there) and a small kernel folds them.  In both cases one warp launched behind the producer
 * exchanges one 16-byte line per sequence with every peer over NVLink (bounded wait: timeout_ms, status
 * word read by lri_comm_status) and writes the winner.
 * scratch: lri_lm_head_argmax_scratch_bytes() bytes, 16-byte aligned, zero before the first call;
 * every call leaves it zero.  All ranks must call with the same M; N may be 0 on a rank whose slice
 * is empty.  Every rank writes the same tokens.
 * Replaces: the output projection + sampling at top_k = 1 / arg-max of the logits,
 * gpt_fast/gpt_ladder_TP.py:282-283 with benchmark.py:56-77, 86-92. */
size_t lri_lm_head_argmax_scratch_bytes(void);
int lri_lm_head_argmax(lri_comm* comm, int dtype, const void* x, const void* w, int64_t M, int N, int K,
                       int64_t index_offset, int32_t* token_out, void* scratch, size_t scratch_bytes,
                       void* logits_ws, size_t logits_ws_bytes, void* workspace, size_t workspace_bytes,
                       int timeout_ms, lri_stream_t stream);
/* Reads (and clears) the device status word: LRI_OK or LRI_ERR_TIMEOUT.  Synchronises `stream`. */
int lri_comm_status(lri_comm* comm, lri_stream_t stream);
int lri_comm_destroy(lri_comm* comm);

#ifdef __cplusplus
}
#endif
#endif /* LRI_B200_H_ */
