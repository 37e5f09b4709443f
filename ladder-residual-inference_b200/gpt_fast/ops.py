"""The fused device operations of the decode/prefill step as Python callables over the C ABI.

`CudaOps` is the only implementation the package ships; it needs liblri_b200.so and CUDA
tensors and raises otherwise.  The engine takes the ops object as a parameter so that host-side
schedule logic can be exercised by tests with a stand-in.
"""
import os

import torch

from . import _C


class CudaOps:
    name = "sm_100a"

    # ---- F1 and embedding -----------------------------------------------------------------
    @staticmethod
    def embedding(table, idx, out):
        _C.require_cuda(table, idx, out)
        if idx.dtype not in (torch.int32, torch.int64):
            idx = idx.to(torch.int64)
        idx = idx.contiguous()
        n = idx.numel()
        _C.check(_C.lib.lri_embedding(_C.dtype_code(table.dtype), table.data_ptr(), idx.data_ptr(),
                                      int(idx.dtype == torch.int64), out.data_ptr(), n, table.shape[1],
                                      table.shape[0], _C.stream_handle()))

    @staticmethod
    def add_rmsnorm(residual, add1, add2, weight, eps, residual_out, normed_out, rows, scale=1.0):
        _C.require_cuda(residual)
        dim = residual.shape[-1]
        _C.check(_C.lib.lri_add_rmsnorm(_C.dtype_code(residual.dtype), residual.data_ptr(), _C.ptr(add1), _C.ptr(add2),
                                        float(scale), _C.ptr(weight), float(eps), _C.ptr(residual_out),
                                        _C.ptr(normed_out), rows, dim, _C.stream_handle()))

    # ---- linear family -----------------------------------------------------------------------
    @staticmethod
    def linear(x, w, out, rows, addend=None, workspace=None):
        _C.require_cuda(x, w, out)
        n, k = w.shape
        ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        _C.check(_C.lib.lri_linear(_C.dtype_code(x.dtype), x.data_ptr(), w.data_ptr(), _C.ptr(addend), out.data_ptr(),
                                   rows, n, k, ws_ptr, ws_bytes, _C.stream_handle()))

    @staticmethod
    def linear_workspace_bytes(rows, n):
        return _C.lib.lri_linear_workspace_bytes(rows, n)

    @staticmethod
    def qkv_workspace_bytes(rows, n_head, n_kv, head_dim):
        return _C.lib.lri_qkv_workspace_bytes(rows, n_head, n_kv, head_dim)

    @staticmethod
    def gateup_workspace_bytes(rows, inter):
        return _C.lib.lri_gateup_workspace_bytes(rows, inter)

    @staticmethod
    def qkv_rope_kvcache(x, wqkv, table, table_gathered, input_pos, q_out, k_cache, v_cache, B, S, n_head, n_kv,
                         head_dim, workspace):
        _C.require_cuda(x, wqkv, table, input_pos, q_out, k_cache, v_cache)
        assert input_pos.dtype in (torch.int32, torch.int64)
        k = wqkv.shape[1]
        smax = k_cache.shape[2]
        ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        _C.check(_C.lib.lri_qkv_rope_kvcache(
            _C.dtype_code(x.dtype), x.data_ptr(), wqkv.data_ptr(), table.data_ptr(), input_pos.data_ptr(),
            int(input_pos.dtype == torch.int64), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), B, S, k,
            n_head, n_kv, head_dim, smax, table.shape[0], int(table_gathered), ws_ptr, ws_bytes, _C.stream_handle()))

    @staticmethod
    def gateup_swiglu(x, w1, h, rows, workspace):
        _C.require_cuda(x, w1, h)
        two_i, k = w1.shape
        ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        _C.check(_C.lib.lri_gateup_swiglu(_C.dtype_code(x.dtype), x.data_ptr(), w1.data_ptr(), h.data_ptr(), rows,
                                          two_i // 2, k, ws_ptr, ws_bytes, _C.stream_handle()))

    # ---- attention ---------------------------------------------------------------------------------
    @staticmethod
    def attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits):
        return _C.lib.lri_attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits)

    @staticmethod
    def attention(q, k_cache, v_cache, input_pos, out, B, S, n_head, n_kv, head_dim, scratch, num_splits):
        _C.require_cuda(q, k_cache, v_cache, input_pos, out)
        code = _C.dtype_code(q.dtype)
        smax = k_cache.shape[2]
        i64 = int(input_pos.dtype == torch.int64)
        if S == 1:
            _C.check(_C.lib.lri_attn_decode(code, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            input_pos.data_ptr(), i64, out.data_ptr(), B, n_head, n_kv, head_dim,
                                            smax, num_splits, scratch.data_ptr(),
                                            scratch.numel() * scratch.element_size(), _C.stream_handle()))
        else:
            _C.check(_C.lib.lri_attn_prefill(code, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                             input_pos.data_ptr(), i64, out.data_ptr(), B, S, n_head, n_kv, head_dim,
                                             smax, _C.stream_handle()))


def decode_splits(B, n_head, n_kv, smax, sm_count=148, head_dim=128):
    """Number of sequence ranges for decode attention, fixed per cache geometry so that the launch
    grid never depends on the current position.  Up to 8 ranges (a power of two) run as one
    thread-block cluster and merge through shared memory; that form is kept as long as a CTA
    then streams at most ~1 MB of K/V.  Longer caches take more ranges (up to 64, at least 64
    positions each) and merge through the scratch buffer."""
    forced = os.environ.get("LRI_DECODE_SPLITS")  # tuning knob
    if forced:
        return max(1, min(64, int(forced), max(1, smax // 32)))
    g = n_head // n_kv
    mma = os.environ.get("LRI_ATTN_MMA")
    if g <= 16 and (mma == "1" or (mma is None and B * n_kv >= 128)):
        # tensor-core kernel (one CTA per sequence, KV head and range; two CTAs per SM): a second
        # range only while one range per pair would leave SMs without work; more ranges cost more
        # in the merge than they gain
        return 2 if (B * n_kv < 2 * sm_count and smax >= 256) else 1
    gt = 4 if g % 4 == 0 else (2 if g % 2 == 0 else 1)
    base = max(1, B * n_kv * (g // gt))
    want = max(1, -(-2 * sm_count // base))
    bytes_per_cta_at_8 = smax * head_dim * 2 * 2 / 8
    if want <= 8 or bytes_per_cta_at_8 <= (1 << 20):
        n = 1
        while n * 2 <= min(want, 8) and smax // (n * 2) >= 32:
            n *= 2
        return n
    return int(max(1, min(want, 64, max(1, smax // 64))))
