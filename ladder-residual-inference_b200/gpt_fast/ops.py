"""The fused device operations of the decode/prefill step as Python callables over the C ABI.

`CudaOps` is the only implementation the package ships; it needs liblri_b200.so and CUDA
tensors and raises otherwise.  The engine takes the ops object as a parameter so that host-side
schedule logic can be exercised by tests with a stand-in.
"""
import ctypes

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

    # ---- greedy head ---------------------------------------------------------------------------------
    @staticmethod
    def lm_head_argmax_scratch_bytes(rows=0, n=0):
        return _C.lib.lri_lm_head_argmax_scratch_bytes()

    @staticmethod
    def lm_head_argmax(x, w, index_offset, token_out, rows, scratch, comm_handle=None, logits_ws=None, workspace=None,
                       timeout_ms=2000):
        """token_out[m] = arg-max over the whole vocabulary of sequence m, where `w` holds this rank's rows
        starting at vocabulary index `index_offset` (w may have no rows)."""
        _C.require_cuda(x, token_out, scratch)
        assert token_out.dtype == torch.int32
        n = w.shape[0]
        k = w.shape[1] if w.dim() == 2 else x.shape[-1]
        lw_ptr, lw_bytes = (logits_ws.data_ptr(), logits_ws.numel() * logits_ws.element_size()) if logits_ws is not None else (None, 0)
        ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        _C.check(_C.lib.lri_lm_head_argmax(comm_handle, _C.dtype_code(x.dtype), x.data_ptr(), w.data_ptr() if n else None,
                                           rows, n, k, index_offset, token_out.data_ptr(), scratch.data_ptr(),
                                           scratch.numel() * scratch.element_size(), lw_ptr, lw_bytes, ws_ptr, ws_bytes,
                                           timeout_ms, _C.stream_handle()))

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


def decode_splits(B, n_head, n_kv, smax, head_dim=128):
    """Number of sequence ranges for decode attention, fixed per cache geometry so that the launch
    grid never depends on the current position.  The rule lives in the library
    (lri_attn_decode_plan), next to the choice of the kernel it has to agree with."""
    n = ctypes.c_int(0)
    _C.check(_C.lib.lri_attn_decode_plan(B, n_head, n_kv, head_dim, smax, ctypes.byref(n)))
    return n.value
