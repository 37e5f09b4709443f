"""ctypes binding of liblri_b200.so (declared in include/lri_b200.h).

No logic lives here: tensors become `data_ptr()` values, the current CUDA stream becomes its raw
handle, and a negative status becomes a RuntimeError carrying lri_last_error().  There is no
fallback: if the shared library is missing the import fails with the command that builds it.
"""
import ctypes
import os

import torch

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "liblri_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python {os.path.join(_PKG_ROOT, 'build.py')}` "
        "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")

lib = ctypes.CDLL(LIB_PATH)

c_void_p, c_int, c_int64, c_float, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); the order of arguments is that of include/lri_b200.h
_SIGNATURES = {
    "lri_last_error": (ctypes.c_char_p, []),
    "lri_version": (c_int, []),
    "lri_set_gemm_backend": (c_int, [c_int]),
    "lri_launch_count": (c_int64, []),
    "lri_gemm_status": (c_int, []),
    "lri_set_option": (c_int, [ctypes.c_char_p, c_int]),
    "lri_get_option": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_int)]),
    "lri_attn_decode_plan": (c_int, [c_int, c_int, c_int, c_int, c_int64, ctypes.POINTER(c_int)]),
    "lri_add_rmsnorm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p,
                                c_int64, c_int, c_void_p]),
    "lri_embedding": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int64, c_void_p]),
    "lri_linear": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t,
                           c_void_p]),
    "lri_qkv_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int]),
    "lri_qkv_rope_kvcache": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,  # .. pos_is_i64
                                     c_void_p, c_void_p, c_void_p,  # q_out, k_cache, v_cache
                                     c_int, c_int, c_int, c_int, c_int, c_int,  # B, S, K, n_head, n_kv, head_dim
                                     c_int64, c_int64, c_int,  # smax, table_rows, table_gathered
                                     c_void_p, c_size_t, c_void_p]),
    "lri_gateup_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "lri_linear_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "lri_streamk_plan": (c_int, [c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lri_gateup_swiglu": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t,
                                  c_void_p]),
    "lri_attn_decode_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "lri_attn_decode": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "lri_attn_decode_static_scratch_capacity": (c_size_t, []),
    "lri_attn_decode_static": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int64, c_int, c_void_p]),
    "lri_attn_prefill": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                 c_int, c_int, c_int64, c_void_p]),
    "lri_comm_create": (c_int, [c_int, c_int, c_int64, ctypes.POINTER(c_void_p), ctypes.c_char_p]),
    "lri_comm_connect": (c_int, [c_void_p, ctypes.c_char_p]),
    "lri_allreduce": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "lri_comm_push_max_elems": (c_int64, []),
    "lri_linear_push": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                c_void_p]),
    "lri_comm_push": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "lri_add_rmsnorm_gather": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p,
                                       c_float, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "lri_add_rmsnorm_allreduce": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p,
                                          c_float, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "lri_lm_head_argmax_scratch_bytes": (c_size_t, []),
    "lri_lm_head_argmax": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p, c_void_p,
                                   c_size_t, c_void_p, c_size_t, c_void_p, c_size_t, c_int, c_void_p]),
    "lri_comm_status": (c_int, [c_void_p, c_void_p]),
    "lri_comm_destroy": (c_int, [c_void_p]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

BF16, FP16 = 0, 1
GEMM_AUTO, GEMM_TCGEN05, GEMM_SIMT = 0, 1, 2


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return FP16
    raise TypeError(f"the sm_100a kernels take bfloat16 or float16 tensors, not {dtype}")


def check(status: int) -> None:
    if status < 0:
        raise RuntimeError(f"lri_b200 error {status}: {lib.lri_last_error().decode()}")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("this build has no CPU path: tensors must live on a CUDA (sm_100a) device")
