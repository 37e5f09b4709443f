"""Sublayer modules with the reference's names, constructor arguments, parameter layouts and
forward signatures (gpt_fast/utils.py of the reference), executed by the sm_100a kernels.

Every nn.Linear here only OWNS its weight in the reference's per-rank layout; its own forward
is never called.  The modules' `forward`s allocate their outputs and call the fused device
ops, so each one works on its own exactly like the reference module it mirrors; a whole-model
forward goes through `engine.Engine`, which runs the same ops on preallocated buffers.

Tensor parallelism is fixed at construction, as in the reference: every projection is created
already divided by the TP world size (utils.py:142-143, 165-166, 277-281 of the reference).
"""
import itertools
import math
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .tp import maybe_init_dist

_USE_FLASH_ATTENTION: bool = False


@contextmanager
def set_flash_attention(enable: bool):
    """Kept for the benchmark driver.  The flag is recorded but changes nothing: attention always
    runs the package's own decode / prefill kernels."""
    global _USE_FLASH_ATTENTION
    previous = _USE_FLASH_ATTENTION
    _USE_FLASH_ATTENTION = enable
    try:
        yield
    finally:
        _USE_FLASH_ATTENTION = previous


def is_flash_attention_enabled() -> bool:
    return _USE_FLASH_ATTENTION


maybe_init_dist()
tp_rank = dist.get_rank()
tp_world_size = dist.get_world_size()
tp_group = list(range(tp_world_size))


def _ops():
    from .ops import CudaOps  # imported late: needs the built shared library
    return CudaOps


class KVCache(nn.Module):
    """Dense cache, two buffers [max_batch, n_heads, max_seq, head_dim] (reference utils.py:43-59)."""

    def __init__(self, max_batch_size, max_seq_length, n_heads, head_dim, dtype=torch.bfloat16):
        super().__init__()
        shape = (max_batch_size, n_heads, max_seq_length, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype))
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype))

    def update(self, input_pos, k_val, v_val):
        """k_val, v_val: [B, H, S, D] written at positions input_pos [S]; returns the full caches.
        The fused QKV kernel writes the cache itself; this method is the reference's stand-alone
        interface and uses a plain indexed copy."""
        assert input_pos.shape[0] == k_val.shape[2]
        self.k_cache[: k_val.shape[0], :, input_pos.long()] = k_val
        self.v_cache[: v_val.shape[0], :, input_pos.long()] = v_val
        return self.k_cache, self.v_cache


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        x = x.contiguous()
        out = torch.empty_like(x)
        _ops().add_rmsnorm(x, None, None, self.weight, self.eps, None, out, x.numel() // x.shape[-1])
        return out


def apply_rope_scaling(freqs: torch.Tensor, rope_scaling: dict):
    """Llama-3.1 frequency scaling (reference utils.py:81-100): long wavelengths are divided by
    `factor`, short ones kept, the band between interpolated."""
    factor = rope_scaling["factor"]
    lo, hi = rope_scaling["low_freq_factor"], rope_scaling["high_freq_factor"]
    ctx = rope_scaling["original_max_position_embeddings"]
    wavelen = 2 * math.pi / freqs
    smooth = (ctx / wavelen - lo) / (hi - lo)
    mid = (1 - smooth) * freqs / factor + smooth * freqs
    return torch.where(wavelen < ctx / hi, freqs, torch.where(wavelen > ctx / lo, freqs / factor, mid))


def precompute_freqs_cis(seq_len: int, n_elem: int, base: int = 10000, dtype: torch.dtype = torch.bfloat16,
                         rope_scaling: Optional[dict] = None) -> Tensor:
    """[seq_len, n_elem/2, 2] table of (cos, sin) of pos * base^(-2i/n_elem), evaluated in fp32 and
    rounded to `dtype` (reference utils.py:103-117)."""
    freqs = 1.0 / (base ** (torch.arange(0, n_elem, 2)[: n_elem // 2].float() / n_elem))
    if rope_scaling is not None:
        freqs = apply_rope_scaling(freqs, rope_scaling)
    angles = torch.outer(torch.arange(seq_len, device=freqs.device), freqs)
    return torch.stack([torch.cos(angles), torch.sin(angles)], dim=-1).to(dtype=dtype)


def _as_pos(input_pos: Tensor) -> Tensor:
    return input_pos if input_pos.dtype in (torch.int32, torch.int64) else input_pos.to(torch.int64)


class FeedForward(nn.Module):
    """w1 [2I/t, d] rows = [up | gate], w2 [d, I/t]; returns the rank's partial sum."""

    def __init__(self, config) -> None:
        super().__init__()
        assert config.intermediate_size % tp_world_size == 0
        assert config.dim % tp_world_size == 0
        self.w1 = nn.Linear(config.dim, 2 * config.intermediate_size // tp_world_size, bias=False)
        self.w2 = nn.Linear(config.intermediate_size // tp_world_size, config.dim, bias=False)

    def forward(self, x: Tensor) -> Tensor:
        ops = _ops()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        rows = x2.shape[0]
        inter = self.w1.weight.shape[0] // 2
        h = torch.empty(rows, inter, dtype=x.dtype, device=x.device)
        ws_bytes = ops.gateup_workspace_bytes(rows, inter)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        ops.gateup_swiglu(x2, self.w1.weight, h, rows, ws)
        y = torch.empty(rows, self.w2.weight.shape[0], dtype=x.dtype, device=x.device)
        ops.linear(h, self.w2.weight, y, rows)
        return y.view(*shape[:-1], -1)


def _attention_core(mod, q, input_pos, bsz, seqlen):
    """Attention over the module's cache for queries q [B, S, n_head, hd] -> [B*S, n_head*hd]."""
    ops = _ops()
    from .ops import decode_splits
    kc, vc = mod.kv_cache.k_cache, mod.kv_cache.v_cache
    y = torch.empty(bsz * seqlen, mod.n_head * mod.head_dim, dtype=q.dtype, device=q.device)
    scratch, splits = None, 1
    if seqlen == 1:
        splits = decode_splits(bsz, mod.n_head, mod.n_local_heads, kc.shape[2], mod.head_dim)
        nbytes = ops.attn_decode_scratch_bytes(bsz, mod.n_head, mod.n_local_heads, mod.head_dim, splits)
        scratch = torch.zeros(nbytes, dtype=torch.uint8, device=q.device)
    ops.attention(q, kc, vc, input_pos, y, bsz, seqlen, mod.n_head, mod.n_local_heads, mod.head_dim, scratch, splits)
    return y


def _qkv(mod, x2, weight_rows, freqs_cis, input_pos, bsz, seqlen):
    ops = _ops()
    rows = bsz * seqlen
    q = torch.empty(rows, mod.n_head * mod.head_dim, dtype=x2.dtype, device=x2.device)
    ws_bytes = ops.qkv_workspace_bytes(rows, mod.n_head, mod.n_local_heads, mod.head_dim)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x2.device) if ws_bytes else None
    # freqs_cis arrives already indexed by position (freqs_cis[input_pos]), as the reference passes it
    ops.qkv_rope_kvcache(x2, weight_rows, freqs_cis.contiguous(), True, input_pos, q, mod.kv_cache.k_cache,
                         mod.kv_cache.v_cache, bsz, seqlen, mod.n_head, mod.n_local_heads, mod.head_dim, ws)
    return q


class Attention(nn.Module):
    """wqkv [(nh + 2 nkv) hd / t, d] rows = [q heads | k heads | v heads] of this rank, wo [d, nh hd / t].
    forward(x, freqs_cis, mask, input_pos): `freqs_cis` holds the table rows of the tokens'
    positions and `mask` is accepted for interface compatibility; the kernels derive the causal
    mask from `input_pos` (the reference builds it as causal_mask[input_pos])."""

    def __init__(self, config):
        super().__init__()
        assert config.dim % config.n_head == 0
        total_head_dim = (config.n_head + 2 * config.n_local_heads) * config.head_dim
        assert total_head_dim % tp_world_size == 0
        assert config.dim % tp_world_size == 0
        assert config.n_head % tp_world_size == 0
        assert config.n_local_heads % tp_world_size == 0
        self.wqkv = nn.Linear(config.dim, total_head_dim // tp_world_size, bias=False)
        self.wo = nn.Linear(config.dim // tp_world_size, config.dim, bias=False)
        self.kv_cache = None
        self.head_dim = config.head_dim
        self.n_head = config.n_head // tp_world_size
        self.dim = config.dim // tp_world_size
        self.n_local_heads = config.n_local_heads // tp_world_size
        self._register_load_state_dict_pre_hook(self.load_hook)

    def load_hook(self, state_dict, prefix, *args):
        """Checkpoints with separate wq / wk / wv are fused on load (reference utils.py:178-185)."""
        if prefix + "wq.weight" in state_dict:
            parts = [state_dict.pop(prefix + n + ".weight") for n in ("wq", "wk", "wv")]
            state_dict[prefix + "wqkv.weight"] = torch.cat(parts)

    def forward(self, x: Tensor, freqs_cis: Tensor, mask: Tensor, input_pos: Optional[Tensor] = None) -> Tensor:
        assert self.kv_cache is not None, "Caches must be initialized first"
        ops = _ops()
        bsz, seqlen, _ = x.shape
        pos = _as_pos(input_pos)
        x2 = x.reshape(bsz * seqlen, -1).contiguous()
        q = _qkv(self, x2, self.wqkv.weight, freqs_cis, pos, bsz, seqlen)
        y = _attention_core(self, q, pos, bsz, seqlen)
        out = torch.empty(bsz * seqlen, self.wo.weight.shape[0], dtype=x.dtype, device=x.device)
        ops.linear(y, self.wo.weight, out, bsz * seqlen)
        return out.view(bsz, seqlen, -1)


class FuseAttentionMLP(nn.Module):
    """Parallel block's fused sublayer: one input projection wqkv1 with rows [q | k | v | up | gate],
    attention and MLP from the same normed input, wo and w2 partials summed (reference utils.py:263-387)."""

    def __init__(self, config):
        super().__init__()
        assert config.dim % config.n_head == 0
        total_head_dim = (config.n_head + 2 * config.n_local_heads) * config.head_dim
        assert total_head_dim % tp_world_size == 0
        assert config.dim % tp_world_size == 0
        assert config.intermediate_size % tp_world_size == 0
        assert config.n_head % tp_world_size == 0
        assert config.n_local_heads % tp_world_size == 0
        self.wqkv1 = nn.Linear(
            config.dim, total_head_dim // tp_world_size + 2 * config.intermediate_size // tp_world_size, bias=False)
        self.wo = nn.Linear(config.dim // tp_world_size, config.dim, bias=False)
        self.w2 = nn.Linear(config.intermediate_size // tp_world_size, config.dim, bias=False)
        self.kv_cache = None
        self.head_dim = config.head_dim
        self.n_head = config.n_head // tp_world_size
        self.dim = config.dim // tp_world_size
        self.n_local_heads = config.n_local_heads // tp_world_size
        self.intermediate_size = config.intermediate_size // tp_world_size
        self._register_load_state_dict_pre_hook(self.load_hook)

    def load_hook(self, state_dict, prefix, *args):
        if prefix + "wq.weight" in state_dict:
            parts = [state_dict.pop(prefix + n + ".weight") for n in ("wq", "wk", "wv")]
            state_dict[prefix + "wqkv.weight"] = torch.cat(parts)

    @property
    def qkv_rows(self) -> int:
        return (self.n_head + 2 * self.n_local_heads) * self.head_dim

    def forward(self, x: Tensor, freqs_cis: Tensor, mask: Tensor, input_pos: Optional[Tensor] = None) -> Tensor:
        assert self.kv_cache is not None, "Caches must be initialized first"
        ops = _ops()
        bsz, seqlen, _ = x.shape
        rows = bsz * seqlen
        pos = _as_pos(input_pos)
        x2 = x.reshape(rows, -1).contiguous()
        w = self.wqkv1.weight
        q = _qkv(self, x2, w[: self.qkv_rows], freqs_cis, pos, bsz, seqlen)
        y = _attention_core(self, q, pos, bsz, seqlen)
        attn = torch.empty(rows, self.wo.weight.shape[0], dtype=x.dtype, device=x.device)
        ops.linear(y, self.wo.weight, attn, rows)
        h = torch.empty(rows, self.intermediate_size, dtype=x.dtype, device=x.device)
        ws_bytes = ops.gateup_workspace_bytes(rows, self.intermediate_size)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        ops.gateup_swiglu(x2, w[self.qkv_rows:], h, rows, ws)
        out = torch.empty_like(attn)
        ops.linear(h, self.w2.weight, out, rows, addend=attn)
        return out.view(bsz, seqlen, -1)


def all_reduce_func(x: torch.Tensor, clone: bool, async_op=False):
    """In-place SUM over the TP group; returns (tensor, handle) like the reference (utils.py:390-397).
    `clone=True` (the reference's functional-collective branch) reduces a copy.  The handle's
    wait() makes the current stream wait for the result."""
    from .comm import make_comm
    comm = make_comm()
    if clone:
        x = x.clone()
    handle = comm.all_reduce_async(x)
    if not async_op:
        comm.wait(handle)
        return x, None
    return x, _Handle(comm, handle)


class _Handle:
    def __init__(self, comm, inner):
        self._comm, self._inner = comm, inner

    def wait(self):
        self._comm.wait(self._inner)


def _get_model_size(model):
    """Bytes and parameter count per rank of everything except nn.Embedding children
    (reference utils.py:400-409; the benchmark prints bandwidth from it)."""
    model_size, params = 0, 0
    for _, child in model.named_children():
        if not isinstance(child, torch.nn.Embedding):
            for p in itertools.chain(child.parameters(), child.buffers()):
                model_size += p.numel() * p.dtype.itemsize
                params += p.numel()
    return model_size, params
