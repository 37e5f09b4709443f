"""Pieces shared by the four family modules: ModelArgs, the model shell and the block shell.

The reference repeats these in every family file (gpt_fast/gpt_ladder_TP.py:20-62, 210-288 and
its three siblings); here the family files keep only what differs between schedules.
"""
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .engine import Engine
from .utils import KVCache, RMSNorm, precompute_freqs_cis


def find_multiple(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class ModelArgsBase:
    block_size: int = 2048
    vocab_size: int = 32000
    n_layer: int = 32
    n_head: int = 32
    dim: int = 4096
    intermediate_size: int = None
    n_local_heads: int = -1
    head_dim: int = 64
    rope_base: float = 10000
    norm_eps: float = 1e-5
    rope_scaling: Optional[dict] = None
    semi_compiled_model: bool = False

    def __post_init__(self):
        world = dist.get_world_size()
        if self.n_local_heads == -1:
            self.n_local_heads = self.n_head
        if self.intermediate_size is None:
            # the usual Llama rule: 2/3 of 4*dim, rounded up to a multiple of 256
            self.intermediate_size = find_multiple(int(2 * (4 * self.dim) / 3), 256)
        self.head_dim = self.dim // self.n_head
        assert self.dim % world == 0
        assert self.intermediate_size % world == 0


def args_from_name(cls, table, name):
    if name not in table:
        raise KeyError(f"unknown preset {name!r}; known presets: {sorted(table)}")
    return cls(**table[name])


class TPModelBase(nn.Module):
    """tok_embeddings, layers, norm, output (replicated LM head), freqs_cis, causal_mask,
    max_batch_size, max_seq_length: the attributes the benchmark driver and the reference's own
    code use.  forward(idx [B, S], input_pos [S]) -> logits [B, S, vocab]."""

    family = ""

    def __init__(self, config, blocks) -> None:
        super().__init__()
        self.config = config
        self.tok_embeddings = nn.Embedding(config.vocab_size, config.dim)
        self.layers = nn.ModuleList(blocks)
        self.norm = RMSNorm(config.dim, eps=config.norm_eps)
        self.output = nn.Linear(config.dim, config.vocab_size, bias=False)
        self.freqs_cis: Optional[Tensor] = None
        self.mask_cache: Optional[Tensor] = None
        self.max_batch_size = -1
        self.max_seq_length = -1
        self._engine = None

    def setup_caches(self, max_batch_size, max_seq_length):
        if self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        cfg = self.config
        world = dist.get_world_size()
        head_dim = cfg.dim // cfg.n_head
        max_seq_length = find_multiple(max_seq_length, 8)
        self.max_seq_length = max_seq_length
        self.max_batch_size = max_batch_size
        dtype = self.output.weight.dtype
        device = self.output.weight.device
        for b in self.layers:
            b.attention.kv_cache = KVCache(max_batch_size, max_seq_length, cfg.n_local_heads // world, head_dim,
                                           dtype).to(device)
        self.freqs_cis = precompute_freqs_cis(cfg.block_size, head_dim, cfg.rope_base, dtype,
                                              cfg.rope_scaling).to(device).contiguous()
        # kept because callers of the reference may read it; the kernels derive causality from input_pos
        self.causal_mask = torch.tril(torch.ones(max_seq_length, max_seq_length, dtype=torch.bool, device=device))
        self._engine = Engine(self, self.family)
        self._engine.setup(max_batch_size, max_seq_length, device, dtype)

    def forward(self, idx: Tensor, input_pos: Optional[Tensor] = None) -> Tensor:
        assert self.freqs_cis is not None, "Caches must be initialized first"
        return self._engine.forward(idx, input_pos)

    def prefill_last(self, idx: Tensor, input_pos: Tensor) -> Tensor:
        """forward(idx, input_pos)[:, -1:] without computing the other positions' logits (no
        counterpart in the reference, whose forward always projects every position)."""
        assert self.freqs_cis is not None, "Caches must be initialized first"
        return self._engine.forward_last(idx, input_pos)

    def decode_greedy(self, idx: Tensor, input_pos: Tensor) -> Tensor:
        """Arg-max next token of every sequence, int32 [B, 1]; equal to
        `forward(idx, input_pos)[:, -1].argmax(-1)` but with the output projection split by
        vocabulary over the tensor-parallel ranks (no counterpart in the reference, which
        samples from the replicated logits, benchmark.py:74-92)."""
        assert self.freqs_cis is not None, "Caches must be initialized first"
        return self._engine.forward_greedy(idx, input_pos)

    def decode_sample(self, idx: Tensor, input_pos: Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                      generator=None) -> Tensor:
        """One sampled next token per sequence, int32 [B, 1], by the reference's rule
        (`sample(model(idx, input_pos), temperature, top_k)[0]`, benchmark.py:56-92), computed on the
        vocabulary-split output projection; see Engine.forward_sample."""
        assert self.freqs_cis is not None, "Caches must be initialized first"
        return self._engine.forward_sample(idx, input_pos, temperature, top_k, generator)


class BlockBase(nn.Module):
    def extra_repr(self) -> str:
        return f"semi_compiled = {self.semi_compiled_model}"
