"""Desynchronised family: a per-layer pattern says which sublayers all-reduce at all; between
all-reduces every rank carries its own residual (reference: gpt_fast/gpt_desync_TP.py).  The
`*-upper-bound` presets never communicate and give the no-communication speed ceiling."""
from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist
from torch import Tensor

from .model_base import BlockBase, ModelArgsBase, TPModelBase, args_from_name, find_multiple  # noqa: F401
from .presets import family_presets
from .tp import maybe_init_dist
from .utils import Attention, FeedForward, RMSNorm, _ops, all_reduce_func

maybe_init_dist()
tp_rank = dist.get_rank()
tp_world_size = dist.get_world_size()
tp_group = list(range(tp_world_size))

transformer_configs = family_presets("desync")


@dataclass
class ModelArgs(ModelArgsBase):
    reduce_pattern: Optional[list] = None
    force_disable_last_all_reduce: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.reduce_pattern is None:
            self.reduce_pattern = [{"attention": False, "mlp": True} for _ in range(self.n_layer)]

    @classmethod
    def from_name(cls, name: str):
        return args_from_name(cls, transformer_configs, name)


def _add_scaled(y: Tensor, x: Tensor, scale: float) -> Tensor:
    """y + round(x * scale), rounded: the desync block's `y + x / tp_world_size`."""
    out = x.new_empty(x.shape)
    _ops().add_rmsnorm(x.contiguous(), y.contiguous(), None, None, 0.0, out, None, x.numel() // x.shape[-1], scale)
    return out


class DesyncTransformerBlock(BlockBase):
    def __init__(self, config: ModelArgs, layer_idx: int) -> None:
        super().__init__()
        self.attention = Attention(config)
        self.feed_forward = FeedForward(config)
        self.ffn_norm = RMSNorm(config.dim, config.norm_eps)
        self.attention_norm = RMSNorm(config.dim, config.norm_eps)
        last = layer_idx == config.n_layer - 1
        self.do_attention_all_reduce = config.reduce_pattern[layer_idx]["attention"]
        self.do_mlp_all_reduce = last or config.reduce_pattern[layer_idx]["mlp"]
        if last and config.force_disable_last_all_reduce:
            self.do_mlp_all_reduce = False
        self.semi_compiled_model = config.semi_compiled_model

    def _sublayer(self, y: Tensor, residual: Tensor, reduce: bool) -> Tensor:
        if reduce:
            return all_reduce_func(_add_scaled(y, residual, 1.0 / tp_world_size), clone=False)[0]
        return _add_scaled(y, residual, 1.0)

    def forward(self, x: Tensor, input_pos: Tensor, freqs_cis: Tensor, mask: Tensor) -> Tensor:
        y = self.attention(self.attention_norm(x), freqs_cis, mask, input_pos)
        x = self._sublayer(y, x, self.do_attention_all_reduce)
        y = self.feed_forward(self.ffn_norm(x))
        return self._sublayer(y, x, self.do_mlp_all_reduce)


class GPTDesync(TPModelBase):
    family = "desync"

    def __init__(self, config: ModelArgs) -> None:
        super().__init__(config, (DesyncTransformerBlock(config, layer_idx=i) for i in range(config.n_layer)))

    @classmethod
    def from_name(cls, name: str):
        return cls(ModelArgs.from_name(name))
