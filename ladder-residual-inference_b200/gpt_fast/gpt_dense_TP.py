"""Standard (dense) tensor-parallel family: a blocking all-reduce after every sublayer
(reference: gpt_fast/gpt_dense_TP.py)."""
from dataclasses import dataclass

import torch.distributed as dist
from torch import Tensor

from .gpt_ladder_TP import add_tensors
from .model_base import BlockBase, ModelArgsBase, TPModelBase, args_from_name, find_multiple  # noqa: F401
from .presets import family_presets
from .tp import maybe_init_dist
from .utils import Attention, FeedForward, RMSNorm, all_reduce_func

maybe_init_dist()
tp_rank = dist.get_rank()
tp_world_size = dist.get_world_size()
tp_group = list(range(tp_world_size))

transformer_configs = family_presets("dense")


@dataclass
class ModelArgs(ModelArgsBase):
    @classmethod
    def from_name(cls, name: str):
        return args_from_name(cls, transformer_configs, name)


class DenseTransformerBlock(BlockBase):
    def __init__(self, config: ModelArgs) -> None:
        super().__init__()
        self.attention = Attention(config)
        self.feed_forward = FeedForward(config)
        self.ffn_norm = RMSNorm(config.dim, config.norm_eps)
        self.attention_norm = RMSNorm(config.dim, config.norm_eps)
        self.semi_compiled_model = config.semi_compiled_model

    def forward(self, x: Tensor, input_pos: Tensor, freqs_cis: Tensor, mask: Tensor) -> Tensor:
        a = all_reduce_func(self.attention(self.attention_norm(x), freqs_cis, mask, input_pos), clone=False)[0]
        x = add_tensors(x, a)
        f = all_reduce_func(self.feed_forward(self.ffn_norm(x)), clone=False)[0]
        return add_tensors(x, f)


class GPTDense(TPModelBase):
    family = "dense"

    def __init__(self, config: ModelArgs) -> None:
        super().__init__(config, (DenseTransformerBlock(config) for _ in range(config.n_layer)))

    @classmethod
    def from_name(cls, name: str):
        return cls(ModelArgs.from_name(name))
