"""Ladder-Residual family (reference: gpt_fast/gpt_ladder_TP.py).

In a ladder block the all-reduced output of a sublayer is added to the residual one sublayer
later, so the all-reduce runs while the next sublayer computes.  `GPTLadder.forward` runs the
whole schedule in `engine.Engine`; `LadderTransformerBlock.forward` keeps the reference's
block-level signature for callers that drive blocks themselves.
"""
from dataclasses import dataclass
from typing import List, Optional, Union

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

transformer_configs = family_presets("ladder")


@dataclass
class ModelArgs(ModelArgsBase):
    # Indices of the layers that use the ladder dataflow; the others run as dense layers.  None (the
    # default, and all the reference's gpt_fast presets): every layer is a ladder layer.  An int n means
    # the last n layers.  This is the `ladder_layers` field of the reference's Hugging Face config
    # (hf_modeling_utils/configuration_llama_ladder.py:38-45), needed to run converted checkpoints.
    ladder_layers: Optional[Union[int, List[int]]] = None

    def __post_init__(self):
        super().__post_init__()
        if isinstance(self.ladder_layers, int):
            self.ladder_layers = list(range(self.n_layer - self.ladder_layers, self.n_layer))
        if self.ladder_layers is not None:
            assert all(0 <= i < self.n_layer for i in self.ladder_layers), "ladder_layers out of range"

    @classmethod
    def from_name(cls, name: str):
        return args_from_name(cls, transformer_configs, name)


def add_tensors(x: Tensor, y: Tensor) -> Tensor:
    """x + y rounded to the storage type: the reference's Triton kernel
    add_tensor_forward_triton_kernel (gpt_ladder_TP.py:364-377) as one F1 launch without a norm."""
    out = x.new_empty(x.shape)
    _ops().add_rmsnorm(x.contiguous(), y.contiguous(), None, None, 0.0, out, None, x.numel() // x.shape[-1])
    return out


class LadderTransformerBlock(BlockBase):
    def __init__(self, config: ModelArgs) -> None:
        super().__init__()
        self.attention = Attention(config)
        self.feed_forward = FeedForward(config)
        self.ffn_norm = RMSNorm(config.dim, config.norm_eps)
        self.attention_norm = RMSNorm(config.dim, config.norm_eps)
        self.semi_compiled_model = config.semi_compiled_model

    def forward(self, previous_attention_out: Tensor, previous_mlp_out: Tensor, residual: Tensor, attention_handle,
                mlp_handle, input_pos: Tensor, freqs_cis: Tensor, mask: Tensor):
        if attention_handle is not None:
            attention_handle.wait()
        residual = add_tensors(residual, previous_attention_out)
        current_attention_out = self.attention(self.attention_norm(residual), freqs_cis, mask, input_pos)
        current_attention_out, attention_handle = all_reduce_func(current_attention_out, clone=False, async_op=True)
        if mlp_handle is not None:
            mlp_handle.wait()
        residual = add_tensors(residual, previous_mlp_out)
        current_mlp_out = self.feed_forward(self.ffn_norm(residual))
        current_mlp_out, mlp_handle = all_reduce_func(current_mlp_out, clone=False, async_op=True)
        return current_attention_out, current_mlp_out, residual, attention_handle, mlp_handle


class GPTLadder(TPModelBase):
    family = "ladder"

    def __init__(self, config: ModelArgs) -> None:
        super().__init__(config, (LadderTransformerBlock(config) for _ in range(config.n_layer)))

    @classmethod
    def from_name(cls, name: str):
        return cls(ModelArgs.from_name(name))
