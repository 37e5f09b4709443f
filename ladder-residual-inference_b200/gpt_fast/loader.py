"""Hugging Face Llama / LlamaLadder checkpoints -> the fused, sharded parameter layout of this package.

The reference has no loader (every rank draws its own random shard, benchmark.py:242-243); the only
conversion it carries is the load hook that fuses separate wq / wk / wv into wqkv
(gpt_fast/utils.py:178-185, kept in this package's Attention).  Real checkpoints of the Ladder
models use the Hugging Face Llama names (reference hf_modeling_utils/modeling_llama_ladder.py:
self_attn.{q,k,v,o}_proj at 281-284, mlp.{gate,up,down}_proj at 235-237); this module maps them onto
the per-rank layout that the kernels read:

    wqkv  [(nh + 2 nkv) hd / t, d]  rows [q heads of the rank | k heads | v heads]
    wo    [d, nh hd / t]            columns of the rank's heads
    w1    [2 I / t, d]              rows [up slice | gate slice]
    w2    [d, I / t]                columns of the slice
    tok_embeddings, output, all norm weights: replicated

Rotary layout: Hugging Face rotates the pairs (i, i + hd/2) of a head ("rotate half"), gpt_fast the
adjacent pairs (2i, 2i + 1) (gpt_fast/utils.py:120-132).  The rows of q_proj and k_proj are
therefore re-ordered inside every head, new row 2i + j = old row j hd/2 + i; scores q.k are
unchanged by a permutation applied to both, and v / o_proj are untouched.
"""
import glob
import json
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor


def _interleave_rotary_rows(w: Tensor, n_heads: int, head_dim: int) -> Tensor:
    """[n_heads * head_dim, d] in rotate-half order -> adjacent-pair order."""
    d = w.shape[1]
    return w.view(n_heads, 2, head_dim // 2, d).transpose(1, 2).reshape(n_heads * head_dim, d)


def _rows(w: Tensor, rank: int, world: int) -> Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


def _cols(w: Tensor, rank: int, world: int) -> Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n]


def hf_to_local(hf: Dict[str, Tensor], config, rank: int, world: int, family: str = "ladder") -> Dict[str, Tensor]:
    """State dict of a Hugging Face Llama-style model -> state dict of rank `rank` of `world` for the
    ladder / dense / desync module tree of this package (they share it).  Tensors keep their dtype;
    slices are views where possible."""
    if family == "parallel":
        raise ValueError("the parallel attention/MLP block has one norm per layer; Llama checkpoints do not map onto it")
    nh, nkv, d = config.n_head, config.n_local_heads, config.dim
    hd = d // nh
    inter = config.intermediate_size
    for name, v in (("n_head", nh), ("n_local_heads", nkv), ("intermediate_size", inter), ("dim", d)):
        if v % world:
            raise ValueError(f"{name}={v} is not divisible by the tensor-parallel degree {world}")
    out = {"tok_embeddings.weight": hf["model.embed_tokens.weight"], "norm.weight": hf["model.norm.weight"],
           # tied embeddings: the output projection is the embedding table
           "output.weight": hf.get("lm_head.weight", hf["model.embed_tokens.weight"])}
    for i in range(config.n_layer):
        src = f"model.layers.{i}."
        dst = f"layers.{i}."
        q = _interleave_rotary_rows(hf[src + "self_attn.q_proj.weight"], nh, hd)
        k = _interleave_rotary_rows(hf[src + "self_attn.k_proj.weight"], nkv, hd)
        v = hf[src + "self_attn.v_proj.weight"]
        if tuple(q.shape) != (nh * hd, d) or tuple(k.shape) != (nkv * hd, d) or tuple(v.shape) != (nkv * hd, d):
            raise ValueError(f"layer {i}: projection shapes do not match the preset")
        out[dst + "attention.wqkv.weight"] = torch.cat([_rows(q, rank, world), _rows(k, rank, world), _rows(v, rank, world)])
        out[dst + "attention.wo.weight"] = _cols(hf[src + "self_attn.o_proj.weight"], rank, world)
        out[dst + "feed_forward.w1.weight"] = torch.cat([_rows(hf[src + "mlp.up_proj.weight"], rank, world),
                                                         _rows(hf[src + "mlp.gate_proj.weight"], rank, world)])
        out[dst + "feed_forward.w2.weight"] = _cols(hf[src + "mlp.down_proj.weight"], rank, world)
        out[dst + "attention_norm.weight"] = hf[src + "input_layernorm.weight"]
        out[dst + "ffn_norm.weight"] = hf[src + "post_attention_layernorm.weight"]
    return out


def model_args_from_hf_config(path: str) -> Dict[str, object]:
    """ModelArgs keyword arguments from the config.json of a Hugging Face Llama / LlamaLadder
    checkpoint directory (field names: transformers' LlamaConfig; `ladder_layers` as normalised by
    the reference's hf_modeling_utils/configuration_llama_ladder.py:38-45).  Register the result under
    a preset name in a family's `transformer_configs` and build the model with `from_name`."""
    with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
        c = json.load(f)
    n_layer = c["num_hidden_layers"]
    kw = dict(block_size=c.get("max_position_embeddings", 2048), vocab_size=c["vocab_size"], n_layer=n_layer,
              n_head=c["num_attention_heads"], n_local_heads=c.get("num_key_value_heads", c["num_attention_heads"]),
              dim=c["hidden_size"], intermediate_size=c["intermediate_size"], rope_base=c.get("rope_theta", 10000.0),
              norm_eps=c.get("rms_norm_eps", 1e-5))
    scaling = c.get("rope_scaling")
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        kw["rope_scaling"] = {k: scaling[k] for k in ("factor", "low_freq_factor", "high_freq_factor",
                                                       "original_max_position_embeddings")}
    if "ladder_layers" in c:
        ll = c["ladder_layers"]
        if ll is None:
            ll = []
        elif isinstance(ll, int):
            ll = list(range(n_layer - ll, n_layer))
        kw["ladder_layers"] = [int(i) for i in ll]
    return kw


def load_hf_state_dict(model, hf: Dict[str, Tensor], rank: Optional[int] = None, world: Optional[int] = None) -> None:
    """Copies a Hugging Face Llama-style state dict into `model` (a GPTLadder / GPTDense / GPTDesync
    of this package, already on its device and in its dtype), taking this rank's shard."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    local = hf_to_local(hf, model.config, rank, world, model.family)
    params = dict(model.named_parameters())
    missing = sorted(set(params) - set(local))
    if missing:
        raise KeyError(f"checkpoint has no tensor for {missing[:4]}{' ...' if len(missing) > 4 else ''}")
    with torch.no_grad():
        for name, p in params.items():
            src = local[name]
            if tuple(src.shape) != tuple(p.shape):
                raise ValueError(f"{name}: checkpoint shard {tuple(src.shape)} vs parameter {tuple(p.shape)}")
            p.copy_(src.to(device=p.device, dtype=p.dtype))


def load_hf_checkpoint(model, path: str, rank: Optional[int] = None, world: Optional[int] = None) -> None:
    """`path`: a directory of *.safetensors shards (or one file) in Hugging Face Llama naming."""
    from safetensors.torch import load_file
    files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) if os.path.isdir(path) else [path]
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    hf: Dict[str, Tensor] = {}
    for f in files:
        hf.update(load_file(f))
    load_hf_state_dict(model, hf, rank, world)
