"""Shared helpers for tests that read the golden fixtures written by tests/golden/make_golden.py."""
import os

import numpy as np
import torch

from oracle.ladder_oracle import OracleConfig

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TINY = dict(block_size=128, vocab_size=512, n_layer=3, n_head=4, n_local_heads=2, dim=256,
            intermediate_size=512, rope_base=500000)
DESYNC_PATTERN = [{"attention": False, "mlp": True}, {"attention": True, "mlp": False},
                  {"attention": False, "mlp": False}]
INITS = {"quiet": dict(std=0.02), "loud": dict(std=0.2, norm_mean=1.0, norm_std=0.2)}
BATCH, PROMPT, NEW = 2, 12, 5
SEED = 4242
VARIANTS = [("float32", 1, "quiet"), ("float32", 2, "loud"), ("bfloat16", 1, "loud"), ("bfloat16", 2, "quiet")]
FAMILIES = ("ladder", "dense", "parallel", "desync")


def load(tp):
    return np.load(os.path.join(GOLDEN_DIR, f"reference_tp{tp}.npz"))


def tiny_config(family):
    return OracleConfig(**TINY, reduce_pattern=DESYNC_PATTERN if family == "desync" else None)


def rel_err(a, b):
    """||a-b|| / ||b|| over the whole tensor, in fp64."""
    a = torch.as_tensor(a).double()
    b = torch.as_tensor(b).double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def replay(forward, gold, key):
    """Teacher-forced replay of a golden case through `forward(idx, input_pos) -> logits`.
    Returns the stacked last-position logits [NEW, B, V] (fp32) and row 0 of the prefill logits."""
    prompt = torch.from_numpy(gold[key + "/prompt"])
    fed = torch.from_numpy(gold[key + "/fed"])
    x = prompt.view(1, -1).repeat(BATCH, 1)
    logits = forward(x, torch.arange(PROMPT))
    steps = [logits[:, -1].float().cpu()]
    prefill_row0 = logits[0].float().cpu()
    for n in range(NEW - 1):
        logits = forward(fed[:, n:n + 1], torch.tensor([PROMPT + n], dtype=torch.int32))
        steps.append(logits[:, -1].float().cpu())
    return torch.stack(steps), prefill_row0


def load_shards(model, family, cfg, full, rank, t, dtype):
    """Copies rank `rank`'s shards of the seeded full weights into a model that has the reference's
    module tree (the reference itself or the drop-in package)."""
    from oracle.ladder_oracle import shard_layer
    with torch.no_grad():
        model.tok_embeddings.weight.copy_(full["tok_embeddings"].to(dtype))
        model.output.weight.copy_(full["output"].to(dtype))
        model.norm.weight.copy_(full["norm"].to(dtype))
        for i, layer in enumerate(model.layers):
            sh = shard_layer(cfg, full, i, rank, t, dtype)
            layer.attention_norm.weight.copy_(sh["attention_norm"])
            layer.attention.wo.weight.copy_(sh["wo"])
            if family == "parallel":
                layer.attention.wqkv1.weight.copy_(sh["wqkv1"])
                layer.attention.w2.weight.copy_(sh["w2"])
            else:
                layer.attention.wqkv.weight.copy_(sh["wqkv"])
                layer.feed_forward.w1.weight.copy_(sh["w1"])
                layer.feed_forward.w2.weight.copy_(sh["w2"])
                layer.ffn_norm.weight.copy_(sh["ffn_norm"])


def preset_kwargs(cfg):
    """ModelArgs keyword arguments of an OracleConfig (for registering a run-time preset)."""
    kw = dict(block_size=cfg.block_size, vocab_size=cfg.vocab_size, n_layer=cfg.n_layer, n_head=cfg.n_head,
              n_local_heads=cfg.n_local_heads, dim=cfg.dim, intermediate_size=cfg.intermediate_size,
              rope_base=cfg.rope_base, norm_eps=cfg.norm_eps, rope_scaling=cfg.rope_scaling)
    return kw
