"""Generate the golden fixtures in this directory by running the REFERENCE itself on the CPU.

Run (only where a checkout of the reference exists; the fixtures are committed):

    python tests/golden/make_golden.py --reference /path/to/ladder-residual-inference

What it does: for every case in CASES it starts `tp` gloo ranks, imports the reference's
`gpt_fast` package from the given path, builds the reference model for a tiny preset that is
registered at run time, loads per-rank shards of seeded full weights (the same generator and
shard mapping the oracle uses, `oracle/ladder_oracle.py`), runs a prefill and a few
teacher-forced greedy decode steps through the reference's own `forward`, and stores the
token ids fed and the last-position logits of every step.  It also stores outputs of the
reference's RMSNorm, RoPE table, rotation, FeedForward and Attention modules on seeded inputs.

Three run-time shims make the reference importable without a GPU, none of which changes
its arithmetic: (1) a gloo process group is created before the import, which makes its
`maybe_init_dist` skip the CUDA/NCCL set-up; (2) `RMSNorm.forward` is pointed at the
reference's own non-Triton formula (the branch it takes under torch.compile); (3) the
Triton residual-add kernel object of the ladder block is replaced by a torch add.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.ladder_oracle import OracleConfig, make_full_weights, shard_layer  # noqa: E402

TINY = dict(block_size=128, vocab_size=512, n_layer=3, n_head=4, n_local_heads=2, dim=256,
            intermediate_size=512, rope_base=500000)
DESYNC_PATTERN = [{"attention": False, "mlp": True}, {"attention": True, "mlp": False},
                  {"attention": False, "mlp": False}]
INITS = {"quiet": dict(std=0.02), "loud": dict(std=0.2, norm_mean=1.0, norm_std=0.2)}
BATCH, PROMPT, NEW = 2, 12, 5
SEED = 4242
# (dtype, tp, init)
VARIANTS = [("float32", 1, "quiet"), ("float32", 2, "loud"), ("bfloat16", 1, "loud"), ("bfloat16", 2, "quiet")]
CASES = [(fam, *v) for fam in ("ladder", "dense", "parallel", "desync") for v in VARIANTS]


class _AddKernel:
    """Stands in for the Triton kernel object: kernel[grid](x, y, out, n, BLOCK)."""

    def __getitem__(self, grid):
        def run(x, y, out, n, block):
            out.copy_(x + y)
        return run


def _import_reference(ref_path):
    sys.path.insert(0, ref_path)
    import gpt_fast  # noqa: F401  (needs the process group to exist already)
    from gpt_fast import gpt_dense_TP, gpt_desync_TP, gpt_ladder_TP, gpt_parallel_TP, utils

    def norm_forward(self, x):
        return self._norm(x.float()).type_as(x) * self.weight

    utils.RMSNorm.forward = norm_forward
    gpt_ladder_TP.add_tensor_forward_triton_kernel = _AddKernel()
    mods = {"ladder": (gpt_ladder_TP, gpt_fast.GPTLadder), "dense": (gpt_dense_TP, gpt_fast.GPTDense),
            "parallel": (gpt_parallel_TP, gpt_fast.GPTParallel), "desync": (gpt_desync_TP, gpt_fast.GPTDesync)}
    for fam, (m, _) in mods.items():
        preset = dict(TINY)
        if fam == "desync":
            preset["reduce_pattern"] = DESYNC_PATTERN
        m.transformer_configs["tiny-golden"] = preset
    return mods, utils


def _load(model, family, cfg, full, rank, t, dtype):
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


def _worker(rank, world, port, ref_path, tp_cases, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mods, utils = _import_reference(ref_path)
    saved = {}
    for family, dtype_name, tp, init in tp_cases:
        assert tp == world
        dtype = getattr(torch, dtype_name)
        cfg = OracleConfig(**TINY, reduce_pattern=DESYNC_PATTERN if family == "desync" else None)
        full = make_full_weights(cfg, SEED, **INITS[init])
        mod, cls = mods[family]
        model = cls.from_name("tiny-golden").to(dtype).eval()
        _load(model, family, cfg, full, rank, tp, dtype)
        model.setup_caches(max_batch_size=BATCH, max_seq_length=PROMPT + NEW)
        g = torch.Generator().manual_seed(1234)
        prompt = torch.randint(0, cfg.vocab_size, (PROMPT,), generator=g)
        fed, logits_steps = [], []
        with torch.no_grad():
            x = prompt.view(1, -1).repeat(BATCH, 1)
            logits = model(x, torch.arange(PROMPT))
            logits_steps.append(logits[:, -1].float())
            prefill_all = logits[0].float()
            tok = logits[:, -1].float().argmax(-1, keepdim=True)
            for n in range(NEW - 1):
                fed.append(tok)
                logits = model(tok, torch.tensor([PROMPT + n], dtype=torch.int32))
                logits_steps.append(logits[:, -1].float())
                tok = logits[:, -1].float().argmax(-1, keepdim=True)
        if rank == 0:
            key = f"{family}-{dtype_name}-tp{tp}-{init}"
            saved[key + "/prompt"] = prompt.numpy()
            saved[key + "/fed"] = torch.cat(fed, dim=-1).numpy()
            saved[key + "/logits"] = torch.stack(logits_steps).numpy()  # [NEW, B, V]
            saved[key + "/prefill_row0"] = prefill_all.numpy()  # [PROMPT, V]
            print("done", key, flush=True)
    if rank == 0 and world == 1:
        saved.update(_module_goldens(utils))
    if rank == 0:
        np.savez_compressed(os.path.join(out_dir, f"reference_tp{world}.npz"), **saved)
    dist.barrier()
    dist.destroy_process_group()


def _module_goldens(utils):
    """Outputs of the reference's sublayer modules on seeded inputs (TP = 1)."""
    out = {}
    g = torch.Generator().manual_seed(99)
    for dtype_name in ("float32", "bfloat16"):
        dtype = getattr(torch, dtype_name)
        x = (torch.randn(3, 5, 256, generator=g) * 1.7).to(dtype)
        norm = utils.RMSNorm(256, eps=1e-5)
        norm.weight.data = (1 + 0.3 * torch.randn(256, generator=g)).to(dtype)
        out[f"ops/{dtype_name}/rms_x"] = x.float().numpy()
        out[f"ops/{dtype_name}/rms_w"] = norm.weight.detach().float().numpy()
        out[f"ops/{dtype_name}/rms_y"] = norm(x).float().detach().numpy()
        table = utils.precompute_freqs_cis(64, 64, 500000, dtype)
        out[f"ops/{dtype_name}/rope_table"] = table.float().numpy()
        scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
        out[f"ops/{dtype_name}/rope_table_scaled"] = utils.precompute_freqs_cis(
            32, 128, 500000, dtype, scaling).float().numpy()
        q = torch.randn(2, 6, 4, 64, generator=g).to(dtype)
        out[f"ops/{dtype_name}/rope_x"] = q.float().numpy()
        out[f"ops/{dtype_name}/rope_y"] = utils.apply_rotary_emb(q, table[3:9]).float().numpy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    for world in (1, 2):
        cases = [c for c in CASES if c[2] == world]
        mp.spawn(_worker, args=(world, 29611 + world, args.reference, cases, HERE), nprocs=world, join=True)


if __name__ == "__main__":
    main()
