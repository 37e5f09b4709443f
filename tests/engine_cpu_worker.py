"""One gloo rank of the engine-schedule test (started by tests/test_host_cpu.py through
torch.distributed.run).  Builds the drop-in model on the CPU, swaps the engine's device ops for
the oracle-based stand-in, replays the reference's golden cases for this world size and checks
rank 0's logits (all ranks check: ladder, dense and parallel are rank-invariant; desync is
compared on rank 0 only)."""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (HERE, ROOT, os.path.join(ROOT, "ladder-residual-inference_b200")):
    sys.path.insert(0, p)

dist.init_process_group("gloo")

import golden_util as gu  # noqa: E402
from cpu_ops import CpuOps  # noqa: E402
from oracle import ladder_oracle as lo  # noqa: E402

import gpt_fast  # noqa: E402
from gpt_fast import gpt_dense_TP, gpt_desync_TP, gpt_ladder_TP, gpt_parallel_TP  # noqa: E402
from gpt_fast.comm import make_comm  # noqa: E402


def check_hf_checkpoint(rank, world, mods):
    """A small random Hugging Face Llama, saved as safetensors, loaded shard by shard into the
    drop-in dense and ladder models; the dense logits must be transformers' own."""
    import tempfile
    try:
        import transformers
        from safetensors.torch import save_file
    except ImportError:
        return
    from gpt_fast.loader import load_hf_checkpoint
    hcfg = transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, rope_theta=500000.0, rms_norm_eps=1e-5,
                                    max_position_embeddings=512, tie_word_embeddings=False)
    torch.manual_seed(3)
    hf = transformers.LlamaForCausalLM(hcfg).eval()
    ids = torch.randint(0, 512, (2, 12), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = hf(ids).logits
    with tempfile.TemporaryDirectory() as tmp:
        sd = {k: v.contiguous() for k, v in hf.state_dict().items()}
        save_file(sd, f"{tmp}/model-rank{rank}.safetensors")
        kw = dict(block_size=512, vocab_size=512, n_layer=2, n_head=4, n_local_heads=2, dim=256, intermediate_size=512,
                  rope_base=500000, norm_eps=1e-5)
        for family in ("dense", "ladder"):
            mod, cls = mods[family]
            mod.transformer_configs["tiny-hf"] = dict(kw)
            model = cls.from_name("tiny-hf").to(torch.float32).eval()
            load_hf_checkpoint(model, f"{tmp}/model-rank{rank}.safetensors")
            model.setup_caches(max_batch_size=2, max_seq_length=16)
            model._engine.ops = CpuOps
            got = model(ids, torch.arange(12))
            if family == "dense":
                err = ((got - want).abs().max() / want.abs().max()).item()
                assert err < 2e-5, f"hf checkpoint, rank {rank}: {err}"
            else:  # a different schedule on the same weights: finite and not the dense logits
                assert torch.isfinite(got).all() and (got - want).abs().max() > 1e-3


def check_mixed_layers(rank, world, mods):
    """A ladder-family model whose config lists `ladder_layers` (some layers dense): the engine's
    hybrid step list against the oracle, prompt pass and two decode steps."""
    import dataclasses
    mod, cls = mods["ladder"]
    for ladder_layers in ([1, 2], [0, 2], []):
        cfg = dataclasses.replace(gu.tiny_config("ladder"), ladder_layers=ladder_layers)
        full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
        kw = gu.preset_kwargs(cfg)
        kw["ladder_layers"] = ladder_layers
        mod.transformer_configs["tiny-mixed"] = kw
        model = cls.from_name("tiny-mixed").to(torch.float32).eval()
        gu.load_shards(model, "ladder", cfg, full, rank, world, torch.float32)
        model.setup_caches(max_batch_size=gu.BATCH, max_seq_length=gu.PROMPT + gu.NEW)
        model._engine.ops = CpuOps
        oracle = lo.OracleModel("ladder", cfg, full, world, torch.float32, gu.BATCH, gu.PROMPT + gu.NEW)
        g = torch.Generator().manual_seed(21)
        idx, pos = torch.randint(0, cfg.vocab_size, (gu.BATCH, gu.PROMPT), generator=g), torch.arange(gu.PROMPT)
        for n in range(3):
            got, want = model(idx, pos), oracle.forward(idx, pos)
            err = gu.rel_err(got, want)
            assert err < 2e-5, f"ladder_layers={ladder_layers} rank {rank} step {n}: {err}"
            idx = want[:, -1].argmax(-1, keepdim=True)
            pos = torch.tensor([gu.PROMPT + n], dtype=torch.int32)


def main():
    rank, world = dist.get_rank(), dist.get_world_size()
    mods = {"ladder": (gpt_ladder_TP, gpt_fast.GPTLadder), "dense": (gpt_dense_TP, gpt_fast.GPTDense),
            "parallel": (gpt_parallel_TP, gpt_fast.GPTParallel), "desync": (gpt_desync_TP, gpt_fast.GPTDesync)}
    gold = gu.load(world)
    assert make_comm().world == world
    for family in gu.FAMILIES:
        for dtype_name, tp, init in gu.VARIANTS:
            if tp != world:
                continue
            dtype = getattr(torch, dtype_name)
            cfg = gu.tiny_config(family)
            full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS[init])
            mod, cls = mods[family]
            kw = gu.preset_kwargs(cfg)
            if family == "desync":
                kw["reduce_pattern"] = cfg.reduce_pattern
            mod.transformer_configs["tiny-golden"] = kw
            model = cls.from_name("tiny-golden").to(dtype).eval()
            # per-rank parameter layout (the reference's sharding scheme)
            att = model.layers[0].attention
            nq = (cfg.n_head + 2 * cfg.n_local_heads) * cfg.head_dim // world
            if family == "parallel":
                assert tuple(att.wqkv1.weight.shape) == (nq + 2 * cfg.intermediate_size // world, cfg.dim)
                assert tuple(att.w2.weight.shape) == (cfg.dim, cfg.intermediate_size // world)
            else:
                assert tuple(att.wqkv.weight.shape) == (nq, cfg.dim)
                assert tuple(model.layers[0].feed_forward.w1.weight.shape) == (2 * cfg.intermediate_size // world, cfg.dim)
            assert tuple(att.wo.weight.shape) == (cfg.dim, cfg.dim // world)
            gu.load_shards(model, family, cfg, full, rank, world, dtype)
            model.setup_caches(max_batch_size=gu.BATCH, max_seq_length=gu.PROMPT + gu.NEW)
            assert tuple(att.kv_cache.k_cache.shape) == (gu.BATCH, cfg.n_local_heads // world, 24, cfg.head_dim)
            model._engine.ops = CpuOps
            key = f"{family}-{dtype_name}-tp{tp}-{init}"
            steps, prefill_row0 = gu.replay(model.forward, gold, key)
            ref = torch.from_numpy(gold[key + "/logits"])
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            if family != "desync" or rank == 0:
                err = gu.rel_err(steps, ref)
                assert err < tol, f"{key} rank {rank}: {err}"
                assert gu.rel_err(prefill_row0, gold[key + "/prefill_row0"]) < tol
            if family != "desync":
                # vocabulary-parallel greedy head: same token as the arg-max of the replicated logits
                fed = torch.from_numpy(gold[key + "/fed"])
                n = gu.NEW - 2
                tok = model.decode_greedy(fed[:, n:n + 1], torch.tensor([gu.PROMPT + n], dtype=torch.int32))
                want = steps[-1].argmax(-1).to(torch.int32).view(-1, 1)
                assert torch.equal(tok, want), f"{key} rank {rank}: greedy {tok.flatten().tolist()} vs {want.flatten().tolist()}"
                # vocabulary-parallel sampling: the reference's rule on the full logits, same noise
                last = steps[-1].to(dtype)
                for temperature, top_k in ((1.0, None), (0.7, 5), (1.3, 40), (1.0, 1), (1.0, 10 ** 6)):
                    got = model.decode_sample(fed[:, n:n + 1], torch.tensor([gu.PROMPT + n], dtype=torch.int32),
                                              temperature, top_k, generator=torch.Generator().manual_seed(11))
                    ref_tok, _ = lo.sample(last, temperature, top_k, generator=torch.Generator().manual_seed(11))
                    assert torch.equal(got, ref_tok), f"{key} rank {rank} T={temperature} k={top_k}: " \
                                                      f"{got.flatten().tolist()} vs {ref_tok.flatten().tolist()}"
    check_hf_checkpoint(rank, world, mods)
    check_mixed_layers(rank, world, mods)
    dist.barrier()
    if rank == 0:
        print("ENGINE-CPU-OK")


if __name__ == "__main__":
    main()
