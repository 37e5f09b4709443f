"""Whole-model parity on one GPU (TP = 1): the drop-in package against fixtures produced by the
reference itself and against the CPU oracle, for all four schedules, prefill and teacher-forced
decode.  Tolerance from the task statement: logits within 2e-2 relative error and >= 99 % top-1
agreement (on steps whose reference top-1 margin exceeds the tolerance)."""
import pytest
import torch

import golden_util as gu
from oracle import ladder_oracle as lo

pytestmark = pytest.mark.gpu


def _family_module(family):
    import gpt_fast
    from gpt_fast import gpt_dense_TP, gpt_desync_TP, gpt_ladder_TP, gpt_parallel_TP
    return {"ladder": (gpt_ladder_TP, gpt_fast.GPTLadder), "dense": (gpt_dense_TP, gpt_fast.GPTDense),
            "parallel": (gpt_parallel_TP, gpt_fast.GPTParallel), "desync": (gpt_desync_TP, gpt_fast.GPTDesync)}[family]


def build_model(family, cfg, full, dtype, batch, max_seq, name="test-preset"):
    mod, cls = _family_module(family)
    kw = gu.preset_kwargs(cfg)
    if family == "desync":
        kw.update(reduce_pattern=cfg.reduce_pattern, force_disable_last_all_reduce=cfg.force_disable_last_all_reduce)
    mod.transformer_configs[name] = kw
    with torch.device("meta"):
        model = cls.from_name(name)
    model = model.to(dtype=dtype).to_empty(device="cuda").eval()
    gu.load_shards(model, family, cfg, full, 0, 1, dtype)
    model.setup_caches(max_batch_size=batch, max_seq_length=max_seq)
    return model


def _cuda_forward(model):
    def fwd(idx, pos):
        with torch.no_grad():
            return model(idx.cuda(), pos.cuda())
    return fwd


def _top1_agreement(got, ref, margin_tol):
    """Share of rows with equal argmax among rows whose reference top-1 margin is above the
    numeric tolerance (a near-tie can flip legitimately)."""
    top2 = ref.topk(2, dim=-1).values
    decided = (top2[..., 0] - top2[..., 1]) > margin_tol * ref.abs().amax(dim=-1)
    same = got.argmax(-1) == ref.argmax(-1)
    return same[decided].float().mean().item() if decided.any() else 1.0


@pytest.mark.parametrize("family", gu.FAMILIES)
@pytest.mark.parametrize("init", ["loud", "quiet"])
def test_matches_reference_fixture_and_oracle(family, init):
    """bf16, TP=1.  The `loud` fixture was produced by the reference in bf16; for `quiet` the
    fixture is the reference's fp32 run, which a bf16 engine must approach as closely as the
    reference's own bf16 path does (about 1e-2)."""
    gold = gu.load(1)
    cfg = gu.tiny_config(family)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS[init])
    model = build_model(family, cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
    key = f"{family}-bfloat16-tp1-loud" if init == "loud" else f"{family}-float32-tp1-quiet"
    steps, prefill_row0 = gu.replay(_cuda_forward(model), gold, key)
    ref = torch.from_numpy(gold[key + "/logits"])
    assert torch.isfinite(steps).all()
    err = gu.rel_err(steps, ref)
    assert err < 2e-2, f"{key}: relative error {err:.3e}"
    assert gu.rel_err(prefill_row0, gold[key + "/prefill_row0"]) < 2e-2
    assert _top1_agreement(steps, ref, 2e-2) >= 0.99
    # and against the oracle run with the same dtype on the same teacher-forced tokens
    oracle = lo.OracleModel(family, cfg, full, 1, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
    osteps, _ = gu.replay(oracle.forward, gold, key)
    assert gu.rel_err(steps, osteps) < 2e-2


def test_schedules_differ_on_gpu():
    """With the loud init the ladder and dense engines must be far apart: an engine that ran the
    wrong schedule would still pass the 2e-2 parity test under the quiet init."""
    gold = gu.load(1)
    out = {}
    for family in ("ladder", "dense"):
        cfg = gu.tiny_config(family)
        full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
        model = build_model(family, cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
        out[family], _ = gu.replay(_cuda_forward(model), gold, "ladder-bfloat16-tp1-loud")
    assert gu.rel_err(out["ladder"], out["dense"]) > 0.3


MEDIUM = dict(block_size=512, vocab_size=4096, n_layer=4, n_head=8, n_local_heads=2, dim=1024, intermediate_size=2816,
              rope_base=500000)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("family", ["ladder", "parallel"])
def test_medium_shape_head_dim_128(dtype, family):
    """head_dim 128, GQA group 4, prompt of 150 tokens x batch 2 (300 rows: the prefill GEMM and
    flash-attention paths with ragged tiles), then 3 decode steps; against the fp32 oracle."""
    cfg = lo.OracleConfig(**MEDIUM)
    full = lo.make_full_weights(cfg, 77, std=0.05, norm_mean=1.0, norm_std=0.1)
    B, T, NEW = 2, 150, 4
    model = build_model(family, cfg, full, dtype, B, T + NEW, name="medium")
    same = lo.OracleModel(family, cfg, full, 1, dtype, B, T + NEW)       # same storage type: the parity bar
    exact = lo.OracleModel(family, cfg, full, 1, torch.float32, B, T + NEW)  # fp32: how far 16-bit storage is
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (T,), generator=g)
    x = prompt.view(1, -1).repeat(B, 1)
    fwd = _cuda_forward(model)
    # 2e-2 against the path with the same storage type (the task's tolerance); against fp32 the
    # error is that of 16-bit storage itself, which the same-dtype oracle shows too
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3

    def check(got, idx, pos, what):
        ref_same, ref_exact = same.forward(idx, pos).float(), exact.forward(idx, pos)
        assert gu.rel_err(got, ref_same) < tol, what
        assert gu.rel_err(got, ref_exact) < 1.5 * max(gu.rel_err(ref_same, ref_exact), tol / 2), what
        return ref_exact

    ref = check(fwd(x, torch.arange(T)).float().cpu(), x, torch.arange(T), "prefill")
    tok = ref[:, -1].argmax(-1, keepdim=True)
    for n in range(NEW - 1):
        pos = torch.tensor([T + n], dtype=torch.int32)
        ref = check(fwd(tok.to(torch.int32), pos).float().cpu(), tok, pos, f"decode step {n}")
        tok = ref[:, -1].argmax(-1, keepdim=True)


def test_decode_step_in_cuda_graph_follows_device_position():
    """A captured decode step must stay correct when the caller advances the position tensor in
    place between replays (the reference's benchmark driver does exactly that)."""
    gold = gu.load(1)
    family, key = "ladder", "ladder-bfloat16-tp1-loud"
    cfg = gu.tiny_config(family)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
    model = build_model(family, cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
    prompt = torch.from_numpy(gold[key + "/prompt"])
    fed = torch.from_numpy(gold[key + "/fed"])
    ref = torch.from_numpy(gold[key + "/logits"])
    x = prompt.view(1, -1).repeat(gu.BATCH, 1).cuda()
    with torch.no_grad():
        model(x, torch.arange(gu.PROMPT, device="cuda"))
        static_tok = fed[:, 0:1].to(torch.int32).cuda()
        static_pos = torch.tensor([gu.PROMPT], dtype=torch.int32, device="cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                model(static_tok, static_pos)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_logits = model(static_tok, static_pos)
        for n in range(gu.NEW - 1):
            static_tok.copy_(fed[:, n:n + 1].to(torch.int32))
            static_pos.fill_(gu.PROMPT + n)
            graph.replay()
            torch.cuda.synchronize()
            assert gu.rel_err(static_logits[:, -1].float().cpu(), ref[n + 1]) < 2e-2, f"replay {n}"


@pytest.mark.parametrize("family", ["ladder", "dense", "parallel"])
def test_decode_greedy_and_decode_sample_match_the_rule_on_the_logits(family):
    """decode_greedy / decode_sample (vocabulary-split head; one rank here) against the arg-max and the
    reference's sampling rule applied to the logits of the same step, same noise."""
    gold = gu.load(1)
    key = f"{family}-bfloat16-tp1-loud"
    cfg = gu.tiny_config(family)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
    model = build_model(family, cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
    prompt = torch.from_numpy(gold[key + "/prompt"])
    fed = torch.from_numpy(gold[key + "/fed"])
    x = prompt.view(1, -1).repeat(gu.BATCH, 1).cuda()
    with torch.no_grad():
        model(x, torch.arange(gu.PROMPT, device="cuda"))
        tok = fed[:, 0:1].cuda()
        pos = torch.tensor([gu.PROMPT], dtype=torch.int32, device="cuda")
        logits = model(tok, pos)[:, -1]
        assert torch.equal(model.decode_greedy(tok, pos).cpu(), logits.float().argmax(-1, keepdim=True).to(torch.int32).cpu())
        for temperature, top_k in ((1.0, None), (0.7, 5), (1.0, 1)):
            torch.manual_seed(11)
            got = model.decode_sample(tok, pos, temperature, top_k)
            torch.manual_seed(11)
            want, _ = lo.sample(logits, temperature, top_k)
            assert torch.equal(got.cpu(), want.cpu()), f"T={temperature} k={top_k}"


@pytest.mark.parametrize("head", ["replicated", "vocab-parallel"])
def test_device_loop_matches_oracle_greedy_generate(head):
    """generate.DeviceLoop (several decode steps per graph replay, token feedback and position on the
    device) against the oracle's greedy generation (benchmark.py:118-164 with top_k = 1).  Free-running
    generations may part ways at a near-tie, so a token may differ only where the oracle's own
    top-1 margin at that step is inside the numeric tolerance; up to there the tokens must be equal,
    and the test requires most of the sequence to be decided that way."""
    from gpt_fast.generate import DeviceLoop
    gold = gu.load(1)
    family, key = "ladder", "ladder-bfloat16-tp1-loud"
    cfg = gu.tiny_config(family)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
    n_new = 7
    prompt = torch.from_numpy(gold[key + "/prompt"])
    x = prompt.view(1, -1).repeat(gu.BATCH, 1).cuda()
    oracle = lo.OracleModel(family, cfg, full, 1, torch.bfloat16, gu.BATCH, gu.PROMPT + n_new + 1)
    want, step_logits = lo.greedy_generate(oracle, prompt, gu.BATCH, n_new + 1)   # [B, n_new + 1], first = prompt pass

    model = build_model(family, cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + n_new + 1, name="test-preset-loop")
    with torch.no_grad():
        first = model(x, torch.arange(gu.PROMPT, device="cuda"))[:, -1].argmax(-1, keepdim=True).to(torch.int32)
    loop = DeviceLoop(model, gu.BATCH, steps_per_replay=4, head=head)
    loop.start(first, gu.PROMPT)
    got = torch.cat([first, loop.run(n_new)], dim=1).cpu().long()
    equal_steps = 0
    for b in range(gu.BATCH):
        for n in range(n_new + 1):
            if got[b, n] == want[b, n]:
                equal_steps += 1
                continue
            lg = step_logits[n][b].float()
            top2 = lg.topk(2).values
            assert (top2[0] - top2[1]).item() <= 2e-2 * lg.abs().max().item(), \
                f"row {b} step {n}: {got[b].tolist()} vs oracle {want[b].tolist()} at a decided step"
            break  # the sequences legitimately differ from here on
    assert equal_steps >= 0.75 * gu.BATCH * (n_new + 1), f"{got.tolist()} vs {want.tolist()}"


def test_module_level_forward_matches_engine():
    """The reference's block-level interface (blocks driven by hand with gathered RoPE rows and a
    mask) gives the same logits as the engine's whole-model forward."""
    cfg = gu.tiny_config("ladder")
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
    model = build_model("ladder", cfg, full, torch.bfloat16, gu.BATCH, gu.PROMPT + gu.NEW)
    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, cfg.vocab_size, (gu.BATCH, gu.PROMPT), generator=g).cuda()
    pos = torch.arange(gu.PROMPT, device="cuda")
    with torch.no_grad():
        want = model(idx, pos).float()
        mask = model.causal_mask[None, None, pos]
        rows = model.freqs_cis[pos]
        x = model.tok_embeddings.weight[idx]
        pa, pm, ha, hm = torch.zeros_like(x), torch.zeros_like(x), None, None
        for layer in model.layers:
            pa, pm, x, ha, hm = layer(pa, pm, x, ha, hm, pos, rows, mask)
        ha.wait()
        hm.wait()
        got = torch.nn.functional.linear(model.norm((x + pa) + pm), model.output.weight).float()
    assert gu.rel_err(got.cpu(), want.cpu()) < 1e-2
