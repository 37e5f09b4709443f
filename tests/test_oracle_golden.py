"""The CPU oracle against outputs of the reference itself (fixtures in tests/golden/)."""
import pytest
import torch

import golden_util as gu
from oracle import ladder_oracle as lo


@pytest.mark.parametrize("family", gu.FAMILIES)
@pytest.mark.parametrize("dtype_name,tp,init", gu.VARIANTS)
def test_model_matches_reference(family, dtype_name, tp, init):
    gold = gu.load(tp)
    key = f"{family}-{dtype_name}-tp{tp}-{init}"
    dtype = getattr(torch, dtype_name)
    cfg = gu.tiny_config(family)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS[init])
    model = lo.OracleModel(family, cfg, full, tp, dtype, gu.BATCH, gu.PROMPT + gu.NEW)
    steps, prefill_row0 = gu.replay(model.forward, gold, key)
    ref = torch.from_numpy(gold[key + "/logits"])
    # fp32: only summation order differs (observed <= 1.2e-6).  bf16: same rounding points, but the
    # reference's matmul/SDPA kernels accumulate in another order and its all-reduce rounds per hop
    # (observed: 1.41e-2 under the loud init, whose activations are 10x larger, 2.4e-3 under the
    # benchmark's quiet init).  Bounds = observed + margin for another host's BLAS summation order.
    tol = 5e-6 if dtype == torch.float32 else (1.8e-2 if init == "loud" else 5e-3)
    assert gu.rel_err(steps, ref) < tol
    assert gu.rel_err(prefill_row0, gold[key + "/prefill_row0"]) < tol
    # top-1: every row whose reference margin (top-1 minus top-2) exceeds the tolerance must agree
    # (observed: all rows agree in all 16 cases)
    top2 = ref.topk(2, dim=-1).values
    decided = (top2[..., 0] - top2[..., 1]) > tol * ref.abs().amax(dim=-1)
    same = steps.argmax(-1) == ref.argmax(-1)
    assert bool(same[decided].all())
    assert same.float().mean().item() >= (1.0 if dtype == torch.float32 else 0.95)


def test_schedules_are_told_apart_by_loud_init():
    """Under the benchmark's N(0, 0.02) init ladder and dense logits sit inside the parity
    tolerance of each other; the loud init separates them, so a parity test on it would
    catch an engine that ran the wrong schedule."""
    gold = gu.load(2)
    a = torch.from_numpy(gold["ladder-float32-tp2-loud/logits"])
    b = torch.from_numpy(gold["dense-float32-tp2-loud/logits"])
    assert gu.rel_err(a, b) > 0.3


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_ops_match_reference(dtype_name):
    gold = gu.load(1)
    dtype = getattr(torch, dtype_name)
    p = f"ops/{dtype_name}/"
    x = torch.from_numpy(gold[p + "rms_x"]).to(dtype)
    w = torch.from_numpy(gold[p + "rms_w"]).to(dtype)
    y = lo.rmsnorm(x, w, 1e-5).float()
    assert torch.equal(y, torch.from_numpy(gold[p + "rms_y"]))
    cfg = lo.OracleConfig(block_size=64, n_head=4, dim=256, rope_base=500000)
    table = lo.rope_table(cfg, dtype)
    ref_table = torch.from_numpy(gold[p + "rope_table"])
    assert (table.float() - ref_table).abs().max().item() <= (1e-6 if dtype == torch.float32 else 2 ** -8)
    scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    cfg2 = lo.OracleConfig(block_size=32, n_head=2, dim=256, rope_base=500000, rope_scaling=scaling)
    t2 = lo.rope_table(cfg2, dtype).float()
    assert (t2 - torch.from_numpy(gold[p + "rope_table_scaled"])).abs().max().item() <= (
        1e-6 if dtype == torch.float32 else 2 ** -8)
    q = torch.from_numpy(gold[p + "rope_x"]).to(dtype)
    out = lo.rope(q, ref_table[3:9].to(dtype)).float()
    assert torch.equal(out, torch.from_numpy(gold[p + "rope_y"]))


def _hf_ladder_literal(model, idx, pos, ladder_layers):
    """The reference's Hugging Face ladder model, transcribed with its own state variables
    (hf_modeling_utils/modeling_llama_ladder.py:627-663 per layer, 889-948 for the loop):
    `hidden` is the previous layer's mlp_output, `prev_attn` its attn_output."""
    cfg = model.cfg
    hidden = model.emb[idx.long()]
    prev_attn = hidden
    for i in range(cfg.n_layer):
        if i not in ladder_layers:
            attn = lo.all_reduce([model._attn(r, i, hidden, pos) for r in range(model.t)])
            hidden = hidden + attn
            attn_out = hidden
            mlp = lo.all_reduce([model._mlp(r, i, hidden) for r in range(model.t)])
            mlp_out = hidden + mlp
        else:
            prev_mlp = hidden
            attn = lo.all_reduce([model._attn(r, i, prev_attn, pos) for r in range(model.t)])
            attn_out = prev_mlp + attn
            mlp = lo.all_reduce([model._mlp(r, i, prev_mlp) for r in range(model.t)])
            mlp_out = attn_out + mlp
        hidden, prev_attn = mlp_out, attn_out
    return model._logits(hidden)


@pytest.mark.parametrize("ladder_layers", [[], [1, 2], [0, 2], [0, 1, 2], 2])
@pytest.mark.parametrize("tp", [1, 2])
def test_mixed_ladder_and_dense_layers(ladder_layers, tp):
    """Checkpoints with `ladder_layers`: the oracle's residual-plus-pending-addends form against a
    transcription of the reference's Hugging Face loop; all layers listed is the pinned ladder
    schedule, none the pinned dense one."""
    import dataclasses
    base = gu.tiny_config("ladder")
    cfg = dataclasses.replace(base, ladder_layers=ladder_layers)
    full = lo.make_full_weights(cfg, gu.SEED, **gu.INITS["loud"])
    model = lo.OracleModel("ladder", cfg, full, tp, torch.float32, gu.BATCH, gu.PROMPT + gu.NEW)
    lit = lo.OracleModel("ladder", cfg, full, tp, torch.float32, gu.BATCH, gu.PROMPT + gu.NEW)
    g = torch.Generator().manual_seed(9)
    x = torch.randint(0, cfg.vocab_size, (gu.BATCH, gu.PROMPT), generator=g)
    pos = torch.arange(gu.PROMPT)
    got = model.forward(x, pos)
    want = _hf_ladder_literal(lit, x, pos, set(cfg.ladder_layers))
    assert gu.rel_err(got, want) < 1e-5
    tok = want[:, -1].argmax(-1, keepdim=True)
    p1 = torch.tensor([gu.PROMPT])
    assert gu.rel_err(model.forward(tok, p1), _hf_ladder_literal(lit, tok, p1, set(cfg.ladder_layers))) < 1e-5
    if len(cfg.ladder_layers) == cfg.n_layer:
        pinned = lo.OracleModel("ladder", base, full, tp, torch.float32, gu.BATCH, gu.PROMPT + gu.NEW)
        assert torch.equal(pinned.forward(x, pos), got)
    if len(cfg.ladder_layers) == 0:
        pinned = lo.OracleModel("dense", base, full, tp, torch.float32, gu.BATCH, gu.PROMPT + gu.NEW)
        assert gu.rel_err(pinned.forward(x, pos), got) < 1e-6
