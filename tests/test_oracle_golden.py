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
