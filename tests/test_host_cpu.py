"""CPU tests: the C-ABI library loads and exports what the header declares, presets resolve to the
reference's shapes, and the engine's schedules (with a CPU stand-in for the device ops) reproduce
the oracle at TP = 1 in-process and at TP = 2 over gloo."""
import json
import os
import re
import subprocess
import sys

import pytest
import torch

import golden_util as gu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from gpt_fast import _C
    header = open(os.path.join(ROOT, "include", "lri_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(lri_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(_C.lib, name), f"{name} is declared in include/lri_b200.h but not exported"
    assert declared == set(_C.EXPORTED_SYMBOLS), "ctypes signature table and header disagree"
    assert _C.lib.lri_version() >= 100


def test_argument_checks_need_no_gpu():
    from gpt_fast import _C
    rc = _C.lib.lri_linear(0, None, None, None, None, 1, 8, 8, None, 0, None)
    assert rc == -1 and b"NULL" in _C.lib.lri_last_error()
    rc = _C.lib.lri_add_rmsnorm(7, 16, None, None, 1.0, None, 0.0, 16, None, 1, 8, None)
    assert rc == -3
    assert _C.lib.lri_qkv_workspace_bytes(4, 8, 2, 128) == 0
    assert _C.lib.lri_qkv_workspace_bytes(100, 8, 2, 128) == 100 * 12 * 128 * 2
    assert _C.lib.lri_gateup_workspace_bytes(100, 512) == 100 * 1024 * 2


def _streamk_plan(M, N, K):
    import ctypes
    from gpt_fast import _C
    out = [ctypes.c_int() for _ in range(5)]
    _C.check(_C.lib.lri_streamk_plan(M, N, K, *[ctypes.byref(o) for o in out]))
    return [o.value for o in out]


@pytest.mark.parametrize("N", [8, 128, 136, 1000, 4096, 6144, 14336, 28672, 53248, 128256])
@pytest.mark.parametrize("K", [8, 64, 72, 512, 4096, 14336, 53248])
def test_streamk_plan_keeps_every_tile_within_its_workspace(N, K):
    """The kernel deals (tile, K tile) pairs out to CTAs in equal contiguous runs and stores the
    piece of a tile that a CTA holds in slot (CTA - first CTA of the tile) of the tile's workspace.
    For every shape the plan must keep that slot below the capacity it sized the workspace for, every
    CTA must get work, and the pieces of a tile must add up to its whole K range."""
    from gpt_fast import _C
    for M in (9, 16, 33, 64):
        tiles, kt, max_seg, ctas, tok = _streamk_plan(M, N, K)
        assert tiles == -(-N // 128) and kt == -(-K // 64) and tok == (16 if M <= 16 else 32 if M <= 32 else 64)
        assert 2 <= max_seg <= 8 and 1 <= ctas <= 148
        assert _C.lib.lri_linear_workspace_bytes(M, N) == tiles * max_seg * tok * 128 * 4
        assert _C.lib.lri_gateup_workspace_bytes(M, N) == 2 * tiles * max_seg * tok * 128 * 4
    units = tiles * kt
    start = [units * b // ctas for b in range(ctas + 1)]            # the kernel's unit_start()
    cta_of = lambda u: ((u + 1) * ctas - 1) // units                # the kernel's cta_of_unit()
    assert all(start[b + 1] > start[b] for b in range(ctas))
    covered = [0] * tiles
    for b in range(ctas):
        u = start[b]
        while u < start[b + 1]:
            t, k0 = divmod(u, kt)
            nk = min(kt - k0, start[b + 1] - u)
            first, last = cta_of(t * kt), cta_of((t + 1) * kt - 1)
            assert first <= b <= last and last - first + 1 <= max_seg, (N, K, b, t, first, last, max_seg)
            covered[t] += nk
            u += nk
    assert covered == [kt] * tiles


def test_workspace_sizes():
    from gpt_fast import _C
    lib = _C.lib
    # up to 8 rows: streaming kernels, no workspace; 9..64: stream-K partial tiles; above: raw projection
    assert lib.lri_linear_workspace_bytes(8, 4096) == 0 and lib.lri_linear_workspace_bytes(65, 4096) == 0
    assert lib.lri_linear_workspace_bytes(9, 4096) == lib.lri_linear_workspace_bytes(16, 4096) > 0
    assert lib.lri_gateup_workspace_bytes(8, 14336) == 0
    assert lib.lri_gateup_workspace_bytes(16, 14336) == 112 * 3 * 2 * 16 * 128 * 4
    assert lib.lri_qkv_workspace_bytes(16, 32, 8, 128) == 48 * 5 * 16 * 128 * 4
    assert lib.lri_qkv_workspace_bytes(65, 32, 8, 128) == 65 * 48 * 128 * 2
    rc = lib.lri_streamk_plan(65, 4096, 4096, None, None, None, None, None)
    assert rc == -1


def test_decode_splits_choice():
    """Number of position ranges of decode attention: fixed per cache geometry (never a function of
    the current position), a power of two up to 8 for the cluster kernel, up to 64 ranges of at
    least 64 positions for long caches, and one or two ranges once the tensor-core kernel takes over."""
    from gpt_fast import _C
    from gpt_fast.ops import decode_splits
    _C.check(_C.lib.lri_set_option(b"attn_mma", -1))
    _C.check(_C.lib.lri_set_option(b"decode_splits", 0))
    for B in (1, 2, 4, 8):
        for nh, nkv in ((32, 8), (64, 8), (8, 1), (4, 4)):
            for smax in (64, 256, 1288, 8192, 131072):
                n = decode_splits(B, nh, nkv, smax)
                assert 1 <= n <= 64 and smax // n >= 32
                assert n in (1, 2, 4, 8, 16) or smax // n >= 64
    assert decode_splits(1, 32, 8, 1288) == 8          # 8B, batch 1: one cluster of 8 CTAs per head tile
    assert decode_splits(1, 4, 1, 1288) == 16          # a one-KV-head shard (TP=8): a single cluster, 16 CTAs
    assert decode_splits(16, 32, 8, 1288) == 2          # 128 (sequence, KV head) pairs: tensor-core kernel, two ranges
    assert decode_splits(64, 32, 8, 1288) == 1          # 512 pairs: one range each
    assert decode_splits(64, 4, 1, 1288) == 4           # TP=8 shard: below 128 pairs, the cluster kernel
    # single sequence: up to four clusters (query heads spread over them) take the 16-CTA cluster, eight do not
    assert [decode_splits(1, 32 // t, 8 // t, 1288) for t in (1, 2, 4, 8)] == [8, 16, 16, 16]
    try:
        _C.check(_C.lib.lri_set_option(b"attn_mma", 0))
        assert decode_splits(64, 32, 8, 1288) == 1 and decode_splits(16, 32, 8, 1288) == 2   # the cluster kernel's own choice
        _C.check(_C.lib.lri_set_option(b"decode_splits", 5))
        assert decode_splits(3, 32, 8, 1288) == 5
    finally:
        _C.check(_C.lib.lri_set_option(b"attn_mma", -1))
        _C.check(_C.lib.lri_set_option(b"decode_splits", 0))


def test_options_table():
    """Tuning options are one table behind the C ABI: readable, settable, range-checked."""
    import ctypes
    from gpt_fast import _C
    v = ctypes.c_int(-99)
    _C.check(_C.lib.lri_get_option(b"stream_rows", ctypes.byref(v)))
    assert v.value == 8
    assert _C.lib.lri_set_option(b"stream_rows", 17) == -1 and _C.lib.lri_set_option(b"no_such_option", 1) == -1
    assert _C.lib.lri_set_option(b"gemv_rows_per_cta", 3) == -1
    assert _C.lib.lri_set_option(b"attn_head_tile", 3) == -1 and _C.lib.lri_set_option(b"attn_head_tile", 2) == 0
    _C.check(_C.lib.lri_set_option(b"attn_head_tile", 0))
    _C.check(_C.lib.lri_set_option(b"stream_rows", 4))
    _C.check(_C.lib.lri_get_option(b"stream_rows", ctypes.byref(v)))
    assert v.value == 4
    assert _C.lib.lri_linear_workspace_bytes(8, 4096) > 0   # 8 rows now belong to the stream-K kernel
    _C.check(_C.lib.lri_set_option(b"stream_rows", 8))
    assert _C.lib.lri_linear_workspace_bytes(8, 4096) == 0


def test_bench_roofline_arithmetic():
    """Algorithmic bytes per decode step and FLOPs per prompt pass, per rank, for the benchmark's
    shapes: weights once (layer shards, norms, replicated LM head) plus the valid KV cache."""
    sys.path.insert(0, ROOT)
    import bench
    a8, a70 = bench.shape_of("llama-3-8b", "ladder"), bench.shape_of("llama-3-70b", "ladder")
    assert [round(bench.step_bytes(a8, t, 1, 0) / 1e9, 2) for t in (1, 2, 4, 8)] == [15.01, 8.03, 4.54, 2.80]
    assert [round(bench.step_bytes(a70, t, 1, 0) / 1e9, 1) for t in (1, 2, 4, 8)] == [139.0, 70.6, 36.3, 19.2]
    # one cached position of one sequence, all ranks: 2 (K, V) * L * n_kv * hd * 2 bytes
    assert bench.step_bytes(a8, 1, 1, 1) - bench.step_bytes(a8, 1, 1, 0) == 131072
    assert bench.step_bytes(a70, 1, 1, 1) - bench.step_bytes(a70, 1, 1, 0) == 327680
    # vocabulary-parallel head: the LM head's bytes divide by the ranks
    full, split = bench.step_bytes(a8, 8, 1, 0), bench.step_bytes(a8, 8, 1, 0, head_split=True)
    assert full - split == 2 * 128256 * 4096 * 7 // 8
    # prompt pass of 32 x 4096 tokens at TP=8: projections + causal attention + LM head on every position
    assert round(bench.prefill_flops(a8, 8, 32, 4096) / 1e12, 1) == 384.0


def test_no_cpu_fallback():
    """The product must refuse CPU tensors instead of computing somewhere else."""
    from gpt_fast.utils import RMSNorm
    with pytest.raises((RuntimeError, TypeError)):
        RMSNorm(64)(torch.zeros(2, 64, dtype=torch.bfloat16))


def test_presets_match_reference_tables():
    import gpt_fast  # noqa: F401
    from gpt_fast import gpt_dense_TP, gpt_desync_TP, gpt_ladder_TP, gpt_parallel_TP
    ref = json.load(open(os.path.join(gu.GOLDEN_DIR, "reference_presets.json")))
    mods = {"ladder": gpt_ladder_TP, "dense": gpt_dense_TP, "parallel": gpt_parallel_TP, "desync": gpt_desync_TP}
    for family, table in ref.items():
        for name, fields in table.items():
            args = mods[family].ModelArgs.from_name(name)
            for k, v in fields.items():
                assert getattr(args, k) == v, f"{family}:{name}.{k}"


def test_baseline_shapes_have_presets():
    from gpt_fast.gpt_ladder_TP import ModelArgs
    a = ModelArgs.from_name("ladder-llama-1b")
    assert (a.dim, a.n_layer, a.n_head, a.n_local_heads, a.head_dim, a.intermediate_size, a.rope_base) == (
        2048, 16, 32, 8, 64, 8192, 500000)
    a = ModelArgs.from_name("ladder-llama-405b-kv8")
    assert (a.dim, a.n_layer, a.n_head, a.n_local_heads, a.head_dim) == (16384, 126, 128, 8, 128)
    with pytest.raises(KeyError):
        ModelArgs.from_name("no-such-preset")


def test_rope_table_matches_reference_fixture():
    from gpt_fast.utils import precompute_freqs_cis
    gold = gu.load(1)
    for name, dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        t = precompute_freqs_cis(64, 64, 500000, dtype)
        assert (t.float() - torch.from_numpy(gold[f"ops/{name}/rope_table"])).abs().max() <= (
            1e-6 if dtype == torch.float32 else 2 ** -8)
        scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
        t = precompute_freqs_cis(32, 128, 500000, dtype, scaling)
        assert (t.float() - torch.from_numpy(gold[f"ops/{name}/rope_table_scaled"])).abs().max() <= (
            1e-6 if dtype == torch.float32 else 2 ** -8)


@pytest.mark.parametrize("world", [1, 2])
def test_engine_schedules_on_cpu_ranks(world):
    """Runs tests/engine_cpu_worker.py as `world` gloo ranks; each checks all four schedules
    against the golden fixtures of the reference for that TP degree."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29730 + world),
           os.path.join(ROOT, "tests", "engine_cpu_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ENGINE-CPU-OK" in r.stdout


def test_message_size_threshold_and_elided_comm():
    """Host logic of the communicator module: the peer-kernel / NCCL size threshold per world size (from the
    measured latency table) and the comm-elided stand-in used to measure the exposed all-reduce time."""
    from gpt_fast.comm import ElidedComm, p2p_max_bytes
    assert p2p_max_bytes(2) == 8 << 20 and p2p_max_bytes(4) == 2 << 20 and p2p_max_bytes(8) == 1 << 20
    # every decode message of the benchmark configurations stays on the peer kernels at 8 ranks
    for batch, dim in ((1, 4096), (16, 4096), (64, 8192), (16, 16384)):
        assert batch * dim * 2 <= p2p_max_bytes(8)

    class Like:
        handle, timeout_ms = object(), 123

    e = ElidedComm(8, 3, like=Like)
    assert (e.world, e.rank, e.handle, e.timeout_ms) == (8, 3, Like.handle, 123)
    assert e.all_reduce_async(None) is None and e.wait(None) is None and not e.can_split(8, 1)
    assert e.reduce_mode(4096, 1, hidden=True) == "kernel"


def test_reduce_mode_selection():
    """How a row-parallel partial becomes a sum, by LRI_SPLIT_AR value, message size and schedule: the stand-alone
    all-reduce kernel, the split form (single-row decode only) or the one-kernel form (any rows while the message
    fits a push channel)."""
    from gpt_fast.comm import P2PComm

    class Stub:
        _push_max = 64 * 1024
        can_split = P2PComm.can_split
        reduce_mode = P2PComm.reduce_mode

        def __init__(self, mode, world=2):
            self.split_mode, self.world = mode, world

    auto, off, on, fused = Stub("auto"), Stub("0"), Stub("1"), Stub("fused")
    assert auto.reduce_mode(4096, 1, hidden=True) == "kernel"      # ladder: hidden behind the other sublayer
    assert auto.reduce_mode(4096, 1, hidden=False) == "split"      # dense / parallel single-row decode
    assert auto.reduce_mode(16 * 4096, 16, hidden=False) == "kernel"
    assert Stub("auto", world=8).reduce_mode(4096, 1, hidden=False) == "kernel"   # the gathering norm polls peer by peer
    assert Stub("1", world=8).reduce_mode(4096, 1, hidden=False) == "split"
    assert off.reduce_mode(4096, 1) == "kernel"
    assert on.reduce_mode(4096, 1, hidden=True) == "split" and on.reduce_mode(2 * 4096, 2, hidden=True) == "kernel"
    assert fused.reduce_mode(4096, 1, hidden=True) == "fused" and fused.reduce_mode(16 * 4096, 16) == "fused"
    assert fused.reduce_mode(16384 * 4096, 16384) == "kernel"      # a prompt pass does not fit a push channel
    assert fused.reduce_mode(4100, 1) == "kernel"                  # not a multiple of 8 elements
    assert not fused.can_split(4096, 1)


def test_model_args_from_hf_config(tmp_path):
    """config.json of a Hugging Face Llama / LlamaLadder checkpoint -> ModelArgs keyword arguments, with the
    reference's normalisation of `ladder_layers` (an int means the last n layers)."""
    import json
    from gpt_fast.loader import model_args_from_hf_config
    cfg = dict(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=6, num_attention_heads=4,
               num_key_value_heads=2, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=4096,
               rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192), ladder_layers=2)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    kw = model_args_from_hf_config(str(tmp_path))
    assert kw["ladder_layers"] == [4, 5] and kw["n_local_heads"] == 2 and kw["block_size"] == 4096
    assert kw["rope_scaling"]["factor"] == 8.0 and "rope_type" not in kw["rope_scaling"]
    from gpt_fast import gpt_ladder_TP
    args = gpt_ladder_TP.ModelArgs(**kw)
    assert args.ladder_layers == [4, 5] and args.head_dim == 64
    cfg.pop("ladder_layers")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert "ladder_layers" not in model_args_from_hf_config(str(tmp_path / "config.json"))
