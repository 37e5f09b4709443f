"""Per-kernel parity on the GPU: every fused op, called through the C ABI, against the CPU oracle
on the same seeded inputs.  Tolerances: the kernels keep the oracle's rounding points, so results
differ only by fp32 summation order, i.e. by at most one unit in the last place of the 16-bit
storage type on a small fraction of elements."""
import math

import pytest
import torch

import golden_util as gu
from oracle import ladder_oracle as lo

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16]


def _ops():
    from gpt_fast.ops import CudaOps
    return CudaOps


def _C():
    from gpt_fast import _C as c
    return c


def _ulp_close(got, ref, dtype, ulps=1.0):
    """Every element within `ulps` units in the last place of `dtype`, where the unit is taken at
    the element's own magnitude or, for elements much smaller than typical (results of a
    cancellation), at the tensor's rms magnitude; and the whole tensor within 2e-3 relative error."""
    got, ref = got.float().cpu(), ref.float().cpu()
    assert torch.isfinite(got).all(), "non-finite values in the kernel output"
    eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    rms = ref.pow(2).mean().sqrt().item()
    unit = 2 * eps * torch.maximum(torch.maximum(got.abs(), ref.abs()), torch.full_like(ref, rms))
    ratio = (got - ref).abs() / unit
    worst = ratio.max().item()
    if worst > ulps * 1.01:
        i = ratio.argmax().item()
        bad = (ratio > ulps * 1.01).float().mean().item()
        raise AssertionError(f"worst element error {worst:.2f} ulp (allowed {ulps}) at flat index {i}: got "
                             f"{got.view(-1)[i].item():.6g} ref {ref.view(-1)[i].item():.6g}; {bad:.2%} of elements "
                             f"over; whole-tensor rel err {gu.rel_err(got, ref):.3e}")
    assert gu.rel_err(got, ref) < 2e-3


def _randn(gen, *shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,dim", [(1, 256), (5, 4096), (3, 16384), (2, 264)])
def test_add_rmsnorm(dtype, rows, dim):
    g = torch.Generator().manual_seed(rows * 1000 + dim)
    r, a, b = (_randn(g, rows, dim, scale=1.5, dtype=dtype) for _ in range(3))
    w = (1 + 0.3 * torch.randn(dim, generator=g)).to(dtype)
    ops = _ops()
    rc, ac, bc, wc = r.cuda(), a.cuda(), b.cuda(), w.cuda()
    # two-way add + norm, in place on the residual
    res, normed = rc.clone(), torch.empty_like(rc)
    ops.add_rmsnorm(res, ac, None, wc, 1e-5, res, normed, rows)
    ref_res = r + a
    assert torch.equal(res.cpu(), ref_res)
    _ulp_close(normed, lo.rmsnorm(ref_res, w, 1e-5), dtype, ulps=2)
    # three-way add, norm only output
    normed3 = torch.empty_like(rc)
    ops.add_rmsnorm(rc, ac, bc, wc, 1e-5, None, normed3, rows)
    _ulp_close(normed3, lo.rmsnorm(r + a + b, w, 1e-5), dtype, ulps=2)
    # scaled residual, add only (desync): y + x / t
    out = torch.empty_like(rc)
    ops.add_rmsnorm(rc, ac, None, None, 0.0, out, None, rows, 0.25)
    assert torch.equal(out.cpu(), a + r / 4)
    # norm only
    n0 = torch.empty_like(rc)
    ops.add_rmsnorm(rc, None, None, wc, 1e-5, None, n0, rows)
    _ulp_close(n0, lo.rmsnorm(r, w, 1e-5), dtype, ulps=2)


@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_embedding(idx_dtype):
    g = torch.Generator().manual_seed(3)
    table = _randn(g, 1000, 256)
    idx = torch.randint(0, 1000, (3, 7), generator=g).to(idx_dtype)
    out = torch.empty(21, 256, dtype=torch.bfloat16, device="cuda")
    _ops().embedding(table.cuda(), idx.cuda(), out)
    assert torch.equal(out.cpu(), table[idx.long().view(-1)])


GEMV_SHAPES = [(64, 256), (130, 512), (4096, 4096), (1002, 14336), (256, 72), (6, 8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("n,k", GEMV_SHAPES)
def test_linear_gemv(dtype, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    x, w = _randn(g, m, k, dtype=dtype), _randn(g, n, k, scale=1 / math.sqrt(k), dtype=dtype)
    add = _randn(g, m, n, dtype=dtype)
    y = torch.empty(m, n, dtype=dtype, device="cuda")
    _ops().linear(x.cuda(), w.cuda(), y, m)
    _ulp_close(y, lo.linear(x, w), dtype)
    _ops().linear(x.cuda(), w.cuda(), y, m, addend=add.cuda())
    _ulp_close(y, lo.linear(x, w) + add, dtype, ulps=6)


@pytest.mark.parametrize("rows_per_cta,depth", [(2, 0), (8, 0), (4, 2), (0, 0)])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_linear_gemv_tuning_options(rows_per_cta, depth, m):
    """The streaming kernel's tuning options (weight rows per CTA, loads in flight per thread) change the launch
    shape, not the result: every setting against the oracle, including the short-K shapes for which the library
    itself picks 8 rows per CTA."""
    C = _C()
    try:
        assert C.lib.lri_set_option(b"gemv_rows_per_cta", rows_per_cta) == 0
        assert C.lib.lri_set_option(b"gemv_depth", depth) == 0
        for n, k in [(4096, 512), (1000, 256), (520, 4096), (4096, 1792)]:
            g = torch.Generator().manual_seed(m + n + k)
            x = _randn(g, m, k)
            w = _randn(g, n, k, scale=1 / math.sqrt(k))
            y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            _ops().linear(x.cuda(), w.cuda(), y, m)
            _ulp_close(y, lo.linear(x, w), torch.bfloat16)
            inter = n // 2 // 8 * 8
            h = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
            ws = torch.empty(max(_ops().gateup_workspace_bytes(m, inter), 16), dtype=torch.uint8, device="cuda")
            w1 = (w[: 2 * inter] * 2).contiguous()
            _ops().gateup_swiglu(x.cuda(), w1.cuda(), h, m, ws)
            _ulp_close(h, lo.swiglu(lo.linear(x, w1)), torch.bfloat16, ulps=8)
    finally:
        C.lib.lri_set_option(b"gemv_rows_per_cta", 0)
        C.lib.lri_set_option(b"gemv_depth", 0)


GEMM_M = [9, 16, 24, 33, 64, 65, 128, 200, 300]
GEMM_NK = [(64, 64), (136, 72), (512, 256), (1000, 4096), (384, 1024)]


@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", GEMM_M)
@pytest.mark.parametrize("n,k", GEMM_NK)
def test_linear_gemm(backend, dtype, m, n, k):
    c = _C()
    c.check(c.lib.lri_set_gemm_backend(c.GEMM_TCGEN05 if backend == "tcgen05" else c.GEMM_SIMT))
    try:
        g = torch.Generator().manual_seed(m * 7 + n + k)
        x, w = _randn(g, m, k, dtype=dtype), _randn(g, n, k, scale=1 / math.sqrt(k), dtype=dtype)
        y = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        _ops().linear(x.cuda(), w.cuda(), y, m)
        torch.cuda.synchronize()
        c.check(c.lib.lri_gemm_status())
        _ulp_close(y, lo.linear(x, w), dtype)
    finally:
        c.lib.lri_set_gemm_backend(c.GEMM_AUTO)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [9, 16, 17, 24, 33, 64])
@pytest.mark.parametrize("n,k", GEMM_NK + [(256, 8192), (1024, 7168), (8192, 512), (24000, 256)])
@pytest.mark.parametrize("ws_scale", [1.0, 0.3, 0.0])
def test_linear_streamk(dtype, m, n, k, ws_scale):
    """9..64 rows with a workspace: the tcgen05 stream-K kernel (fp32 partial tiles in the workspace,
    addend applied by the CTA that completes a tile); with a workspace that is too small or
    absent the call falls back to the plain GEMM."""
    c, ops = _C(), _ops()
    g = torch.Generator().manual_seed(m * 11 + n + k)
    x, w = _randn(g, m, k, dtype=dtype), _randn(g, n, k, scale=1 / math.sqrt(k), dtype=dtype)
    add = _randn(g, m, n, dtype=dtype)
    full = ops.linear_workspace_bytes(m, n)
    assert full > 0
    nbytes = int(full * ws_scale) // 16 * 16
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda") if nbytes else None
    y = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    ops.linear(x.cuda(), w.cuda(), y, m, workspace=ws)
    torch.cuda.synchronize()
    c.check(c.lib.lri_gemm_status())
    _ulp_close(y, lo.linear(x, w), dtype)
    ops.linear(x.cuda(), w.cuda(), y, m, addend=add.cuda(), workspace=ws)
    _ulp_close(y, lo.linear(x, w) + add, dtype, ulps=6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 3, 8, 12, 16, 24, 40, 64, 200])
@pytest.mark.parametrize("inter,k", [(512, 256), (1000, 1024), (14336 // 8, 4096)])
def test_gateup_swiglu(dtype, m, inter, k):
    g = torch.Generator().manual_seed(m + inter + k)
    x, w1 = _randn(g, m, k, dtype=dtype), _randn(g, 2 * inter, k, scale=2 / math.sqrt(k), dtype=dtype)
    ops = _ops()
    h = torch.empty(m, inter, dtype=dtype, device="cuda")
    nbytes = ops.gateup_workspace_bytes(m, inter)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda") if nbytes else None
    ops.gateup_swiglu(x.cuda(), w1.cuda(), h, m, ws)
    _ulp_close(h, lo.swiglu(lo.linear(x, w1)), dtype, ulps=8)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,S", [(1, 1), (3, 1), (2, 3), (2, 8), (2, 12), (4, 10), (3, 20), (1, 200)])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (8, 2, 128)])
@pytest.mark.parametrize("gathered", [False, True])
def test_qkv_rope_kvcache(dtype, B, S, nh, nkv, hd, gathered):
    dim, smax, bmax = 256, 256, 4
    cfg = lo.OracleConfig(block_size=512, n_head=nh, n_local_heads=nkv, dim=nh * hd, rope_base=500000)
    g = torch.Generator().manual_seed(B * 100 + S + nh)
    x = _randn(g, B, S, dim, dtype=dtype)
    wqkv = _randn(g, (nh + 2 * nkv) * hd, dim, scale=1 / math.sqrt(dim), dtype=dtype)
    table = lo.rope_table(cfg, dtype)
    pos = torch.arange(S) + 17 if S > 1 else torch.tensor([41], dtype=torch.int32)
    kc = _randn(g, bmax, nkv, smax, hd, dtype=dtype)
    vc = _randn(g, bmax, nkv, smax, hd, dtype=dtype)
    kref, vref = kc.clone(), vc.clone()
    qref = lo.qkv_rope_cache(cfg, 1, lo.linear(x, wqkv), table, pos, kref, vref)  # [B, nh, S, hd]
    ops = _ops()
    kd, vd = kc.cuda(), vc.cuda()
    q = torch.empty(B * S, nh * hd, dtype=dtype, device="cuda")
    nbytes = ops.qkv_workspace_bytes(B * S, nh, nkv, hd)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda") if nbytes else None
    tab = table[pos.long()].contiguous() if gathered else table
    ops.qkv_rope_kvcache(x.view(B * S, dim).cuda(), wqkv.cuda(), tab.cuda(), gathered, pos.cuda(), q, kd, vd, B, S, nh,
                         nkv, hd, ws)
    _ulp_close(q.view(B, S, nh, hd).transpose(1, 2), qref, dtype, ulps=8)
    _ulp_close(kd, kref, dtype, ulps=8)
    _ulp_close(vd, vref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B", [1, 3])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (8, 1, 128), (4, 4, 128), (6, 2, 64), (32, 8, 128)])
@pytest.mark.parametrize("pos,splits", [(0, 1), (5, 4), (63, 3), (200, 7), (255, 64), (130, 1), (100, 8), (17, 2),
                                        (3, 8), (250, 16), (40, 16), (7, 16)])
def test_attn_decode(dtype, B, nh, nkv, hd, pos, splits):
    smax, bmax = 256, 3
    g = torch.Generator().manual_seed(nh * 10 + pos)
    q = _randn(g, B, nh, 1, hd, dtype=dtype)
    kc, vc = _randn(g, bmax, nkv, smax, hd, dtype=dtype), _randn(g, bmax, nkv, smax, hd, dtype=dtype)
    ipos = torch.tensor([pos], dtype=torch.int32)
    ref = lo.attention_core(q, kc, vc, ipos).transpose(1, 2).reshape(B, nh * hd)
    ops = _ops()
    scratch = torch.zeros(ops.attn_decode_scratch_bytes(B, nh, nkv, hd, splits), dtype=torch.uint8, device="cuda")
    out = torch.empty(B, nh * hd, dtype=dtype, device="cuda")
    for _ in range(2):  # the second call checks that the arrival counters were left at zero
        out.fill_(float("nan"))
        ops.attention(q.view(B, nh * hd).cuda(), kc.cuda(), vc.cuda(), ipos.cuda(), out, B, 1, nh, nkv, hd, scratch,
                      splits)
        got = out.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - ref.float()).abs().max().item() < 2e-2 * ref.float().abs().max().item() + 1e-3
        assert gu.rel_err(got, ref) < 6e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,nh,nkv,hd", [(16, 32, 8, 128), (64, 8, 2, 64), (32, 64, 4, 128), (17, 24, 8, 64)])
@pytest.mark.parametrize("pos", [0, 15, 16, 200, 255])
def test_attn_decode_many_sequences(dtype, B, nh, nkv, hd, pos):
    """From 128 (sequence, KV head) pairs on the decode attention runs on tensor cores (the query
    heads of a KV head are the rows of the tiles); the number of ranges is the engine's choice."""
    from gpt_fast.ops import decode_splits
    smax = 256
    g = torch.Generator().manual_seed(B + nh + pos)
    q = _randn(g, B, nh, 1, hd, dtype=dtype)
    kc, vc = _randn(g, B, nkv, smax, hd, dtype=dtype), _randn(g, B, nkv, smax, hd, dtype=dtype)
    ipos = torch.tensor([pos], dtype=torch.int32)
    ref = lo.attention_core(q, kc, vc, ipos).transpose(1, 2).reshape(B, nh * hd)
    ops = _ops()
    splits = decode_splits(B, nh, nkv, smax)
    assert splits in (1, 2)
    scratch = torch.zeros(ops.attn_decode_scratch_bytes(B, nh, nkv, hd, splits), dtype=torch.uint8, device="cuda")
    out = torch.empty(B, nh * hd, dtype=dtype, device="cuda")
    for _ in range(2):  # twice: the arrival counters must be back at zero
        out.fill_(float("nan"))
        ops.attention(q.view(B, nh * hd).cuda(), kc.cuda(), vc.cuda(), ipos.cuda(), out, B, 1, nh, nkv, hd, scratch,
                      splits)
        got = out.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - ref.float()).abs().max().item() < 2e-2 * ref.float().abs().max().item() + 1e-3
        assert gu.rel_err(got, ref) < 6e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,S,pos0", [(1, 12, 0), (2, 64, 0), (1, 65, 0), (2, 130, 7), (1, 300, 0), (1, 2, 100)])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (8, 2, 128)])
def test_attn_prefill(dtype, B, S, pos0, nh, nkv, hd):
    smax, bmax = 320, 2
    g = torch.Generator().manual_seed(S * 10 + nh)
    q = _randn(g, B, nh, S, hd, dtype=dtype)
    kc, vc = _randn(g, bmax, nkv, smax, hd, dtype=dtype), _randn(g, bmax, nkv, smax, hd, dtype=dtype)
    ipos = torch.arange(S) + pos0
    ref = lo.attention_core(q, kc, vc, ipos).transpose(1, 2).reshape(B, S, nh * hd)
    out = torch.full((B, S, nh * hd), float("nan"), dtype=dtype, device="cuda")
    q_rows = q.transpose(1, 2).contiguous().view(B * S, nh * hd)  # [B, S, nh, hd]
    _ops().attention(q_rows.cuda(), kc.cuda(), vc.cuda(), ipos.cuda(), out, B, S, nh, nkv, hd, None, 1)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    # probabilities are rounded to the storage type before the PV product (flash-attention practice)
    assert gu.rel_err(got, ref) < (1.5e-2 if dtype == torch.bfloat16 else 3e-3)


def test_argument_errors_are_reported():
    c = _C()
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 8"):
        c.check(c.lib.lri_add_rmsnorm(0, x.data_ptr(), None, None, 1.0, x.data_ptr(), 1e-5, None, x.data_ptr(), 1, 12,
                                      None))
    with pytest.raises(RuntimeError, match="NULL"):
        c.check(c.lib.lri_linear(0, None, x.data_ptr(), None, x.data_ptr(), 1, 8, 8, None, 0, None))
    with pytest.raises(RuntimeError, match="head_dim"):
        c.check(c.lib.lri_attn_prefill(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, x.data_ptr(), 1,
                                       1, 4, 2, 48, 16, None))
    with pytest.raises(TypeError):
        c.dtype_code(torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 1000, 256), (1, 16032, 4096), (2, 4104, 512), (5, 777 * 8, 1024), (8, 2048, 2048),
                                   (9, 4096, 512), (16, 16032, 1024), (33, 520, 256)])
def test_lm_head_argmax_single_rank(dtype, M, N, K):
    """Projection + arg-max in one launch (M <= 8) or projection, then fold (M > 8), against the
    arg-max of the oracle's rounded logits; two calls in a row on one scratch buffer (each call must
    leave the keys and tickets at zero); an index offset; duplicated rows to force exact ties, which
    must resolve to the lowest index."""
    g = torch.Generator().manual_seed(M * 7 + N)
    x = _randn(g, M, K, dtype=dtype)
    w = _randn(g, N, K, scale=0.05, dtype=dtype)
    ops = _ops()
    scratch = torch.zeros(ops.lm_head_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    logits_ws = torch.empty(M * N, dtype=dtype, device="cuda")
    nbytes = ops.linear_workspace_bytes(M, N)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda") if nbytes else None
    for rep, offset in enumerate((0, 4096)):
        if rep == 1:
            # copy the winning row of every sequence to a later and an earlier position: exact ties
            ref = lo.linear(x, w).float()
            for m in range(M):
                win = ref[m].argmax().item()
                w[(win + 17) % N] = w[win]
                w[(win * 3 + 5) % N] = w[win]
        ref = lo.linear(x, w).float()   # rounded to the storage type, as the projection stores them
        want = ref.argmax(-1)
        # lowest index among exact ties
        want = torch.tensor([int((ref[m] == ref[m].max()).nonzero()[0]) for m in range(M)])
        tok = torch.full((M,), -1, dtype=torch.int32, device="cuda")
        ops.lm_head_argmax(x.cuda(), w.cuda(), offset, tok, M, scratch, None, logits_ws=logits_ws, workspace=ws)
        got = tok.cpu().long() - offset
        for m in range(M):
            if got[m] != want[m]:
                # a different summation order may move a logit by one rounding step: accept another row
                # only if its oracle logit is within one unit in the last place of the maximum
                eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
                assert 0 <= got[m] < N and ref[m, got[m]] >= ref[m].max() - 2 * eps * ref[m].max().abs(), \
                    f"rep {rep} row {m}: token {got[m].item()} (logit {ref[m, got[m]].item()}) vs {want[m].item()} ({ref[m].max().item()})"
    assert int(scratch.view(torch.int32).abs().sum().item()) == 0


def test_lm_head_argmax_empty_slice_and_errors():
    ops = _ops()
    c = _C()
    x = torch.randn(2, 64).to(torch.bfloat16).cuda()
    scratch = torch.zeros(ops.lm_head_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    tok = torch.full((2,), 7, dtype=torch.int32, device="cuda")
    w = torch.empty(0, 64, dtype=torch.bfloat16, device="cuda")
    ops.lm_head_argmax(x, w, 0, tok, 2, scratch)     # a rank without rows still takes part; one rank: key 0
    torch.cuda.synchronize()
    assert int(scratch.view(torch.int32).abs().sum().item()) == 0
    small = torch.zeros(64, dtype=torch.uint8, device="cuda")
    w2 = torch.randn(8, 64).to(torch.bfloat16).cuda()
    rc = c.lib.lri_lm_head_argmax(None, c.BF16, x.data_ptr(), w2.data_ptr(), 2, 8, 64, 0, tok.data_ptr(), small.data_ptr(),
                                  64, None, 0, None, 0, 100, None)
    assert rc == -5
