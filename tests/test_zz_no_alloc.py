"""The allocation-free decode-attention entry point, lri_attn_decode_static.

It serves callers that cannot give the kernel scratch memory because they may not allocate on
the hot path (a plug-in handed only tensors and a stream, a server with a fixed memory plan):
the scratch is an array inside the library.  The test calls it through the C ABI twice in a row
(the second call finds the first call's partials in the shared array and must not be disturbed
by them) and compares with lri_attn_decode on caller-owned scratch and with the CPU oracle.  Collected last on purpose,
so that a run which stops at the first failure has already run every other test."""
import pytest
import torch

from oracle import ladder_oracle as lo

pytestmark = pytest.mark.gpu


def _decode(c, static, q, kc, vc, pos, out, B, nh, nkv, hd, splits, scratch=None):
    smax = kc.shape[2]
    stream = torch.cuda.current_stream().cuda_stream
    if static:
        rc = c.lib.lri_attn_decode_static(c.BF16, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), 0,
                                          out.data_ptr(), B, nh, nkv, hd, smax, splits, stream)
    else:
        rc = c.lib.lri_attn_decode(c.BF16, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), 0,
                                   out.data_ptr(), B, nh, nkv, hd, smax, splits, scratch.data_ptr(), scratch.numel(),
                                   stream)
    c.check(rc)


def test_static_scratch_entry_point_matches_and_is_reusable():
    from gpt_fast import _C as c
    B, nh, nkv, hd, smax = 2, 8, 2, 128, 512
    g = torch.Generator().manual_seed(17)
    kc = torch.randn(B, nkv, smax, hd, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(B, nkv, smax, hd, generator=g).to(torch.bfloat16).cuda()
    # two calls in a row with different queries, positions and split counts
    for pos_value, splits in ((300, 7), (41, 3)):
        q = torch.randn(B, nh * hd, generator=g).to(torch.bfloat16).cuda()
        pos = torch.tensor([pos_value], dtype=torch.int32, device="cuda")
        need = c.lib.lri_attn_decode_scratch_bytes(B, nh, nkv, hd, splits)
        assert need <= c.lib.lri_attn_decode_static_scratch_capacity()
        scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")
        want = torch.empty(B, nh * hd, dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(want, float("nan"))
        _decode(c, False, q, kc, vc, pos, want, B, nh, nkv, hd, splits, scratch)
        _decode(c, True, q, kc, vc, pos, got, B, nh, nkv, hd, splits)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same kernel, same inputs: the tolerance of the decode-attention parity test is ample
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2e-2 * want.float().abs().max().item() + 1e-3, diff
        _check_against_oracle(got, q, kc, vc, pos_value, B, nh, hd)


def _check_against_oracle(got, q, kc, vc, pos_value, B, nh, hd):
    ref = lo.attention_core(q.cpu().view(B, nh, 1, hd), kc.cpu(), vc.cpu(), torch.tensor([pos_value]))
    ref = ref.transpose(1, 2).reshape(B, nh * hd).float()
    diff = (got.float().cpu() - ref).abs().max().item()
    assert diff <= 2e-2 * ref.abs().max().item() + 1e-3, diff


def test_static_scratch_serves_the_tensor_core_kernel_too():
    """From 128 (sequence, KV head) pairs on, the ranges are merged through the scratch by the
    tensor-core kernel.  It shares the built-in array with the SIMT kernel: a call of one kind right
    after a call of the other must find the arrival counters at zero."""
    from gpt_fast import _C as c
    B, nh, nkv, hd, smax = 16, 32, 8, 128, 256
    g = torch.Generator().manual_seed(23)
    kc = torch.randn(B, nkv, smax, hd, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(B, nkv, smax, hd, generator=g).to(torch.bfloat16).cuda()
    small = dict(B=2, nh=8, nkv=2)  # a SIMT-path call on the same array in between
    for pos_value, splits in ((200, 2), (77, 3)):
        q = torch.randn(B, nh * hd, generator=g).to(torch.bfloat16).cuda()
        pos = torch.tensor([pos_value], dtype=torch.int32, device="cuda")
        need = c.lib.lri_attn_decode_scratch_bytes(B, nh, nkv, hd, splits)
        assert need <= c.lib.lri_attn_decode_static_scratch_capacity()
        scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")
        want = torch.empty(B, nh * hd, dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(want, float("nan"))
        _decode(c, False, q, kc, vc, pos, want, B, nh, nkv, hd, splits, scratch)
        _decode(c, True, q, kc, vc, pos, got, B, nh, nkv, hd, splits)
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert torch.isfinite(got.float()).all() and diff <= 2e-2 * want.float().abs().max().item() + 1e-3, diff
        _check_against_oracle(got, q, kc, vc, pos_value, B, nh, hd)
        # SIMT scratch kernel (7 ranges) on a slice of the same caches, through the same array
        sq = q[: small["B"], : small["nh"] * hd].contiguous()
        sgot = torch.full((small["B"], small["nh"] * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        skc, svc = kc[: small["B"], : small["nkv"]].contiguous(), vc[: small["B"], : small["nkv"]].contiguous()
        _decode(c, True, sq, skc, svc, pos, sgot, small["B"], small["nh"], small["nkv"], hd, 7)
        torch.cuda.synchronize()
        _check_against_oracle(sgot, sq, skc, svc, pos_value, small["B"], small["nh"], hd)


def test_static_scratch_entry_point_refuses_oversized_requests():
    from gpt_fast import _C as c
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    p = x.data_ptr()
    # 64 sequences x 128 heads x 64 splits x head_dim 128 needs far more than the built-in array
    rc = c.lib.lri_attn_decode_static(c.BF16, p, p, p, p, 0, p, 64, 128, 8, 128, 4096, 64, None)
    assert rc == -5
    assert b"built-in" in c.lib.lri_last_error()
