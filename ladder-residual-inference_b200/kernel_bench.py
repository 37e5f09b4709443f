"""Per-kernel timing of the decode hot path on one GPU, through the C ABI.

    python ladder-residual-inference_b200/kernel_bench.py [--shape 8b|70b|1b|405b] [--tp 1] [--batch 1]
           [--ctx 1152] [--only NAME[,NAME]] [--reps 20] [--json PATH]

For each fused op of a decode step it allocates several independent copies of the operands
(enough that consecutive launches never find their weights in the 126 MB L2), times `reps`
rounds with CUDA events on the launching stream and prints the mean duration, the algorithmic
bytes per launch and the achieved GB/s against the measured HBM copy bandwidth
(MEASURED_PEAKS.json at the repository root when present).  It is also the small, bounded
workload used for `ncu` captures of single kernels.
"""
import argparse
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

SHAPES = {
    "1b": dict(dim=2048, n_layer=16, n_head=32, n_kv=8, hd=64, inter=8192, vocab=128256),
    "8b": dict(dim=4096, n_layer=32, n_head=32, n_kv=8, hd=128, inter=14336, vocab=128256),
    "70b": dict(dim=8192, n_layer=80, n_head=64, n_kv=8, hd=128, inter=28672, vocab=128256),
    "405b": dict(dim=16384, n_layer=126, n_head=128, n_kv=8, hd=128, inter=53248, vocab=128256),
}


def peak_gbs():
    try:
        return float(json.load(open(os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--json", default="")
    ap.add_argument("--eager", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    args = ap.parse_args()

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import gpt_fast  # noqa: F401
    from gpt_fast.ops import CudaOps as ops, decode_splits

    s, t, B = SHAPES[args.shape], args.tp, args.batch
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    dev = torch.device("cuda")
    d, hd = s["dim"], s["hd"]
    nh, nkv, inter = s["n_head"] // t, s["n_kv"] // t, s["inter"] // t
    smax = (args.ctx + 256 + 7) // 8 * 8
    only = set(filter(None, args.only.split(",")))

    def copies(nbytes):
        # enough independent operand sets to cycle through > 2x the L2 capacity, between 2 and 16
        return int(max(2, min(16, math.ceil(2 * 126e6 / max(nbytes, 1)))))

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, device=dev) * scale).to(dt)

    pos = torch.tensor([args.ctx - 1], dtype=torch.int32, device=dev)
    table = rnd(smax + 8, hd // 2, 2, scale=1.0)
    cases = []

    def add(name, nbytes, make, run):
        if only and name not in only:
            return
        cases.append((name, nbytes, make, run))

    # F1: add + norm
    add("add_rmsnorm", 5 * B * d * 2,
        lambda: (rnd(B, d, scale=1), rnd(B, d, scale=1), rnd(d, scale=1), torch.empty(B, d, dtype=dt, device=dev)),
        lambda o: ops.add_rmsnorm(o[0], o[1], None, o[2], 1e-5, o[0], o[3], B))
    # F2: QKV GEMV + RoPE + cache write
    nqkv = (nh + 2 * nkv) * hd
    add("qkv_rope_kvcache", nqkv * d * 2 + B * d * 2 + B * nqkv * 2,
        lambda: (rnd(B, d, scale=1), rnd(nqkv, d), torch.empty(B, nh * hd, dtype=dt, device=dev),
                 torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev), torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev),
                 (torch.empty(ops.qkv_workspace_bytes(B, nh, nkv, hd), dtype=torch.uint8, device=dev)
                  if ops.qkv_workspace_bytes(B, nh, nkv, hd) else None)),
        lambda o: ops.qkv_rope_kvcache(o[0], o[1], table, False, pos, o[2], o[3], o[4], B, 1, nh, nkv, hd, o[5]))
    # F3: decode attention
    splits = decode_splits(B, nh, nkv, smax)
    kv_bytes = 2 * B * nkv * args.ctx * hd * 2
    add("attn_decode", kv_bytes + 2 * B * nh * hd * 2,
        lambda: (rnd(B, nh * hd, scale=1), rnd(B, nkv, smax, hd, scale=1), rnd(B, nkv, smax, hd, scale=1),
                 torch.empty(B, nh * hd, dtype=dt, device=dev),
                 torch.zeros(ops.attn_decode_scratch_bytes(B, nh, nkv, hd, splits), dtype=torch.uint8, device=dev)),
        lambda o: ops.attention(o[0], o[1], o[2], pos, o[3], B, 1, nh, nkv, hd, o[4], splits))
    # F5: wo and w2
    def lin_ws(n):
        nbytes = ops.linear_workspace_bytes(B, n)
        return torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None

    add("wo", d * nh * hd * 2 + B * nh * hd * 2 + B * d * 2,
        lambda: (rnd(B, nh * hd, scale=1), rnd(d, nh * hd), torch.empty(B, d, dtype=dt, device=dev), lin_ws(d)),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))
    add("w2", d * inter * 2 + B * inter * 2 + B * d * 2,
        lambda: (rnd(B, inter, scale=1), rnd(d, inter), torch.empty(B, d, dtype=dt, device=dev), lin_ws(d)),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))
    # F6: gate/up + SwiGLU
    ws_bytes = ops.gateup_workspace_bytes(B, inter)
    add("gateup_swiglu", 2 * inter * d * 2 + B * d * 2 + B * inter * 2,
        lambda: (rnd(B, d, scale=1), rnd(2 * inter, d), torch.empty(B, inter, dtype=dt, device=dev),
                 torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev) if ws_bytes else None),
        lambda o: ops.gateup_swiglu(o[0], o[1], o[2], B, o[3]))
    # F7: LM head
    add("lm_head", s["vocab"] * d * 2 + B * d * 2 + B * s["vocab"] * 2,
        lambda: (rnd(B, d, scale=1), rnd(s["vocab"], d), torch.empty(B, s["vocab"], dtype=dt, device=dev),
                 lin_ws(s["vocab"])),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))

    peak, kind = peak_gbs()
    rows = []
    print(f"shape {args.shape} tp {t} batch {B} ctx {args.ctx} dtype {args.dtype}; peak {peak:.0f} GB/s ({kind})")
    print(f"{'kernel':<20}{'MB/launch':>12}{'us':>10}{'GB/s':>10}{'of peak':>9}")
    for name, nbytes, make, run in cases:
        sets = [make() for _ in range(copies(nbytes))]
        for o in sets:
            run(o)
        torch.cuda.synchronize()
        # one round over all operand sets as a CUDA graph, so that short kernels are timed back to
        # back on the device and not at the pace of the Python launch loop
        graph = None
        if not args.eager:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for o in sets:
                    run(o)
            graph.replay()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            if graph is not None:
                graph.replay()
            else:
                for o in sets:
                    run(o)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.reps * len(sets))
        gbs = nbytes / us / 1e3
        rows.append(dict(kernel=name, bytes=nbytes, us=us, gbs=gbs, frac=gbs / peak, copies=len(sets)))
        print(f"{name:<20}{nbytes / 1e6:>12.2f}{us:>10.2f}{gbs:>10.0f}{gbs / peak:>9.2f}")
        del sets
    if args.json:
        json.dump(dict(args=vars(args), peak=peak, peak_kind=kind, rows=rows), open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
