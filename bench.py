"""Decode-throughput bench of the tensor-parallel Ladder-Llama step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--preset llama-3-8b]
                    [--family ladder] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N ...

A step is ONE decode step: one new token for each of the B sequences through the whole model at
TP = N (one process per GPU), greedy next-token choice included, with the context already in
the KV cache (prompt of --prompt random ids prefilled before the timed region).  The step is
captured in a CUDA graph whose position and token tensors live on the device, so K replays are
K consecutive decode steps at growing context.  Timed on the device with CUDA events between
barriers, maximum over ranks; rank 0 prints one JSON line.

  value     B*K / time, inputs resident in HBM.
  e2e       the same loop driven from HOST buffers: every step copies the token ids and the
            position from pinned host memory, replays the step, copies the chosen tokens back
            and waits for them (what a serving loop does).
  roofline  the dominant kernel (the gate/up GEMV+SwiGLU, ~58 % of the bytes of a step): its
            algorithmic bytes per launch / its CUDA-event duration, against the measured HBM copy
            bandwidth; plus the same figure for the whole step.
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path) timed on the host cores
            on a bounded sample of the same step.
--impl reference times that CPU path alone and prints its own line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "ladder-residual-inference_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--family", default="ladder", choices=["ladder", "dense", "parallel", "desync"])
    ap.add_argument("--preset", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"],
                    help="prefill: time the prompt pass alone (tensor-core bound; an extra measurement, not the default metric)")
    ap.add_argument("--head", default="replicated", choices=["replicated", "vocab-parallel"],
                    help="vocab-parallel: greedy choice through model.decode_greedy (output rows split over the ranks); "
                         "replicated (default) is the reference's scheme")
    ap.add_argument("--steps-per-replay", type=int, default=1,
                    help="decode steps captured into one CUDA graph (token feedback and position stay on the device); "
                         "--steps must be a multiple")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="run the step eagerly (for kernel profiling)")
    ap.add_argument("--cpu-layers", type=int, default=2, help="layers in the CPU sample")
    return ap.parse_args()


def measured_tensor_peak():
    """Sustained dense bf16 TFLOP/s of this pool's B200s (the prompt pass is a long tensor-core job)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1400.0, "fallback"


def prefill_flops(a, t, batch, seq):
    """Algorithmic FLOPs of one prompt pass per rank: projections, causal attention, LM head on every position."""
    d, L, V = a["dim"], a["n_layer"], a["vocab_size"]
    nh, nkv, hd, inter = a["n_head"], a["n_local_heads"], a["head_dim"], a["intermediate_size"]
    proj = 2 * batch * seq * L * ((nh + 2 * nkv) * hd * d + nh * hd * d + 3 * inter * d) // t
    attn = 4 * batch * seq * seq * (nh // t) * hd * L // 2
    head = 2 * batch * seq * V * d
    return proj + attn + head


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def shape_of(preset, family="ladder"):
    from gpt_fast.presets import family_presets
    a = dict(family_presets(family)[preset])
    a.setdefault("n_local_heads", a["n_head"])
    a.setdefault("vocab_size", 32000)
    if a.get("intermediate_size") is None:
        n = int(2 * (4 * a["dim"]) / 3)
        a["intermediate_size"] = n if n % 256 == 0 else n + 256 - n % 256
    a["head_dim"] = a["dim"] // a["n_head"]
    return a


def step_bytes(a, t, batch, ctx, head_split=False):
    """Algorithmic HBM bytes of one decode step on one rank: every weight shard, norm weight and
    the LM head once (all of it, or this rank's 1/t of the rows with the vocabulary-parallel greedy head),
    the valid part of the KV cache once, the new K/V once."""
    d, hd, nh, nkv, inter, L, V = a["dim"], a["head_dim"], a["n_head"], a["n_local_heads"], a["intermediate_size"], a["n_layer"], a["vocab_size"]
    per_layer = ((nh + 2 * nkv) * hd * d + nh * hd * d + 3 * inter * d) // t + 2 * d
    weights = 2 * (L * per_layer + d + V * d // (t if head_split else 1))
    kv = 2 * 2 * L * (nkv // t) * hd * batch * ctx + 2 * 2 * L * (nkv // t) * hd * batch
    return weights + kv


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, str(gpu_index)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", self.gpu], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for ts, r in self.rows if t0 - 0.05 <= ts <= t1 + 0.15] or [r for _, r in self.rows]
        sm, reasons, mx = [], set(), None
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle's restatement of the reference path, on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_decode_sample(a, family, batch, ctx, layers, steps, warmup):
    """Times `steps` decode steps of a `layers`-layer slice of the model (fp32, the precision of the
    reference's CPU-runnable configuration) plus the final norm and LM head, with the KV cache
    holding `ctx` positions, and scales the layer part to the full depth.  Returns tokens/s."""
    import torch
    from oracle import ladder_oracle as lo
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = lo.OracleConfig(block_size=max(2048, ctx + 64), vocab_size=a["vocab_size"], n_layer=layers, n_head=a["n_head"],
                          n_local_heads=a["n_local_heads"], dim=a["dim"], intermediate_size=a["intermediate_size"],
                          rope_base=a.get("rope_base", 10000), rope_scaling=None)
    full = {}
    g = torch.Generator().manual_seed(0)

    def draw(*shape):
        return torch.empty(*shape, dtype=torch.float32).normal_(0, 0.02, generator=g)

    d, hd, nh, nkv, inter = cfg.dim, cfg.head_dim, cfg.n_head, cfg.n_local_heads, cfg.intermediate_size
    full["tok_embeddings"] = draw(cfg.vocab_size, d)
    full["output"] = draw(cfg.vocab_size, d)
    full["norm"] = draw(d)
    for i in range(layers):
        for name, shp in (("wq", (nh * hd, d)), ("wk", (nkv * hd, d)), ("wv", (nkv * hd, d)), ("wo", (d, nh * hd)),
                          ("w_up", (inter, d)), ("w_gate", (inter, d)), ("w2", (d, inter)), ("attention_norm", (d,)),
                          ("ffn_norm", (d,))):
            full[f"l{i}.{name}"] = draw(*shp)
    model = lo.OracleModel(family, cfg, full, 1, torch.float32, batch, ctx + steps + warmup + 8)
    for st in model.ranks:
        for kc, vc in zip(st.k, st.v):
            kc.normal_(0, 1, generator=g)
            vc.normal_(0, 1, generator=g)
    tok = torch.zeros(batch, 1, dtype=torch.long)
    # time the layer stack and the head separately so the layer part can be scaled to full depth
    def one(pos):
        t0 = time.perf_counter()
        x = model.emb[tok]
        saved_logits = model._logits
        timing = {}

        def timed_logits(xx):
            timing["t_layers"] = time.perf_counter() - t0
            t1 = time.perf_counter()
            out = saved_logits(xx)
            timing["t_head"] = time.perf_counter() - t1
            return out

        model._logits = timed_logits
        try:
            getattr(model, "_" + family)(x, torch.tensor([pos]))
        finally:
            model._logits = saved_logits
        return timing["t_layers"], timing["t_head"]

    tl, th = [], []
    with torch.no_grad():
        for i in range(warmup + steps):
            a_, b_ = one(ctx + i)
            if i >= warmup:
                tl.append(a_)
                th.append(b_)
    per_token = statistics.mean(tl) * (a["n_layer"] / layers) + statistics.mean(th)
    return batch / per_token, cores, per_token


def run_reference_arm(args):
    """The reference's own CPU implementation of the step is its PyTorch path; its source is not
    present where this bench runs, so the oracle port of it is timed (kind = "port")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    a = shape_of(args.preset, args.family)
    ctx = args.prompt
    steps, warmup = max(1, min(args.steps, 8)), max(1, min(args.warmup, 2))
    t0 = time.time()
    tps, cores, per_token = cpu_decode_sample(a, args.family, args.batch, ctx, args.cpu_layers, steps, warmup)
    sample = (f"{args.cpu_layers} of {a['n_layer']} layers + final norm + LM head of one decode step at context {ctx}, "
              f"fp32, batch {args.batch}, {steps} timed steps, layer time scaled to full depth")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_token * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, a, note="CPU port of the reference path, host cores only"),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.time() - t0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, a, note=None):
    cfg = {"workload": f"gpt_{args.family}:{args.preset} decode, batch {args.batch}, prompt {args.prompt} random ids, "
                       f"greedy, TP={args.gpus}",
           "dim": a["dim"], "n_layer": a["n_layer"], "n_head": a["n_head"], "n_kv_head": a["n_local_heads"],
           "intermediate_size": a["intermediate_size"], "vocab_size": a["vocab_size"], "batch": args.batch,
           "context": args.prompt, "parallelism": f"tp{args.gpus}",
           "l2": "inputs larger than L2: a step streams every weight shard once (GBs against 126 MB of L2), no flush"}
    if note:
        cfg["note"] = note
    return cfg


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    import gpt_fast  # initialises the process group from the torchrun environment
    from gpt_fast import _C
    from gpt_fast.comm import make_comm

    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == args.gpus, f"--gpus {args.gpus} but the process group has {world} ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    a = shape_of(args.preset, args.family)
    cls = {"ladder": gpt_fast.GPTLadder, "dense": gpt_fast.GPTDense, "parallel": gpt_fast.GPTParallel,
           "desync": gpt_fast.GPTDesync}[args.family]
    with torch.device("meta"):
        model = cls.from_name(args.preset)
    model = model.to(dtype=dtype).to_empty(device=dev).eval()
    torch.manual_seed(1234)  # same stream on every rank: replicated parameters are identical
    with torch.no_grad():
        for p in model.parameters():
            torch.nn.init.normal_(p, mean=0.0, std=0.02)
    B, T, K, W = args.batch, args.prompt, args.steps, args.warmup
    spr = args.steps_per_replay if not args.no_graph else 1
    assert K % spr == 0, "--steps must be a multiple of --steps-per-replay"
    total_steps = 2 * (W * spr + K) + 16 + 4 * spr
    model.setup_caches(max_batch_size=B, max_seq_length=min(T + total_steps, model.config.block_size))
    comm = make_comm()

    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, a["vocab_size"], (T,), generator=g)
    x = prompt.view(1, -1).repeat(B, 1).to(dev)
    with torch.no_grad():
        logits = model(x, torch.arange(T, device=dev))
        first = logits[:, -1].float().argmax(-1, keepdim=True).to(torch.int32)
    del logits
    torch.cuda.synchronize()

    if args.mode == "prefill":
        return run_prefill(args, a, model, x, comm, rank, world, dev)

    tok = first.clone()
    pos = torch.tensor([T], dtype=torch.int32, device=dev)
    nxt = torch.empty_like(tok)

    def step():
        with torch.no_grad():
            if args.head == "vocab-parallel":
                nxt.copy_(model.decode_greedy(tok, pos))
            else:
                lg = model(tok, pos)
                nxt.copy_(torch.argmax(lg[:, -1], dim=-1, keepdim=True))
            tok.copy_(nxt)
            pos.add_(1)

    # launches of this library per step (counted on an eager step; the graph replays the same list)
    c0 = _C.lib.lri_launch_count()
    step()
    launches_per_step = _C.lib.lri_launch_count() - c0
    torch.cuda.synchronize()

    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(spr):
                step()
    run = graph.replay if graph is not None else step

    def reset():
        tok.copy_(first)
        pos.fill_(T)

    def timed(n_steps, body):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            body()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    # ---- device-resident loop ---------------------------------------------------------------------
    reset()
    for _ in range(W):
        run()
    sampler = ClockSampler(torch.cuda.current_device())
    K_runs = K // spr
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    t_wall0 = time.time()
    ms = timed(K_runs, run)
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    value = B * K / (ms / 1e3)

    # ---- end to end from host buffers ---------------------------------------------------------------
    h_tok = torch.empty(B, 1, dtype=torch.int32).pin_memory()
    h_pos = torch.empty(1, dtype=torch.int32).pin_memory()
    h_next = torch.empty(B, 1, dtype=torch.int32).pin_memory()
    h_tok.copy_(first.cpu())
    state = {"pos": T}

    def e2e_step():
        h_pos[0] = state["pos"]
        tok.copy_(h_tok, non_blocking=True)
        pos.copy_(h_pos, non_blocking=True)
        run()
        h_next.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_tok.copy_(h_next)
        state["pos"] += spr

    for _ in range(W):
        e2e_step()
    state["pos"] = T + W * spr
    ms_e2e = timed(K_runs, e2e_step)
    e2e_value = B * K / (ms_e2e / 1e3)
    comm.status()

    # ---- dominant kernel, timed alone with CUDA events on the launching stream -------------------------
    roof = dominant_kernel_roofline(model, a, world, B, dtype, dev)
    ctx_mid = T + W + K // 2
    sb = step_bytes(a, world, B, ctx_mid, head_split=args.head == "vocab-parallel")
    peak, peak_kind = measured_hbm_peak()
    step_gbs = sb / (ms / K / 1e3) / 1e9
    roof.update({"peak": peak, "peak_kind": f"{peak_kind} HBM copy bandwidth", "frac": roof["achieved"] / peak,
                 "step": {"bytes_per_rank": sb, "achieved": step_gbs, "frac": step_gbs / peak, "unit": "GB/s"}})

    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": workload_config(args, a, note=f"comm={comm.name}; cuda_graph={graph is not None}; head={args.head}; steps_per_replay={spr}"),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (B * 4 + 4) / spr, "d2h_bytes_per_step": B * 4 / spr,
                "ms_per_step": ms_e2e / K},
        "gpu_launches": int(launches_per_step * K),
        "launches_per_step": int(launches_per_step),
        "roofline": roof,
    }
    if world == 1 and not args.no_cpu_baseline:
        tps, cores, per_token = cpu_decode_sample(a, args.family, B, T, args.cpu_layers, 3, 1)
        line["cpu_baseline"] = {
            "value": tps, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{args.cpu_layers} of {a['n_layer']} layers + final norm + LM head of one decode step at context "
                      f"{T}, fp32, batch {B}, 3 timed steps, layer time scaled to full depth"}
    print(json.dumps(line), flush=True)


def run_prefill(args, a, model, x, comm, rank, world, dev):
    """Prompt pass alone: K timed calls of model(prompt, arange(T)) after W warm-up calls."""
    import torch
    import torch.distributed as dist
    from gpt_fast import _C
    B, T, K, W = args.batch, args.prompt, args.steps, args.warmup
    positions = torch.arange(T, device=dev)
    c0 = _C.lib.lri_launch_count()
    with torch.no_grad():
        for _ in range(W):
            model(x, positions)
        launches = (_C.lib.lri_launch_count() - c0) // max(W, 1)
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        t0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            model(x, positions)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.item()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    comm.status()
    _C.check(_C.lib.lri_gemm_status())
    if rank != 0:
        return
    flops = prefill_flops(a, world, B, T)
    peak, kind = measured_tensor_peak()
    achieved = flops / (ms / K / 1e3) / 1e12
    line = {
        "metric": "prefill tokens/s", "value": B * T * K / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"gpt_{args.family}:{args.preset} prompt pass, batch {B}, {T} random ids per sequence, "
                               f"logits for every position, TP={world}", "comm": comm.name,
                   "l2": "operands of every GEMM exceed the 126 MB L2"},
        "clocks": clocks, "gpu_launches": int(launches * K), "launches_per_step": int(launches),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": f"{kind} sustained cuBLAS bf16", "flops_per_rank_per_step": flops, "traffic": None},
    }
    print(json.dumps(line), flush=True)


def dominant_kernel_roofline(model, a, world, B, dtype, dev):
    """The gate/up GEMV + SwiGLU of every layer, each launch bracketed by CUDA events on the current
    stream (layers' weights differ, 100+ MB each, so no launch finds its weights in L2)."""
    import torch
    from gpt_fast.ops import CudaOps
    d, inter = a["dim"], a["intermediate_size"] // world
    x = torch.randn(B, d, device=dev).to(dtype)
    h = torch.empty(B, inter, dtype=dtype, device=dev)
    nbytes = CudaOps.gateup_workspace_bytes(B, inter)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev) if nbytes else None
    weights = [layer.attention.wqkv1.weight[layer.attention.qkv_rows:] if hasattr(layer.attention, "wqkv1")
               else layer.feed_forward.w1.weight for layer in model.layers]
    times = []
    for rep in range(3):
        evs = []
        for w in weights:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            CudaOps.gateup_swiglu(x, w, h, B, ws)
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        if rep > 0:
            times += [e0.elapsed_time(e1) for e0, e1 in evs]
    avg_ms = statistics.mean(times)
    algo = 2 * inter * d * 2 + B * d * 2 + B * inter * 2  # weights once, activations in and out
    return {"bound": "hbm", "kernel": "gemv_kernel<SWIGLU> (gate/up projection + SwiGLU)", "achieved": algo / (avg_ms / 1e3) / 1e9,
            "unit": "GB/s", "bytes_per_launch": algo, "us_per_launch": avg_ms * 1e3, "launches_timed": len(times),
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
            # profiles/gemv_gateup_swiglu_8b_tp1_batch1.txt (only that shape was captured)
            "traffic": 238414848 if (d == 4096 and inter == 14336 and B == 1) else None}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
