"""Decode-throughput bench of the tensor-parallel Ladder-Llama step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--preset llama-3-8b]
                    [--family ladder] [--impl ours|reference] [--mode decode|prefill|kernels]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N ...

A step is ONE decode step: one new token for each of the B sequences through the whole model at
TP = N (one process per GPU), greedy next-token choice included, with the context already in
the KV cache (prompt of --prompt random ids prefilled before the timed region).  The step is
captured in a CUDA graph whose position and token tensors live on the device, so K replays are
K consecutive decode steps at growing context.  Timed on the device with CUDA events between
barriers, maximum over ranks; the K-step region is repeated (--repeats, default 5) from the same
starting context and the median is reported.  Rank 0 prints one JSON line.

  value     B*K / time, inputs resident in HBM (median over the repeats; all repeats listed).
  e2e       the same loop driven from HOST buffers: every step copies the token ids and the
            position from pinned host memory, replays the step, copies the chosen tokens back
            and waits for them (what a serving loop does).
  exposed_ar_us_per_token
            step time minus the time of the same engine, schedule, streams and kernels with the
            collective left out (gpt_fast.comm.ElidedComm), for the ladder and the dense schedule on
            the same weights; `ladder_vs_dense` is the ratio of their throughputs.
  roofline  the dominant kernel (the gate/up GEMV+SwiGLU, ~58 % of the bytes of a step): its
            algorithmic bytes per launch / its duration when the launches of all layers are
            replayed back to back from a CUDA graph, against the measured HBM copy bandwidth; plus
            the same figure for the whole step.
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path) timed on the host cores
            on a bounded sample of the same step; cpu_baseline_config1 is the reference's own
            CPU-runnable configuration (Ladder-Llama 1B, fp32, two ranks) run whole.
--impl reference times that CPU path alone and prints its own line.
--mode kernels times every fused op of a decode step on its own (per-kernel GB/s table; also the
small, bounded workload used for profiler captures of single kernels).
"""
import argparse
import importlib.util
import json
import math
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

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from profiler
# captures summarised under profiles/ (keyed by hidden size, local FFN width, token rows)
DOMINANT_KERNEL_TRAFFIC = {
    (4096, 14336, 1): (238414848, "profiles/gemv_gateup_swiglu_8b_tp1_batch1.txt"),
}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="repeats of the K-step timed region (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--family", default="ladder", choices=["ladder", "dense", "parallel", "desync"])
    ap.add_argument("--preset", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill", "kernels", "comm"],
                    help="prefill: time the prompt pass alone (tensor-core bound; an extra measurement, not the default "
                         "metric); kernels: per-kernel table of one decode step; comm: all-reduce latency by message size")
    ap.add_argument("--head", default="vocab-parallel", choices=["replicated", "vocab-parallel"],
                    help="vocab-parallel (default): greedy choice through model.decode_greedy, the LM-head rows split over "
                         "the ranks and the arg-max fused into the projection (same tokens); replicated: the reference's "
                         "scheme, full logits on every rank followed by an arg-max")
    ap.add_argument("--steps-per-replay", type=int, default=1,
                    help="decode steps captured into one CUDA graph (token feedback and position stay on the device); "
                         "--steps must be a multiple")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-compare", action="store_true",
                    help="skip the second schedule (dense next to ladder) and the comm-elided runs")
    ap.add_argument("--no-graph", action="store_true", help="run the step eagerly (for kernel profiling)")
    ap.add_argument("--last-logits-only", action="store_true",
                    help="prefill mode: LM head on the last position only (the reference computes every position)")
    ap.add_argument("--trace", action="store_true",
                    help="prefill mode: after the timed region run one more pass eagerly with per-operation CUDA-event "
                         "timing (gpt_fast.trace) and print the table on rank 0")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU sample")
    # --mode kernels
    ap.add_argument("--shape", default="8b", choices=["1b", "8b", "70b", "405b"])
    ap.add_argument("--tp", type=int, default=1, help="kernels mode: shard sizes of one rank of this TP degree")
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--eager", action="store_true", help="kernels mode: launch from Python instead of replaying a graph")
    return ap.parse_args(argv)


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def measured_tensor_peak():
    """Sustained dense bf16 TFLOP/s of this pool's B200s (the prompt pass is a long tensor-core job)."""
    v = _peaks().get("bf16_tflops_sustained")
    return (float(v), "measured") if v else (1400.0, "fallback")


def measured_hbm_peak():
    v = _peaks().get("hbm_gbs")
    return (float(v), "measured") if v else (FALLBACK_HBM_GBS, "fallback")


def prefill_flops(a, t, batch, seq, head_positions=None):
    """Algorithmic FLOPs of one prompt pass per rank: projections, causal attention, LM head on every
    position (or on `head_positions` positions per sequence)."""
    d, L, V = a["dim"], a["n_layer"], a["vocab_size"]
    nh, nkv, hd, inter = a["n_head"], a["n_local_heads"], a["head_dim"], a["intermediate_size"]
    proj = 2 * batch * seq * L * ((nh + 2 * nkv) * hd * d + nh * hd * d + 3 * inter * d) // t
    attn = 4 * batch * seq * seq * (nh // t) * hd * L // 2
    head = 2 * batch * (seq if head_positions is None else head_positions) * V * d
    return proj + attn + head


_PRESETS = None


def _presets_module():
    """The preset table is plain Python: loaded from its file, so that the CPU arm neither imports the
    package (which loads the CUDA library and creates a process group) nor needs a GPU."""
    global _PRESETS
    if _PRESETS is None:
        spec = importlib.util.spec_from_file_location("lri_presets", os.path.join(PKG, "gpt_fast", "presets.py"))
        _PRESETS = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_PRESETS)
    return _PRESETS


def shape_of(preset, family="ladder"):
    a = dict(_presets_module().family_presets(family)[preset])
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
# CPU baselines: the oracle's restatement of the reference path, on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_decode_sample(a, family, batch, ctx, layers, steps, warmup, t=1):
    """Times `steps` decode steps of a `layers`-layer slice of the model (fp32, the precision of the
    reference's CPU-runnable configuration) plus the final norm and LM head, with the KV cache
    holding `ctx` positions, `t` simulated ranks, and scales the layer part to the full depth.
    Returns (tokens/s, cores, seconds per token)."""
    import torch
    from oracle import ladder_oracle as lo
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layers = min(layers, a["n_layer"])
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
    model = lo.OracleModel(family, cfg, full, t, torch.float32, batch, ctx + steps + warmup + 8)
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


def cpu_config1_baseline(new_tokens=32, prompt_len=32):
    """The reference's own CPU-runnable configuration, whole: Ladder-Llama 1B (hidden 2048, 16 layers,
    32 query / 8 KV heads, FFN 8192, vocabulary 128256), fp32, two tensor-parallel ranks (simulated one
    after the other in this process, each using all host cores), batch 1, prompt of 32 random ids,
    32 greedy tokens; decode tokens/s = (new - 1) / decode time, as benchmark.py:140-159 measures it."""
    import torch
    from oracle import ladder_oracle as lo
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    a = shape_of("ladder-llama-1b", "ladder")
    cfg = lo.OracleConfig(block_size=2048, vocab_size=a["vocab_size"], n_layer=a["n_layer"], n_head=a["n_head"],
                          n_local_heads=a["n_local_heads"], dim=a["dim"], intermediate_size=a["intermediate_size"],
                          rope_base=a["rope_base"])
    full = lo.make_full_weights(cfg, 1234, std=0.02)
    model = lo.OracleModel("ladder", cfg, full, 2, torch.float32, 1, prompt_len + new_tokens)
    del full
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g)
    with torch.no_grad():
        t0 = time.perf_counter()
        logits = model.forward(prompt.view(1, -1), torch.arange(prompt_len))
        t_prefill = time.perf_counter() - t0
        tok = logits[:, -1].argmax(-1, keepdim=True)
        t0 = time.perf_counter()
        for n in range(new_tokens - 1):
            logits = model.forward(tok, torch.tensor([prompt_len + n]))
            tok = logits[:, -1].argmax(-1, keepdim=True)
        t_decode = time.perf_counter() - t0
    return {"value": (new_tokens - 1) / t_decode, "unit": UNIT, "cores": cores, "kind": "port",
            "prefill_s": t_prefill, "decode_s": t_decode,
            "sample": f"Ladder-Llama 1B whole (16 layers), fp32, TP=2 simulated rank by rank in one process, batch 1, "
                      f"prompt {prompt_len} random ids, {new_tokens} greedy tokens; decode tokens/s over the last "
                      f"{new_tokens - 1}"}


def cpu_sample_text(a, layers, ctx, batch, steps, warmup, t):
    return (f"{min(layers, a['n_layer'])} of {a['n_layer']} layers + final norm + LM head of one decode step at context "
            f"{ctx}, fp32, batch {batch}, {t} simulated rank(s), {steps} timed steps after {warmup} warm-up, layer time "
            f"scaled to full depth")


def run_reference_arm(args):
    """The reference's own CPU implementation of the step is its PyTorch path; its source is not
    present where this bench runs, so the oracle port of it is timed (kind = "port").  Nothing of the
    CUDA package is imported here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    a = shape_of(args.preset, args.family)
    ctx, t = args.prompt, max(1, args.gpus)
    steps, warmup = max(1, min(args.steps, 32)), max(1, min(args.warmup, 4))  # bounded: what is printed is what ran
    t0 = time.time()
    tps, cores, per_token = cpu_decode_sample(a, args.family, args.batch, ctx, args.cpu_layers, steps, warmup, t=t)
    sample = cpu_sample_text(a, args.cpu_layers, ctx, args.batch, steps, warmup, t)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": per_token * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, a, note=f"CPU port of the reference path, host cores only, {t} simulated rank(s)"),
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

FAMILY_CLASS = {"ladder": "GPTLadder", "dense": "GPTDense", "parallel": "GPTParallel", "desync": "GPTDesync"}


class DecodeLoop:
    """One model's decode step (greedy choice included) with device-resident token and position,
    captured into a CUDA graph of `spr` consecutive steps."""

    def __init__(self, model, B, T, first, head, spr, use_graph):
        import torch
        self.torch, self.model, self.B, self.T, self.head, self.spr = torch, model, B, T, head, spr
        dev = first.device
        self.first = first
        self.tok = first.clone()
        self.pos = torch.tensor([T], dtype=torch.int32, device=dev)
        self.nxt = torch.empty_like(self.tok)
        self.graph = None
        self.use_graph = use_graph

    def step(self):
        torch = self.torch
        with torch.no_grad():
            if self.head == "vocab-parallel":
                self.nxt.copy_(self.model.decode_greedy(self.tok, self.pos))
            else:
                lg = self.model(self.tok, self.pos)
                self.nxt.copy_(torch.argmax(lg[:, -1], dim=-1, keepdim=True))
            self.tok.copy_(self.nxt)
            self.pos.add_(1)

    def capture(self):
        torch = self.torch
        if not self.use_graph:
            return
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            for _ in range(self.spr):
                self.step()

    def run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()

    def reset(self):
        self.tok.copy_(self.first)
        self.pos.fill_(self.T)


def build_model(gpt_fast, family, preset, dtype, dev, share_with=None):
    import torch
    cls = getattr(gpt_fast, FAMILY_CLASS[family])
    with torch.device("meta"):
        model = cls.from_name(preset)
    if share_with is not None:
        # same parameter names and shapes (ladder, dense and desync share a module tree): the second
        # schedule runs on the very same weight tensors, no copy
        model = model.to(dtype=dtype)
        model.load_state_dict(dict(share_with.named_parameters()), assign=True)
        return model.eval()
    model = model.to(dtype=dtype).to_empty(device=dev).eval()
    torch.manual_seed(1234)  # same stream on every rank: replicated parameters are identical
    with torch.no_grad():
        for p in model.parameters():
            torch.nn.init.normal_(p, mean=0.0, std=0.02)
    return model


def run_ours(args):
    import torch
    import torch.distributed as dist
    import gpt_fast  # initialises the process group from the torchrun environment
    from gpt_fast import _C
    from gpt_fast.comm import ElidedComm, make_comm

    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == args.gpus, f"--gpus {args.gpus} but the process group has {world} ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    a = shape_of(args.preset, args.family)
    model = build_model(gpt_fast, args.family, args.preset, dtype, dev)
    B, T, K, W, R = args.batch, args.prompt, args.steps, args.warmup, max(1, args.repeats)
    spr = args.steps_per_replay if not args.no_graph else 1
    assert K % spr == 0, "--steps must be a multiple of --steps-per-replay"
    total_steps = W * spr + K + 16 + 4 * spr  # every timed repeat starts again from position T
    max_seq = min(T + total_steps, model.config.block_size)
    model.setup_caches(max_batch_size=B, max_seq_length=max_seq)
    comm = make_comm()

    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, a["vocab_size"], (T,), generator=g)
    x = prompt.view(1, -1).repeat(B, 1).to(dev)

    def prefill(m):
        with torch.no_grad():
            logits = m(x, torch.arange(T, device=dev))
            return logits[:, -1].float().argmax(-1, keepdim=True).to(torch.int32)

    first = prefill(model)
    torch.cuda.synchronize()

    if args.mode == "prefill":
        return run_prefill(args, a, model, x, comm, rank, world, dev)

    # ---- outside the timed region: every rank must have chosen the same tokens ---------------------
    loop = DecodeLoop(model, B, T, first, args.head, spr, not args.no_graph)
    c0 = _C.lib.lri_launch_count()
    loop.step()
    launches_per_step = _C.lib.lri_launch_count() - c0  # counted on an eager step; the graph replays the same list
    agree_steps = 4
    seen = [first.clone(), loop.tok.clone()]
    for _ in range(agree_steps - 1):
        loop.step()
        seen.append(loop.tok.clone())
    mine = torch.cat(seen, dim=1).contiguous()
    if world > 1:
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        if args.family != "desync":  # desync ranks hold different residuals between all-reduces by design
            for r, other in enumerate(every):
                assert torch.equal(other, every[0]), f"rank {r} chose tokens {other.tolist()} but rank 0 {every[0].tolist()}"
    torch.cuda.synchronize()
    agreement = (f"{world} ranks chose identical tokens on the prompt pass and {agree_steps} decode steps "
                 f"(checked before the timed region)") if world > 1 and args.family != "desync" else "single rank or desync: not applicable"

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

    K_runs = K // spr

    def measure(lp, repeats):
        """Median (and all) of `repeats` K-step regions, each from position T after W warm-up replays."""
        out = []
        for _ in range(repeats):
            lp.reset()
            for _ in range(W):
                lp.run()
            out.append(timed(K_runs, lp.run))
        return statistics.median(out), out

    # ---- device-resident loop ---------------------------------------------------------------------
    loop.capture()
    loop.reset()
    for _ in range(W):
        loop.run()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    t_wall0 = time.time()
    ms, ms_all = measure(loop, R)
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    value = B * K / (ms / 1e3)

    # ---- end to end from host buffers ---------------------------------------------------------------
    h_tok = torch.empty(B, 1, dtype=torch.int32).pin_memory()
    h_pos = torch.empty(1, dtype=torch.int32).pin_memory()
    h_next = torch.empty(B, 1, dtype=torch.int32).pin_memory()
    state = {"pos": T}

    def e2e_step():
        h_pos[0] = state["pos"]
        loop.tok.copy_(h_tok, non_blocking=True)
        loop.pos.copy_(h_pos, non_blocking=True)
        loop.run()
        h_next.copy_(loop.nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_tok.copy_(h_next)
        state["pos"] += spr

    e2e_all = []
    for _ in range(min(R, 3)):
        h_tok.copy_(first.cpu())
        state["pos"] = T
        for _ in range(W):
            e2e_step()
        e2e_all.append(timed(K_runs, e2e_step))
    ms_e2e = statistics.median(e2e_all)
    e2e_value = B * K / (ms_e2e / 1e3)
    comm.status()

    # ---- exposed all-reduce time and the dense schedule next to the ladder one -----------------------
    extra = {}
    if not args.no_compare and args.family in ("ladder", "dense"):
        other_family = "dense" if args.family == "ladder" else "ladder"
        per = {args.family: {"ms_per_step": ms / K, "value": value}}

        def elided_ms(m, first_tok):
            """The same engine with the collective left out (same kernels, order and streams)."""
            eng = m._engine
            real = eng.comm
            eng.comm = ElidedComm(world, rank, like=real)
            try:
                lp = DecodeLoop(m, B, T, first_tok, args.head, spr, not args.no_graph)
                lp.capture()
                v, _ = measure(lp, min(R, 3))
            finally:
                eng.comm = real
            return v / K

        other = build_model(gpt_fast, other_family, args.preset, dtype, dev, share_with=model)
        other.setup_caches(max_batch_size=B, max_seq_length=max_seq)
        first_o = prefill(other)
        lp_o = DecodeLoop(other, B, T, first_o, args.head, spr, not args.no_graph)
        lp_o.capture()
        ms_o, _ = measure(lp_o, min(R, 3))
        per[other_family] = {"ms_per_step": ms_o / K, "value": B * K / (ms_o / 1e3)}
        comm.status()
        exposed = {}
        if world > 1:
            for fam, m, f in ((args.family, model, first), (other_family, other, first_o)):
                el = elided_ms(m, f)
                per[fam]["comm_elided_ms_per_step"] = el
                exposed[fam] = (per[fam]["ms_per_step"] - el) * 1e3
        else:
            exposed = {args.family: 0.0, other_family: 0.0}
        extra = {
            "exposed_ar_us_per_token": dict(exposed, how="ms_per_step minus ms_per_step of the same engine, schedule, "
                                            "streams and kernels with the collective left out (ElidedComm); 0 at one rank"),
            "ladder_vs_dense": per["ladder"]["value"] / per["dense"]["value"],
            "schedules": per,
        }
        del other, lp_o

    # ---- dominant kernel, replayed back to back from a CUDA graph --------------------------------------
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
        "config": workload_config(args, a, note=f"comm={comm.name}; cuda_graph={loop.graph is not None}; head={args.head}; "
                                                f"steps_per_replay={spr}; value = median of {R} repeats of the {K}-step region"),
        "clocks": clocks,
        "repeats_ms_per_step": [m / K for m in ms_all],
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (B * 4 + 4) / spr, "d2h_bytes_per_step": B * 4 / spr,
                "ms_per_step": ms_e2e / K, "repeats_ms_per_step": [m / K for m in e2e_all]},
        "gpu_launches": int(launches_per_step * K),
        "launches_per_step": int(launches_per_step),
        "rank_agreement": agreement,
        "roofline": roof,
    }
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        steps_cpu, warm_cpu = 5, 1
        tps, cores, per_token = cpu_decode_sample(a, args.family, B, T, args.cpu_layers, steps_cpu, warm_cpu)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": cpu_sample_text(a, args.cpu_layers, T, B, steps_cpu, warm_cpu, 1)}
        line["cpu_baseline_config1"] = cpu_config1_baseline()
    print(json.dumps(line), flush=True)


def run_prefill(args, a, model, x, comm, rank, world, dev):
    """Prompt pass alone: K timed calls of model(prompt, arange(T)) after W warm-up calls."""
    import torch
    import torch.distributed as dist
    from gpt_fast import _C
    B, T, K, W = args.batch, args.prompt, args.steps, args.warmup
    positions = torch.arange(T, device=dev)
    last_only = args.last_logits_only

    def one():
        if last_only:
            return model.prefill_last(x, positions)
        return model(x, positions)

    c0 = _C.lib.lri_launch_count()
    with torch.no_grad():
        for _ in range(W):
            one()
        launches = (_C.lib.lri_launch_count() - c0) // max(W, 1)
        sampler = ClockSampler(torch.cuda.current_device())
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        # the barrier comes AFTER rank 0's wait for the clock sampler: a rank that enters the timed region
        # early would count the time it waits for the others inside its first collective
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            one()
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
    if args.trace:
        from gpt_fast.trace import trace_engine
        tr = trace_engine(model._engine)
        with torch.no_grad():
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            h0 = time.perf_counter()
            one()
            host_ms = (time.perf_counter() - h0) * 1e3
            e1.record()
        table = tr.report()
        tr.stop()
        if rank == 0:
            print(f"one traced pass: {e0.elapsed_time(e1):.2f} ms on the device, {host_ms:.2f} ms for the host to enqueue it",
                  file=sys.stderr)
            print(f"  {'operation':<28}{'calls':>6}{'device ms':>12}{'host ms':>10}", file=sys.stderr)
            for name, (n, t, h) in sorted(table.items(), key=lambda kv: -kv[1][1]):
                print(f"  {name:<28}{n:>6}{t:>12.2f}{h:>10.2f}", file=sys.stderr)
    if rank != 0:
        return
    flops = prefill_flops(a, world, B, T, head_positions=1 if last_only else None)
    peak, kind = measured_tensor_peak()
    achieved = flops / (ms / K / 1e3) / 1e12
    line = {
        "metric": "prefill tokens/s", "value": B * T * K / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"gpt_{args.family}:{args.preset} prompt pass, batch {B}, {T} random ids per sequence, "
                               f"logits for {'the last position' if last_only else 'every position'}, TP={world}",
                   "comm": comm.name, "l2": "operands of every GEMM exceed the 126 MB L2"},
        "clocks": clocks, "gpu_launches": int(launches * K), "launches_per_step": int(launches),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": f"{kind} sustained cuBLAS bf16", "flops_per_rank_per_step": flops, "traffic": None},
    }
    print(json.dumps(line), flush=True)


def dominant_kernel_roofline(model, a, world, B, dtype, dev):
    """The gate/up GEMV + SwiGLU of every layer, one launch per layer captured into a CUDA graph and
    replayed back to back, timed with CUDA events around the replays on the launching stream.  The
    layers' weights differ (tens of MB to hundreds each, GBs together), so no launch finds its weights
    in L2, and the graph keeps the launches at the device's pace whatever the host does."""
    import torch
    from gpt_fast.ops import CudaOps
    d, inter = a["dim"], a["intermediate_size"] // world
    x = torch.randn(B, d, device=dev).to(dtype)
    h = torch.empty(B, inter, dtype=dtype, device=dev)
    nbytes = CudaOps.gateup_workspace_bytes(B, inter)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev) if nbytes else None
    weights = [layer.attention.wqkv1.weight[layer.attention.qkv_rows:] if hasattr(layer.attention, "wqkv1")
               else layer.feed_forward.w1.weight for layer in model.layers]
    # small shards: cycle through the layers more than once per replay so that a replay is long enough to time
    rounds = max(1, math.ceil(64 / len(weights)))

    def launches():
        for _ in range(rounds):
            for w in weights:
                CudaOps.gateup_swiglu(x, w, h, B, ws)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launches()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launches()
    graph.replay()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    n = reps * rounds * len(weights)
    avg_ms = e0.elapsed_time(e1) / n
    algo = 2 * inter * d * 2 + B * d * 2 + B * inter * 2  # weights once, activations in and out
    traffic = DOMINANT_KERNEL_TRAFFIC.get((d, inter, B))
    kernel = "gemv_kernel<SWIGLU>" if B == 1 else ("gemv_mma_kernel<SWIGLU>" if B <= 8 else "gemm_streamk_kernel<SWIGLU>")
    return {"bound": "hbm", "kernel": f"{kernel} (gate/up projection + SwiGLU)", "achieved": algo / (avg_ms / 1e3) / 1e9,
            "unit": "GB/s", "bytes_per_launch": algo, "us_per_launch": avg_ms * 1e3, "launches_timed": n,
            "timing": "CUDA events around graph replays of one launch per layer, back to back",
            "traffic": traffic[0] if traffic else None,
            "traffic_source": traffic[1] if traffic else "no profiler capture of this shape: null"}


# ---------------------------------------------------------------------------------------------
# --mode kernels: every fused op of a decode step on its own
# ---------------------------------------------------------------------------------------------

KERNEL_SHAPES = {
    "1b": dict(dim=2048, n_layer=16, n_head=32, n_kv=8, hd=64, inter=8192, vocab=128256),
    "8b": dict(dim=4096, n_layer=32, n_head=32, n_kv=8, hd=128, inter=14336, vocab=128256),
    "70b": dict(dim=8192, n_layer=80, n_head=64, n_kv=8, hd=128, inter=28672, vocab=128256),
    "405b": dict(dim=16384, n_layer=126, n_head=128, n_kv=8, hd=128, inter=53248, vocab=128256),
}


def run_kernels(args):
    """For each fused op of a decode step: several independent copies of the operands (enough that
    consecutive launches never find their weights in the 126 MB L2), one round over them captured into a
    CUDA graph, `reps` replays timed with CUDA events; prints mean duration, algorithmic bytes per launch
    and achieved GB/s against the measured HBM copy bandwidth."""
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import torch
    import gpt_fast  # noqa: F401
    from gpt_fast.ops import CudaOps as ops, decode_splits

    s, t, B = KERNEL_SHAPES[args.shape], args.tp, args.batch
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

    add("add_rmsnorm", 5 * B * d * 2,
        lambda: (rnd(B, d, scale=1), rnd(B, d, scale=1), rnd(d, scale=1), torch.empty(B, d, dtype=dt, device=dev)),
        lambda o: ops.add_rmsnorm(o[0], o[1], None, o[2], 1e-5, o[0], o[3], B))
    nqkv = (nh + 2 * nkv) * hd
    add("qkv_rope_kvcache", nqkv * d * 2 + B * d * 2 + B * nqkv * 2,
        lambda: (rnd(B, d, scale=1), rnd(nqkv, d), torch.empty(B, nh * hd, dtype=dt, device=dev),
                 torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev), torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev),
                 (torch.empty(ops.qkv_workspace_bytes(B, nh, nkv, hd), dtype=torch.uint8, device=dev)
                  if ops.qkv_workspace_bytes(B, nh, nkv, hd) else None)),
        lambda o: ops.qkv_rope_kvcache(o[0], o[1], table, False, pos, o[2], o[3], o[4], B, 1, nh, nkv, hd, o[5]))
    if hasattr(ops, "norm_qkv_rope_kvcache"):
        add("norm_qkv_rope_kvcache", nqkv * d * 2 + 5 * B * d * 2 + B * nqkv * 2,
            lambda: (rnd(B, d, scale=1), rnd(B, d, scale=1), rnd(d, scale=1), rnd(nqkv, d),
                     torch.empty(B, nh * hd, dtype=dt, device=dev), torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev),
                     torch.zeros(B, nkv, smax, hd, dtype=dt, device=dev)),
            lambda o: ops.norm_qkv_rope_kvcache(o[0], o[1], None, o[2], 1e-5, o[0], o[3], table, pos, o[4], o[5], o[6],
                                                B, nh, nkv, hd))
    splits = decode_splits(B, nh, nkv, smax, hd)
    kv_bytes = 2 * B * nkv * args.ctx * hd * 2
    add("attn_decode", kv_bytes + 2 * B * nh * hd * 2,
        lambda: (rnd(B, nh * hd, scale=1), rnd(B, nkv, smax, hd, scale=1), rnd(B, nkv, smax, hd, scale=1),
                 torch.empty(B, nh * hd, dtype=dt, device=dev),
                 torch.zeros(ops.attn_decode_scratch_bytes(B, nh, nkv, hd, splits), dtype=torch.uint8, device=dev)),
        lambda o: ops.attention(o[0], o[1], o[2], pos, o[3], B, 1, nh, nkv, hd, o[4], splits))

    def lin_ws(n):
        nbytes = ops.linear_workspace_bytes(B, n)
        return torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None

    add("wo", d * nh * hd * 2 + B * nh * hd * 2 + B * d * 2,
        lambda: (rnd(B, nh * hd, scale=1), rnd(d, nh * hd), torch.empty(B, d, dtype=dt, device=dev), lin_ws(d)),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))
    add("w2", d * inter * 2 + B * inter * 2 + B * d * 2,
        lambda: (rnd(B, inter, scale=1), rnd(d, inter), torch.empty(B, d, dtype=dt, device=dev), lin_ws(d)),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))
    ws_bytes = ops.gateup_workspace_bytes(B, inter)
    add("gateup_swiglu", 2 * inter * d * 2 + B * d * 2 + B * inter * 2,
        lambda: (rnd(B, d, scale=1), rnd(2 * inter, d), torch.empty(B, inter, dtype=dt, device=dev),
                 torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev) if ws_bytes else None),
        lambda o: ops.gateup_swiglu(o[0], o[1], o[2], B, o[3]))
    if hasattr(ops, "norm_gateup_swiglu"):
        add("norm_gateup_swiglu", 2 * inter * d * 2 + 5 * B * d * 2 + B * inter * 2,
            lambda: (rnd(B, d, scale=1), rnd(B, d, scale=1), rnd(d, scale=1), rnd(2 * inter, d),
                     torch.empty(B, inter, dtype=dt, device=dev)),
            lambda o: ops.norm_gateup_swiglu(o[0], o[1], None, o[2], 1e-5, o[0], o[3], o[4], B))
    add("lm_head", s["vocab"] * d * 2 + B * d * 2 + B * s["vocab"] * 2,
        lambda: (rnd(B, d, scale=1), rnd(s["vocab"], d), torch.empty(B, s["vocab"], dtype=dt, device=dev),
                 lin_ws(s["vocab"])),
        lambda o: ops.linear(o[0], o[1], o[2], B, workspace=o[3]))
    if hasattr(ops, "lm_head_argmax"):
        vloc = -(-s["vocab"] // (8 * t)) * 8
        add("lm_head_argmax", vloc * d * 2 + B * d * 2,
            lambda: (rnd(B, d, scale=1), rnd(vloc, d), torch.empty(B, dtype=torch.int32, device=dev),
                     torch.zeros(ops.lm_head_argmax_scratch_bytes(B, vloc), dtype=torch.uint8, device=dev)),
            lambda o: ops.lm_head_argmax(o[0], o[1], 0, o[2], B, o[3]))

    # prompt-pass kernels (tensor-core bound; listed only when named in --only): --ctx is the prompt length
    S = args.ctx
    rows_p = B * S
    tpeak, _ = measured_tensor_peak()
    flops = {}

    def add_prefill(name, fl, make, run):
        if name in only:
            flops[name] = fl
            cases.append((name, 0, make, run))

    add_prefill("prefill_attn", 4 * B * S * S * nh * hd // 2,
                lambda: (rnd(rows_p, nh * hd, scale=1), rnd(B, nkv, S + 8, hd, scale=1), rnd(B, nkv, S + 8, hd, scale=1),
                         torch.empty(B, S, nh * hd, dtype=dt, device=dev), torch.arange(S, device=dev)),
                lambda o: ops.attention(o[0], o[1], o[2], o[4], o[3], B, S, nh, nkv, hd, None, 1))
    add_prefill("prefill_gateup", 2 * rows_p * 2 * inter * d,
                lambda: (rnd(rows_p, d, scale=1), rnd(2 * inter, d), torch.empty(rows_p, inter, dtype=dt, device=dev)),
                lambda o: ops.gateup_swiglu(o[0], o[1], o[2], rows_p, None))
    add_prefill("prefill_w2", 2 * rows_p * inter * d,
                lambda: (rnd(rows_p, inter, scale=1), rnd(d, inter), torch.empty(rows_p, d, dtype=dt, device=dev)),
                lambda o: ops.linear(o[0], o[1], o[2], rows_p))
    add_prefill("prefill_add_rmsnorm", 0,
                lambda: (rnd(rows_p, d, scale=1), rnd(rows_p, d, scale=1), rnd(d, scale=1),
                         torch.empty(rows_p, d, dtype=dt, device=dev)),
                lambda o: ops.add_rmsnorm(o[0], o[1], None, o[2], 1e-5, o[0], o[3], rows_p))

    peak, kind = measured_hbm_peak()
    rows = []
    print(f"shape {args.shape} tp {t} batch {B} ctx {args.ctx} dtype {args.dtype}; peak {peak:.0f} GB/s ({kind})")
    print(f"{'kernel':<24}{'MB/launch':>12}{'us':>10}{'GB/s':>10}{'of peak':>9}")
    for name, nbytes, make, run in cases:
        if name == "prefill_add_rmsnorm":
            nbytes = 5 * rows_p * d * 2
        sets = [make() for _ in range(copies(nbytes) if not name.startswith("prefill_") else 2)]
        for o in sets:
            run(o)
        torch.cuda.synchronize()
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
        if name in flops and flops[name]:
            tf = flops[name] / us / 1e6
            rows.append(dict(kernel=name, flops=flops[name], us=us, tflops=tf, frac=tf / tpeak, copies=len(sets)))
            print(f"{name:<24}{flops[name] / 1e9:>10.1f} GF{us:>10.2f}{tf:>8.0f} TF{tf / tpeak:>9.2f}  (of {tpeak:.0f} TFLOP/s sustained)")
            del sets
            continue
        gbs = nbytes / us / 1e3
        rows.append(dict(kernel=name, bytes=nbytes, us=us, gbs=gbs, frac=gbs / peak, copies=len(sets)))
        print(f"{name:<24}{nbytes / 1e6:>12.2f}{us:>10.2f}{gbs:>10.0f}{gbs / peak:>9.2f}")
        del sets
    if args.json:
        json.dump(dict(args=vars(args), peak=peak, peak_kind=kind, rows=rows), open(args.json, "w"), indent=1)


def run_comm(args):
    """All-reduce latency over message sizes for the three back ends (low-latency / one-shot peer kernel,
    NCCL), each timed as a chain of back-to-back in-stream calls replayed from a CUDA graph; rank 0 prints
    a table and one JSON line.  The table is what the size threshold between the peer kernel and NCCL
    (LRI_P2P_MAX_BYTES) is chosen from."""
    import torch
    import torch.distributed as dist
    import gpt_fast  # noqa: F401
    from gpt_fast.comm import P2PComm, TorchComm
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world > 1, "--mode comm needs at least 2 ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    sizes = [8 << 10, 16 << 10, 32 << 10, 64 << 10, 128 << 10, 256 << 10, 512 << 10, 1 << 20, 2 << 20, 4 << 20, 8 << 20]
    p2p = P2PComm(max_bytes=max(sizes))
    nccl = TorchComm()
    chain = 20

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(chain):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() * 1e3 / (args.reps * chain)

    out = []
    for nbytes in sizes:
        x = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device=dev)
        row = {"bytes": nbytes}
        for name, fn in (("p2p", lambda: p2p.all_reduce(x)), ("nccl", lambda: nccl.all_reduce(x))):
            row[name + "_us"] = timed(fn)
        out.append(row)

    # all-reduce + residual add + RMSNorm of a decode step: the all-reduce kernel followed by the norm
    # kernel, against the one kernel that does both (lri_add_rmsnorm_allreduce)
    from gpt_fast.ops import CudaOps as ops
    fused = []
    for rows, dim in ((1, 4096), (1, 8192), (8, 4096), (16, 4096), (8, 8192)):
        part = torch.zeros(rows, dim, dtype=torch.bfloat16, device=dev)
        resid = torch.zeros(rows, dim, dtype=torch.bfloat16, device=dev)
        normed = torch.empty_like(resid)
        w = torch.ones(dim, dtype=torch.bfloat16, device=dev)

        def two():
            p2p.all_reduce(part)
            ops.add_rmsnorm(resid, part, None, w, 1e-5, resid, normed, rows, 1.0)

        def one():
            p2p.add_rmsnorm_gather(resid, 1, part, 0, None, w, 1e-5, resid, normed, rows, 1.0, self_push=True)

        fused.append({"rows": rows, "dim": dim, "allreduce_then_norm_us": timed(two), "fused_us": timed(one),
                      "norm_only_us": timed(lambda: ops.add_rmsnorm(resid, part, None, w, 1e-5, resid, normed, rows, 1.0))})
    p2p.status()
    if rank == 0:
        print(f"all-reduce latency, {world} ranks, bf16, in-stream chain of {chain} calls per graph replay, max over ranks")
        print(f"{'bytes':>10}{'peer kernel us':>16}{'NCCL us':>10}{'kernel':>12}")
        for r in out:
            kind = "LL lines" if r["bytes"] <= 128 * 1024 else "one-shot"
            print(f"{r['bytes']:>10}{r['p2p_us']:>16.2f}{r['nccl_us']:>10.2f}{kind:>12}")
        print(f"all-reduce + add + RMSNorm, {world} ranks, bf16, same chain")
        print(f"{'rows':>6}{'dim':>7}{'kernel + norm us':>18}{'one kernel us':>15}{'norm alone us':>15}")
        for r in fused:
            print(f"{r['rows']:>6}{r['dim']:>7}{r['allreduce_then_norm_us']:>18.2f}{r['fused_us']:>15.2f}{r['norm_only_us']:>15.2f}")
        print(json.dumps({"mode": "comm", "n_gpus": world, "rows": out, "fused_norm": fused}), flush=True)
    p2p.close()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.mode == "comm":
        run_comm(args)
    elif args.mode == "kernels":
        run_kernels(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
