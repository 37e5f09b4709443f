"""CPU oracle for the tensor-parallel decode/prefill step (TEST INFRASTRUCTURE ONLY).

This file restates, in plain PyTorch on the CPU, the arithmetic of the reference's
`gpt_fast` hot path so the CUDA kernels can be checked against it.  It is a checker:
only `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference`
legs of `bench.py` may import it.  The product package never does.

Parity status: the reference ships no tests and no golden vectors, so this oracle is
pinned against outputs of the reference itself (its Python modules imported on the
CPU with a gloo process group); `tests/golden/make_golden.py` generates those
fixtures and `tests/test_oracle_golden.py` checks this file against them.

Each function cites the reference code it follows (paths relative to the reference
repository root).  Tensor parallelism is simulated inside one process: the `t`
ranks' partial results are computed one after another from per-rank weight shards
and summed, which is what the reference's all-reduce does
(gpt_fast/utils.py:390-397).

Rounding points (all kept, because two bf16 implementations that round at different
places can sit ~1.5e-2 apart): every `nn.Linear` output, every residual add, the
RMSNorm result before the weight multiply, the RoPE result, the SiLU result and the
attention output are rounded to the model dtype.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

FAMILIES = ("ladder", "dense", "parallel", "desync")


@dataclass
class OracleConfig:
    """Field names follow ModelArgs (gpt_fast/gpt_ladder_TP.py:32-57,
    gpt_fast/gpt_desync_TP.py:30-61)."""

    block_size: int = 2048
    vocab_size: int = 32000
    n_layer: int = 32
    n_head: int = 32
    dim: int = 4096
    intermediate_size: Optional[int] = None
    n_local_heads: int = -1
    rope_base: float = 10000
    norm_eps: float = 1e-5
    rope_scaling: Optional[dict] = None
    reduce_pattern: Optional[List[dict]] = None
    force_disable_last_all_reduce: bool = False
    # ladder family only: indices of the layers that use the ladder dataflow, the others are dense
    # (hf_modeling_utils/configuration_llama_ladder.py:38-45; an int n means the last n layers).
    # None: every layer is a ladder layer, which is what gpt_fast/gpt_ladder_TP.py runs.
    ladder_layers: Optional[object] = None
    head_dim: int = field(init=False, default=0)

    def __post_init__(self):
        if self.n_local_heads == -1:
            self.n_local_heads = self.n_head
        if self.intermediate_size is None:
            n_hidden = int(2 * (4 * self.dim) / 3)
            self.intermediate_size = n_hidden if n_hidden % 256 == 0 else n_hidden + 256 - n_hidden % 256
        self.head_dim = self.dim // self.n_head
        if self.reduce_pattern is None:
            self.reduce_pattern = [{"attention": False, "mlp": True} for _ in range(self.n_layer)]
        if isinstance(self.ladder_layers, int):
            self.ladder_layers = list(range(self.n_layer - self.ladder_layers, self.n_layer))


# ----------------------------------------------------------------------------------------
# weights: full (unsharded) tensors from a seed, and the per-rank local layouts
# ----------------------------------------------------------------------------------------


def make_full_weights(cfg: OracleConfig, seed: int, std: float = 0.02, norm_mean: float = 0.0,
                      norm_std: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """Full fp32 tensors, one generator per tensor (seed + running index) so a tensor's draw
    does not depend on the others.  The reference draws every parameter, the norm weights
    included, from N(0, 0.02) (benchmark.py:242-243); `norm_mean`/`norm_std` let a test
    use a "loud" init under which the four schedules are far apart."""
    if norm_std is None:
        norm_std = std
    counter = [0]

    def draw(*shape, s=std, mean=0.0):
        g = torch.Generator().manual_seed(seed + counter[0])
        counter[0] += 1
        return torch.randn(*shape, generator=g, dtype=torch.float32) * s + mean

    d, hd, nh, nkv, inter = cfg.dim, cfg.head_dim, cfg.n_head, cfg.n_local_heads, cfg.intermediate_size
    w = {"tok_embeddings": draw(cfg.vocab_size, d), "output": draw(cfg.vocab_size, d),
         "norm": draw(d, s=norm_std, mean=norm_mean)}
    for i in range(cfg.n_layer):
        w[f"l{i}.wq"] = draw(nh * hd, d)
        w[f"l{i}.wk"] = draw(nkv * hd, d)
        w[f"l{i}.wv"] = draw(nkv * hd, d)
        w[f"l{i}.wo"] = draw(d, nh * hd)
        w[f"l{i}.w_up"] = draw(inter, d)
        w[f"l{i}.w_gate"] = draw(inter, d)
        w[f"l{i}.w2"] = draw(d, inter)
        w[f"l{i}.attention_norm"] = draw(d, s=norm_std, mean=norm_mean)
        w[f"l{i}.ffn_norm"] = draw(d, s=norm_std, mean=norm_mean)
    return w


def shard_layer(cfg: OracleConfig, full: Dict[str, torch.Tensor], layer: int, rank: int, t: int,
                dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """Local parameter layout of one rank.  The reference builds every nn.Linear already
    divided by the world size (gpt_fast/utils.py:142-143, 165-166, 277-281) and splits the
    fused outputs as [q | k | v] (utils.py:190-191), [up | gate] (utils.py:146-147) and
    [q | k | v | up | gate] (utils.py:311-313); rank r therefore owns q heads
    r*nh/t.., kv heads r*nkv/t.. and MLP columns r*I/t.. ."""
    hd, nh, nkv, inter = cfg.head_dim, cfg.n_head, cfg.n_local_heads, cfg.intermediate_size
    qs = slice(rank * nh // t * hd, (rank + 1) * nh // t * hd)
    ks = slice(rank * nkv // t * hd, (rank + 1) * nkv // t * hd)
    ms = slice(rank * inter // t, (rank + 1) * inter // t)
    p = f"l{layer}."
    wq, wk, wv = full[p + "wq"][qs], full[p + "wk"][ks], full[p + "wv"][ks]
    up, gate = full[p + "w_up"][ms], full[p + "w_gate"][ms]
    out = {
        "wqkv": torch.cat([wq, wk, wv]),
        "wo": full[p + "wo"][:, qs],
        "w1": torch.cat([up, gate]),
        "w2": full[p + "w2"][:, ms],
        "wqkv1": torch.cat([wq, wk, wv, up, gate]),
        "attention_norm": full[p + "attention_norm"],
        "ffn_norm": full[p + "ffn_norm"],
    }
    return {k: v.to(dtype).contiguous() for k, v in out.items()}


# ----------------------------------------------------------------------------------------
# sublayer arithmetic
# ----------------------------------------------------------------------------------------


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """nn.Linear(bias=False): fp32 accumulation, one rounding to the model dtype."""
    return (x.float() @ w.float().t()).to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """gpt_fast/utils.py:68-74: mean square and rsqrt in fp32, cast to the input dtype,
    then the weight multiply in the input dtype (the Liger kernel the eager branch calls,
    utils.py:76, uses the same "llama" casting)."""
    xf = x.float()
    inv = torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv).to(x.dtype) * weight


def rope_table(cfg: OracleConfig, dtype: torch.dtype) -> torch.Tensor:
    """[block_size, head_dim/2, 2] (cos, sin), rounded to the model dtype
    (gpt_fast/utils.py:103-117); optional llama-3 frequency scaling (utils.py:81-100)."""
    n = cfg.head_dim
    inv_freq = 1.0 / (cfg.rope_base ** (torch.arange(0, n, 2)[: n // 2].float() / n))
    sc = cfg.rope_scaling
    if sc is not None:
        lo_wave = sc["original_max_position_embeddings"] / sc["low_freq_factor"]
        hi_wave = sc["original_max_position_embeddings"] / sc["high_freq_factor"]
        scaled = []
        for f in inv_freq:
            wave = 2 * math.pi / f
            if wave < hi_wave:
                scaled.append(f)
            elif wave > lo_wave:
                scaled.append(f / sc["factor"])
            else:
                s = (sc["original_max_position_embeddings"] / wave - sc["low_freq_factor"]) / (
                    sc["high_freq_factor"] - sc["low_freq_factor"])
                scaled.append((1 - s) * f / sc["factor"] + s * f)
        inv_freq = torch.tensor(scaled, dtype=inv_freq.dtype)
    ang = torch.outer(torch.arange(cfg.block_size), inv_freq)
    # torch.polar(1, ang) in the reference: real = cos, imag = sin, evaluated in fp32
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(dtype)


def rope(x: torch.Tensor, table_rows: torch.Tensor) -> torch.Tensor:
    """Rotate ADJACENT pairs (x[2i], x[2i+1]) in fp32 (gpt_fast/utils.py:120-132).
    x: [B, S, H, hd]; table_rows: [S, hd/2, 2] in the model dtype."""
    xf = x.float()
    even, odd = xf[..., 0::2], xf[..., 1::2]
    c = table_rows[None, :, None, :, 0].float()
    s = table_rows[None, :, None, :, 1].float()
    out = torch.empty_like(xf)
    out[..., 0::2] = even * c - odd * s
    out[..., 1::2] = odd * c + even * s
    return out.to(x.dtype)


def attention_core(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   input_pos: torch.Tensor) -> torch.Tensor:
    """softmax(q k^T / sqrt(hd) + causal) v over cache positions <= the query's position
    (gpt_fast/utils.py:252-255 with mask = causal_mask[None, None, input_pos],
    gpt_ladder_TP.py:254).  q: [B, nh, S, hd]; caches: [B, nkv, Smax, hd]; q head h reads
    kv head h // (nh/nkv) (repeat_interleave).  fp32 inside, one rounding at the end."""
    B, nh, S, hd = q.shape
    nkv = k_cache.shape[1]
    g = nh // nkv
    smax = k_cache.shape[2]
    kf = k_cache[:B].float().repeat_interleave(g, dim=1)
    vf = v_cache[:B].float().repeat_interleave(g, dim=1)
    scores = q.float() @ kf.transpose(-1, -2) / math.sqrt(hd)  # [B, nh, S, Smax]
    allowed = torch.arange(smax)[None, :] <= input_pos.long()[:, None]  # [S, Smax]
    scores = scores.masked_fill(~allowed[None, None], float("-inf"))
    return (torch.softmax(scores, dim=-1) @ vf).to(q.dtype)


class RankState:
    """One simulated rank: its weight shards and its KV caches
    ([B, nkv/t, Smax, hd] per layer, gpt_fast/utils.py:43-48)."""

    def __init__(self, cfg: OracleConfig, full, rank: int, t: int, dtype, max_batch: int, max_seq: int):
        self.layers = [shard_layer(cfg, full, i, rank, t, dtype) for i in range(cfg.n_layer)]
        smax = max_seq if max_seq % 8 == 0 else max_seq + 8 - max_seq % 8  # gpt_ladder_TP.py:229
        shape = (max_batch, cfg.n_local_heads // t, smax, cfg.head_dim)
        self.k = [torch.zeros(shape, dtype=dtype) for _ in range(cfg.n_layer)]
        self.v = [torch.zeros(shape, dtype=dtype) for _ in range(cfg.n_layer)]


def qkv_rope_cache(cfg, t, qkv, table, input_pos, k_cache, v_cache):
    """Split the fused projection, rotate q and k, write k/v at input_pos
    (gpt_fast/utils.py:187-198, 50-59, 247-250).  Returns q as [B, nh/t, S, hd]."""
    B, S, _ = qkv.shape
    nh_l, nkv_l, hd = cfg.n_head // t, cfg.n_local_heads // t, cfg.head_dim
    q, k, v = qkv.split([nh_l * hd, nkv_l * hd, nkv_l * hd], dim=-1)
    rows = table[input_pos.long()]
    q = rope(q.reshape(B, S, nh_l, hd), rows).transpose(1, 2)
    k = rope(k.reshape(B, S, nkv_l, hd), rows).transpose(1, 2)
    v = v.reshape(B, S, nkv_l, hd).transpose(1, 2)
    k_cache[:B, :, input_pos.long()] = k
    v_cache[:B, :, input_pos.long()] = v
    return q


def attention_partial(cfg, t, w, x, table, input_pos, k_cache, v_cache):
    """One rank's attention sublayer before the all-reduce (gpt_fast/utils.py:187-260)."""
    B, S, _ = x.shape
    q = qkv_rope_cache(cfg, t, linear(x, w["wqkv"]), table, input_pos, k_cache, v_cache)
    y = attention_core(q, k_cache, v_cache, input_pos)
    y = y.transpose(1, 2).reshape(B, S, -1)
    return linear(y, w["wo"])


def swiglu(ug: torch.Tensor) -> torch.Tensor:
    """First half of the columns is `up`, second half `gate`; silu(gate) * up with the SiLU
    result rounded before the multiply (gpt_fast/utils.py:146-148)."""
    u, g = ug.chunk(2, dim=-1)
    return torch.nn.functional.silu(g.float()).to(ug.dtype) * u


def mlp_partial(w, x):
    """One rank's MLP sublayer before the all-reduce (gpt_fast/utils.py:145-149)."""
    return linear(swiglu(linear(x, w["w1"])), w["w2"])


def fused_partial(cfg, t, w, x, table, input_pos, k_cache, v_cache):
    """Parallel block: one input projection [q|k|v|up|gate], wo and w2 partials summed
    before the single all-reduce (gpt_fast/utils.py:305-387)."""
    B, S, _ = x.shape
    nh_l, nkv_l, hd = cfg.n_head // t, cfg.n_local_heads // t, cfg.head_dim
    nqkv = (nh_l + 2 * nkv_l) * hd
    z = linear(x, w["wqkv1"])
    q = qkv_rope_cache(cfg, t, z[..., :nqkv], table, input_pos, k_cache, v_cache)
    y = attention_core(q, k_cache, v_cache, input_pos).transpose(1, 2).reshape(B, S, -1)
    y = linear(y, w["wo"])
    return linear(swiglu(z[..., nqkv:]), w["w2"]) + y


def all_reduce(partials: List[torch.Tensor]) -> torch.Tensor:
    """SUM over ranks (gpt_fast/utils.py:395).  Summed in fp32 and rounded once; NCCL's own
    order of bf16 partial sums is not specified, so any order inside the tolerance is right."""
    acc = partials[0].float()
    for p in partials[1:]:
        acc = acc + p.float()
    return acc.to(partials[0].dtype)


# ----------------------------------------------------------------------------------------
# the four schedules
# ----------------------------------------------------------------------------------------


class OracleModel:
    """All `t` simulated ranks of one model.  `forward(idx, input_pos)` returns the logits of
    rank 0 (ladder, dense and parallel are rank-invariant; for desync the ranks differ
    between all-reduces and rank 0 is what the reference prints)."""

    def __init__(self, family: str, cfg: OracleConfig, full: Dict[str, torch.Tensor], t: int,
                 dtype: torch.dtype, max_batch: int, max_seq: int):
        assert family in FAMILIES
        self.family, self.cfg, self.t, self.dtype = family, cfg, t, dtype
        self.ranks = [RankState(cfg, full, r, t, dtype, max_batch, max_seq) for r in range(t)]
        self.emb = full["tok_embeddings"].to(dtype)
        self.out = full["output"].to(dtype)
        self.final_norm = full["norm"].to(dtype)
        self.table = rope_table(cfg, dtype)

    def forward(self, idx: torch.Tensor, input_pos: torch.Tensor) -> torch.Tensor:
        return getattr(self, "_" + self.family)(self.emb[idx.long()], input_pos)

    def _logits(self, x):
        return linear(rmsnorm(x, self.final_norm, self.cfg.norm_eps), self.out)

    def _attn(self, r, i, x, pos):
        st = self.ranks[r]
        w = st.layers[i]
        return attention_partial(self.cfg, self.t, w, rmsnorm(x, w["attention_norm"], self.cfg.norm_eps),
                                 self.table, pos, st.k[i], st.v[i])

    def _mlp(self, r, i, x):
        w = self.ranks[r].layers[i]
        return mlp_partial(w, rmsnorm(x, w["ffn_norm"], self.cfg.norm_eps))

    def _ladder(self, x, pos):
        """gpt_fast/gpt_ladder_TP.py:252-284, 312-358: the all-reduced output of a sublayer is
        added to the residual one sublayer later."""
        if self.cfg.ladder_layers is not None:
            return self._hybrid(x, pos)
        prev_a = torch.zeros_like(x)
        prev_m = torch.zeros_like(x)
        for i in range(self.cfg.n_layer):
            x = x + prev_a
            cur_a = all_reduce([self._attn(r, i, x, pos) for r in range(self.t)])
            x = x + prev_m
            cur_m = all_reduce([self._mlp(r, i, x) for r in range(self.t)])
            prev_a, prev_m = cur_a, cur_m
        return self._logits(x + prev_a + prev_m)

    def _hybrid(self, x, pos):
        """Checkpoints whose config lists `ladder_layers`: the listed layers use the ladder dataflow,
        the others the dense one (hf_modeling_utils/modeling_llama_ladder.py:627-663 for a layer,
        889-948 for the loop).  Stated on the residual stream r with two pending addends, so that
        `hidden_states` of the reference is r + prev_a + prev_m and its `prev_attn_output` is r + prev_a:
          ladder layer   r += prev_a; A = Attn(norm(r)); r += prev_m; M = Mlp(norm(r)); pending (A, M)
          dense layer    r += prev_a + prev_m; r += Attn(norm(r)); M = Mlp(norm(r)); pending (0, M)
        With every layer listed this is _ladder, with none _dense."""
        ladder = set(self.cfg.ladder_layers)
        prev_a = torch.zeros_like(x)
        prev_m = torch.zeros_like(x)
        for i in range(self.cfg.n_layer):
            if i in ladder:
                x = x + prev_a
                cur_a = all_reduce([self._attn(r, i, x, pos) for r in range(self.t)])
                x = x + prev_m
                cur_m = all_reduce([self._mlp(r, i, x) for r in range(self.t)])
                prev_a, prev_m = cur_a, cur_m
            else:
                x = (x + prev_a) + prev_m
                x = x + all_reduce([self._attn(r, i, x, pos) for r in range(self.t)])
                prev_a = torch.zeros_like(x)
                prev_m = all_reduce([self._mlp(r, i, x) for r in range(self.t)])
        return self._logits(x + prev_a + prev_m)

    def _dense(self, x, pos):
        """gpt_fast/gpt_dense_TP.py:281-282."""
        for i in range(self.cfg.n_layer):
            x = x + all_reduce([self._attn(r, i, x, pos) for r in range(self.t)])
            x = x + all_reduce([self._mlp(r, i, x) for r in range(self.t)])
        return self._logits(x)

    def _parallel(self, x, pos):
        """gpt_fast/gpt_parallel_TP.py:220-224: one norm, one fused sublayer, one all-reduce."""
        for i in range(self.cfg.n_layer):
            parts = []
            for r in range(self.t):
                st = self.ranks[r]
                w = st.layers[i]
                h = rmsnorm(x, w["attention_norm"], self.cfg.norm_eps)
                parts.append(fused_partial(self.cfg, self.t, w, h, self.table, pos, st.k[i], st.v[i]))
            x = all_reduce(parts) + x
        return self._logits(x)

    def _desync(self, x, pos):
        """gpt_fast/gpt_desync_TP.py:319-323, 366-382: where a sublayer's flag is on,
        x = AR(f(norm(x)) + x/t); where it is off, x = f(norm(x)) + x on each rank alone."""
        cfg, t = self.cfg, self.t
        xs = [x.clone() for _ in range(t)]
        for i in range(cfg.n_layer):
            do_attn = cfg.reduce_pattern[i]["attention"]
            do_mlp = (i == cfg.n_layer - 1) or cfg.reduce_pattern[i]["mlp"]
            if i == cfg.n_layer - 1 and cfg.force_disable_last_all_reduce:
                do_mlp = False
            ys = [self._attn(r, i, xs[r], pos) for r in range(t)]
            if do_attn:
                red = all_reduce([ys[r] + xs[r] / t for r in range(t)])
                xs = [red.clone() for _ in range(t)]
            else:
                xs = [ys[r] + xs[r] for r in range(t)]
            ys = [self._mlp(r, i, xs[r]) for r in range(t)]
            if do_mlp:
                red = all_reduce([ys[r] + xs[r] / t for r in range(t)])
                xs = [red.clone() for _ in range(t)]
            else:
                xs = [ys[r] + xs[r] for r in range(t)]
        return self._logits(xs[0])


def greedy_generate(model: OracleModel, prompt: torch.Tensor, batch: int, new_tokens: int):
    """benchmark.py:118-164 with top_k=1: the same prompt for every row, prefill over
    arange(T), then one shared position for all rows.  Returns (tokens [B, new], list of
    last-position logits per step)."""
    T = prompt.numel()
    x = prompt.view(1, -1).repeat(batch, 1)
    logits = model.forward(x, torch.arange(T))
    steps = [logits[:, -1]]
    tok = logits[:, -1].float().argmax(dim=-1, keepdim=True)
    toks = [tok]
    for n in range(new_tokens - 1):
        logits = model.forward(tok, torch.tensor([T + n]))
        steps.append(logits[:, -1])
        tok = logits[:, -1].float().argmax(dim=-1, keepdim=True)
        toks.append(tok)
    return torch.cat(toks, dim=-1), steps


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k=None, generator=None):
    """benchmark.py:56-77 on last-position logits [B, V]: divide by max(temperature, 1e-5); with top_k,
    everything below the k-th largest value of a row becomes -inf; softmax; then one draw per row as
    argmax(probs / q) with q ~ Exponential(1) of the shape and type of probs.  Returns (int32 [B, 1], probs)."""
    x = logits / max(temperature, 1e-5)
    if top_k is not None:
        kth = torch.topk(x, min(top_k, x.size(-1))).values[..., -1:]
        x = torch.where(x < kth, torch.full_like(x, float("-inf")), x)
    probs = torch.nn.functional.softmax(x, dim=-1)
    q = torch.empty_like(probs).exponential_(1, generator=generator)
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(torch.int32), probs

