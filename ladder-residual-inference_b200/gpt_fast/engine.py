"""Whole-model forward of the four tensor-parallel schedules on preallocated buffers.

One `Engine` per model.  `setup()` sizes every intermediate buffer for the largest
(batch x sequence) the caches allow, so that `forward()` allocates nothing but the returned
logits, never synchronises with the host, reads positions from the caller's device tensor, and
can be captured into a CUDA graph together with its communication stream.

All four schedules are sequences of the same step

    residual, normed = F1(residual + pending adds, norm weight)      fused add + RMSNorm
    partial          = sublayer(normed)                              F2+F3/F4+F5  or  F6+F5
    handle           = all_reduce_async(partial)

and differ only in WHEN a partial's all-reduce is waited for and added:

  ladder    one sublayer later: attention of layer i is added before attention of layer i+1,
            MLP of layer i before MLP of layer i+1, so each all-reduce overlaps the next sublayer
            (reference gpt_fast/gpt_ladder_TP.py:252-284, 312-358)
  dense     immediately (gpt_fast/gpt_dense_TP.py:274-284)
  parallel  one fused attention+MLP sublayer and one all-reduce per layer
            (gpt_fast/gpt_parallel_TP.py:214-226)
  desync    residual/t is folded into the partial before the all-reduce where a layer's flag is
            set; no communication where it is not (gpt_fast/gpt_desync_TP.py:350-384)
"""
import os

import torch

from .comm import make_comm
from .ops import decode_splits

_MAX_SPLITS = 64


class Engine:
    def __init__(self, model, family, ops=None, comm=None):
        self.model = model
        self.family = family
        self.cfg = model.config
        if ops is None:
            from .ops import CudaOps
            ops = CudaOps
        self.ops = ops
        self.comm = comm if comm is not None else make_comm()
        self.ready = False
        self._norm_pushes = False  # set per step by _reduce_plan

    # ------------------------------------------------------------------------------------------
    def setup(self, max_batch, max_seq, device, dtype):
        cfg, t = self.cfg, self.comm.world
        self.nh, self.nkv, self.hd = cfg.n_head // t, cfg.n_local_heads // t, cfg.head_dim
        self.inter = cfg.intermediate_size // t
        self.d = cfg.dim
        self.max_batch, self.max_seq = max_batch, max_seq
        rows = max_batch * max_seq
        self.max_rows = rows

        def buf(cols):
            return torch.empty(rows, cols, dtype=dtype, device=device)

        self.resid, self.normed = buf(self.d), buf(self.d)
        self.part_a, self.part_m = buf(self.d), buf(self.d)
        self.q, self.y = buf(self.nh * self.hd), buf(self.nh * self.hd)
        self.h = buf(self.inter)

        def workspace(size_fn, *shape):
            # large enough for a prefill of all rows and for a decode step of up to 64 rows (whose
            # split-K partial sums can take more room than a longer prefill's raw projection)
            n = max(size_fn(rows, *shape), size_fn(min(rows, 64), *shape))
            return torch.empty(n, dtype=torch.uint8, device=device) if n else None

        self.ws_qkv = workspace(self.ops.qkv_workspace_bytes, self.nh, self.nkv, self.hd)
        self.ws_ug = workspace(self.ops.gateup_workspace_bytes, self.inter)
        # wo and w2 may run at the same time on two streams: one workspace each (w2's also serves the LM head)
        self.ws_wo = workspace(self.ops.linear_workspace_bytes, self.d)
        self.ws_w2 = workspace(self.ops.linear_workspace_bytes, self.d)
        self.ws_head = workspace(self.ops.linear_workspace_bytes, cfg.vocab_size)
        # vocabulary-parallel greedy head (decode_greedy): this rank's slice of the output rows
        self.vocab_per_rank = -(-cfg.vocab_size // (8 * t)) * 8
        self.vocab_lo = min(cfg.vocab_size, self.comm.rank * self.vocab_per_rank)
        self.vocab_hi = min(cfg.vocab_size, self.vocab_lo + self.vocab_per_rank)
        self.head_logits = torch.empty(max_batch * self.vocab_per_rank, dtype=dtype, device=device)
        self.head_best = torch.empty(t, max_batch, 2, dtype=torch.float32, device=device)
        # fused greedy head (projection + arg-max over rows and ranks in one launch): needs peer memory
        # for the exchange, i.e. one rank or the P2P communicator; NCCL-only groups use the torch ops below
        self.head_tokens = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self.fused_head = hasattr(self.ops, "lm_head_argmax") and self.resid.is_cuda and max_batch <= 64 and \
            (t == 1 or getattr(self.comm, "handle", None) is not None)
        if self.fused_head:
            self.head_scratch = torch.zeros(self.ops.lm_head_argmax_scratch_bytes(), dtype=torch.uint8, device=device)
        nbytes = self.ops.attn_decode_scratch_bytes(max_batch, self.nh, self.nkv, self.hd, _MAX_SPLITS)
        self.scratch = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=device)
        # ladder decode runs the attention and MLP chains of a layer on two streams (LRI_LADDER_OVERLAP=0: one)
        self.overlap_sublayers = (self.family == "ladder" and self.resid.is_cuda and
                                  os.environ.get("LRI_LADDER_OVERLAP", "1") != "0")
        if self.overlap_sublayers:
            self.normed_m = buf(self.d)
            # (same priority as the main stream: giving the MLP chain, four fifths of a layer's bytes, the higher
            # priority was measured slower on B200, 2.80 against 2.58 ms per 8B step)
            self.side_stream = torch.cuda.Stream()
            self._events = [torch.cuda.Event() for _ in range(2 * cfg.n_layer + 2)]
        self.ready = True

    # ------------------------------------------------------------------------------------------
    def _attention(self, att, w_qkv, rows, B, S, pos, out, push=0):
        """push > 0: the output projection also pushes its partial to the peers on that channel."""
        ops = self.ops
        kc, vc = att.kv_cache.k_cache, att.kv_cache.v_cache
        ops.qkv_rope_kvcache(self.normed, w_qkv, self.model.freqs_cis, False, pos, self.q, kc, vc, B, S, self.nh,
                             self.nkv, self.hd, self.ws_qkv)
        ops.attention(self.q, kc, vc, pos, self.y, B, S, self.nh, self.nkv, self.hd, self.scratch, self._splits)
        if push:
            self.comm.linear_push(self.y, att.wo.weight, out, rows, push)
        else:
            ops.linear(self.y, att.wo.weight, out, rows, workspace=self.ws_wo)

    def _mlp(self, w1, w2, rows, out, addend=None, normed=None, push=0):
        self.ops.gateup_swiglu(self.normed if normed is None else normed, w1, self.h, rows, self.ws_ug)
        if push:
            self.comm.linear_push(self.h, w2, out, rows, push, addend=addend)
        else:
            self.ops.linear(self.h, w2, out, rows, addend=addend, workspace=self.ws_w2)

    def _norm(self, weight, rows, add1=None, add2=None, scale=1.0, write_residual=True, normed=None, ch1=0, ch2=0):
        """residual += adds (in place), normed = RMSNorm(residual) * weight.  With ch1 / ch2 > 0 the
        addend is this rank's partial and the sum over ranks is gathered inside the kernel from the
        message pushed on that channel (the reduction half of the all-reduce)."""
        res_out = self.resid if (write_residual and (add1 is not None or add2 is not None or scale != 1.0)) else None
        out = self.normed if normed is None else normed
        if (ch1 and add1 is not None) or (ch2 and add2 is not None):
            self.comm.add_rmsnorm_gather(self.resid, ch1 if add1 is not None else 0, add1,
                                         ch2 if add2 is not None else 0, add2, weight, self.cfg.norm_eps, res_out, out,
                                         rows, scale, self_push=self._norm_pushes)
        else:
            self.ops.add_rmsnorm(self.resid, add1, add2, weight, self.cfg.norm_eps, res_out, out, rows, scale)

    def _reduce_plan(self, rows, hidden=False):
        """(ca, cm, pa, pm, in_norm): the channels on which the norms gather the attention / MLP partial
        (0: they read an all-reduced buffer), the channels on which the projections push from their
        epilogue (0: they do not; with the fused form the norm pushes itself), and whether the
        reduction happens inside the norm at all."""
        mode = self.comm.reduce_mode(rows * self.d, rows, hidden=hidden)
        self._norm_pushes = mode == "fused"
        if mode == "kernel":
            return 0, 0, 0, 0, False
        if mode == "split":
            return 1, 2, 1, 2, True
        return 1, 2, 0, 0, True

    def _issue(self, buf, rows, channel, split):
        """Start the all-reduce of a partial.  Split form: the projection has pushed it already and the
        consuming norm reduces it, nothing to do; else launch the asynchronous all-reduce."""
        if split:
            return None
        return self.comm.all_reduce_async(buf, rows)

    # ------------------------------------------------------------------------------------------
    def _trunk(self, idx, input_pos):
        """Everything up to the final norm; leaves the normalised hidden states in self.normed."""
        assert self.ready, "Caches must be initialized first"
        B, S = idx.shape
        assert input_pos.shape[0] == S, "input_pos must hold one position per token column"
        assert B <= self.max_batch and S <= self.max_seq, "batch or sequence exceeds setup_caches() sizes"
        if input_pos.dtype not in (torch.int32, torch.int64):
            input_pos = input_pos.to(torch.int64)
        rows = B * S
        self._splits = decode_splits(B, self.nh, self.nkv, self.model.max_seq_length, self.hd) if S == 1 else 1
        self.ops.embedding(self.model.tok_embeddings.weight, idx, self.resid)
        getattr(self, "_run_" + self.family)(rows, B, S, input_pos)
        return B, S, rows

    @torch.no_grad()
    def forward(self, idx, input_pos):
        B, S, rows = self._trunk(idx, input_pos)
        logits = torch.empty(B, S, self.cfg.vocab_size, dtype=self.resid.dtype, device=self.resid.device)
        self.ops.linear(self.normed, self.model.output.weight, logits, rows, workspace=self.ws_head)
        return logits

    @torch.no_grad()
    def forward_last(self, idx, input_pos):
        """Prompt pass that returns the logits of the last position only, [B, 1, V].  The reference
        computes the output projection for every position (gpt_fast/gpt_ladder_TP.py:282-283) although
        its generation loop reads only the last one (benchmark.py:82-83); for a long prompt that is
        most of the LM-head work (32 x 4096 positions x 128256 logits = 33.6 GB of output)."""
        B, S, rows = self._trunk(idx, input_pos)
        last = self.normed[:rows].view(B, S, self.d)[:, -1].contiguous()
        logits = torch.empty(B, 1, self.cfg.vocab_size, dtype=self.resid.dtype, device=self.resid.device)
        self.ops.linear(last, self.model.output.weight, logits, B, workspace=self.ws_head)
        return logits

    @torch.no_grad()
    def forward_greedy(self, idx, input_pos):
        """Decode step that returns the arg-max token of every sequence, int32 [B, 1], instead of logits.

        The output projection is replicated on every rank (reference gpt_fast/gpt_ladder_TP.py:218, 283),
        and streaming all of it is the largest single item of a decode step at high TP.  Here rank r
        multiplies only rows [r V/t, (r+1) V/t) of its copy, takes the arg-max of its slice, and the
        ranks exchange one (value, index) pair per sequence.  Up to 8 sequences the streaming kernels
        compute every logit with a fixed K order whatever other rows are computed, so the token is
        exactly the one `forward(...).argmax(-1)` gives (lowest index on ties), on every rank.  From 9
        sequences on the stream-K kernel cuts K per tile by the number of tiles, which differs between
        the full and the sliced head: logits agree to one rounding of the storage type and a near-tie
        may resolve differently.
        """
        import torch.distributed as dist
        B, S, rows = self._trunk(idx, input_pos)
        assert S == 1, "forward_greedy is a decode step (one position per sequence)"
        n = self.vocab_hi - self.vocab_lo
        t = self.comm.world
        if self.fused_head and (t == 1 or getattr(self.comm, "handle", None) is not None):
            self.ops.lm_head_argmax(self.normed, self.model.output.weight[self.vocab_lo:self.vocab_hi], self.vocab_lo,
                                    self.head_tokens, B, self.head_scratch, getattr(self.comm, "handle", None),
                                    logits_ws=self.head_logits, workspace=self.ws_head,
                                    timeout_ms=getattr(self.comm, "timeout_ms", 2000))
            return self.head_tokens[:B].view(B, 1)
        mine = self.head_best[self.comm.rank, :B]
        if n > 0:
            local = self.head_logits[: B * n].view(B, n)
            self.ops.linear(self.normed, self.model.output.weight[self.vocab_lo:self.vocab_hi], local, B,
                            workspace=self.ws_head)
            val, ix = local.float().max(dim=-1)
            mine[:, 0] = val
            mine[:, 1] = ix + self.vocab_lo  # exact in fp32: vocabularies are far below 2**24
        else:
            mine[:, 0] = float("-inf")
            mine[:, 1] = 0
        if t == 1:
            return mine[:, 1].to(torch.int32).view(B, 1)
        best = self.head_best[:, :B].contiguous() if B != self.max_batch else self.head_best
        dist.all_gather_into_tensor(best.view(-1), mine.contiguous().view(-1))
        vals, ids = best[..., 0], best[..., 1]
        top = vals.max(dim=0).values
        winner = torch.where(vals == top, ids, torch.full_like(ids, float("inf"))).min(dim=0).values
        return winner.to(torch.int32).view(B, 1)

    @torch.no_grad()
    def forward_sample(self, idx, input_pos, temperature=1.0, top_k=None, generator=None):
        """Decode step that returns one sampled token per sequence, int32 [B, 1], from the reference's
        sampling rule (benchmark.py:56-77: logits / max(temperature, 1e-5), optional top-k cut at the
        k-th largest value, softmax, argmax(probs / q) with q ~ Exponential(1)), with the output
        projection split by vocabulary as in forward_greedy.

        Every rank draws the same [B, V] noise (same generator state on every rank, as the reference
        seeds its ranks alike) and uses its slice, so all ranks return the same token.  The k-th
        largest value comes from the ranks' local top-k lists, the softmax normaliser from an
        all-reduce of the local maxima and sums; probabilities are rounded to the model type as the
        reference's softmax output is, so the draw is the reference's up to the rounding of the
        normaliser (summation order differs)."""
        import torch.distributed as dist
        B, S, rows = self._trunk(idx, input_pos)
        assert S == 1, "forward_sample is a decode step (one position per sequence)"
        t, V = self.comm.world, self.cfg.vocab_size
        n = self.vocab_hi - self.vocab_lo
        dtype, dev = self.resid.dtype, self.resid.device
        local = self.head_logits[: B * max(n, 1)].view(B, max(n, 1))
        if n > 0:
            self.ops.linear(self.normed, self.model.output.weight[self.vocab_lo:self.vocab_hi], local, B,
                            workspace=self.ws_head)
            x = local / max(temperature, 1e-5)
        else:
            x = torch.full((B, 1), float("-inf"), dtype=dtype, device=dev)

        def gathered(v):  # [B, c] on every rank -> [t, B, c]
            if t == 1:
                return v.unsqueeze(0)
            out = torch.empty((t,) + tuple(v.shape), dtype=v.dtype, device=dev)
            dist.all_gather_into_tensor(out.view(-1), v.contiguous().view(-1))
            return out

        if top_k is not None:
            k = min(top_k, V)
            mine = torch.full((B, k), float("-inf"), dtype=dtype, device=dev)
            kl = min(k, x.shape[1])
            mine[:, :kl] = torch.topk(x, kl).values
            cand = gathered(mine).permute(1, 0, 2).reshape(B, t * k)
            kth = torch.topk(cand, k).values[:, -1:]
            x = torch.where(x < kth, torch.full_like(x, float("-inf")), x)
        xf = x.float()
        top = gathered(xf.max(dim=-1, keepdim=True).values).max(dim=0).values          # [B, 1]
        e = torch.exp(xf - top)
        total = gathered(e.sum(dim=-1, keepdim=True)).sum(dim=0)                        # [B, 1], rank order
        probs = (e / total).to(dtype)
        q = torch.empty(B, V, dtype=dtype, device=dev).exponential_(1, generator=generator)
        score = (probs / q[:, self.vocab_lo:self.vocab_lo + x.shape[1]]).float() if n > 0 else xf
        val, ix = score.max(dim=-1)
        mine = torch.stack([val, (ix + self.vocab_lo).float()], dim=-1)                 # [B, 2]
        best = gathered(mine)
        vals, ids = best[..., 0], best[..., 1]
        win = torch.where(vals == vals.max(dim=0).values, ids, torch.full_like(ids, float("inf"))).min(dim=0).values
        return win.to(torch.int32).view(B, 1)

    # Each _run_* leaves RMSNorm(final residual) * norm.weight in self.normed.
    def _run_ladder(self, rows, B, S, pos):
        mixed = getattr(self.cfg, "ladder_layers", None)
        if mixed is not None and len(set(mixed)) != self.cfg.n_layer:
            return self._run_hybrid(rows, B, S, pos, set(mixed))
        if S == 1 and self.overlap_sublayers:
            return self._run_ladder_two_streams(rows, B, S, pos)
        comm, m = self.comm, self.model
        ca, cm, pa, pm, split = self._reduce_plan(rows, hidden=True)
        h_a = h_m = None
        first = True
        for layer in m.layers:
            comm.wait(h_a)
            self._norm(layer.attention_norm.weight, rows, add1=None if first else self.part_a, ch1=ca)
            self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a, push=pa)
            h_a = self._issue(self.part_a, rows, 1, split)
            comm.wait(h_m)
            self._norm(layer.ffn_norm.weight, rows, add1=None if first else self.part_m, ch1=cm)
            self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m, push=pm)
            h_m = self._issue(self.part_m, rows, 2, split)
            first = False
        comm.wait(h_a)
        comm.wait(h_m)
        self._norm(m.norm.weight, rows, add1=self.part_a, add2=self.part_m, write_residual=False, ch1=ca, ch2=cm)

    def _run_ladder_two_streams(self, rows, B, S, pos):
        """Decode form of the ladder schedule.  In a ladder block the MLP of layer i reads the
        residual BEFORE the attention output of layer i is added, so the attention chain
        (add+norm, QKV, attention, wo) and the MLP chain (add+norm, gate/up, w2) of one layer do
        not depend on each other.  They run on two streams: the latency-bound attention kernels
        hide behind the weight streaming of the MLP, the same slack the reference uses to hide
        its all-reduces.  Arithmetic and the order of the residual adds are unchanged:
            main:  r += P_a(i-1); A_i = attn(norm(r))        side:  r += P_m(i-1); M_i = mlp(norm(r))
        with the side add of layer i ordered after the main add of layer i and before the main add
        of layer i+1 by events."""
        comm, m = self.comm, self.model
        ca, cm, pa, pm, split = self._reduce_plan(rows, hidden=True)
        main = torch.cuda.current_stream()
        side = self.side_stream
        ev = self._events
        ev[0].record(main)
        side.wait_event(ev[0])  # fork (the embedding gather is complete)
        h_a = h_m = None
        n = 1
        first = True
        for layer in m.layers:
            e_attn_add, e_mlp_add = ev[n], ev[n + 1]
            n += 2
            comm.wait(h_a)
            self._norm(layer.attention_norm.weight, rows, add1=None if first else self.part_a, ch1=ca)
            e_attn_add.record(main)
            self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a, push=pa)
            h_a = self._issue(self.part_a, rows, 1, split)
            with torch.cuda.stream(side):
                side.wait_event(e_attn_add)
                comm.wait(h_m)
                self._norm(layer.ffn_norm.weight, rows, add1=None if first else self.part_m, normed=self.normed_m,
                           ch1=cm)
                e_mlp_add.record(side)
                self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m,
                          normed=self.normed_m, push=pm)
                h_m = self._issue(self.part_m, rows, 2, split)
            main.wait_event(e_mlp_add)  # the next attention add reads the residual the MLP add wrote
            first = False
        ev[n].record(side)
        main.wait_event(ev[n])  # join: the last w2 (and its all-reduce issue) is ordered before the final add
        comm.wait(h_a)
        comm.wait(h_m)
        self._norm(m.norm.weight, rows, add1=self.part_a, add2=self.part_m, write_residual=False, ch1=ca, ch2=cm)

    def _run_hybrid(self, rows, B, S, pos, ladder):
        """Some layers ladder, the others dense (a converted checkpoint's `ladder_layers`, reference
        hf_modeling_utils/modeling_llama_ladder.py:627-663, 889-948).  The residual carries two pending
        addends as in the ladder schedule; a dense layer adds both before its attention, consumes its
        attention all-reduce at once and leaves only its MLP output pending:
            ladder   r += P_a; A = attn(norm(r)) -> pending;  r += P_m; M = mlp(norm(r)) -> pending
            dense    r += P_a + P_m; r += AR(attn(norm(r)));  M = mlp(norm(r)) -> pending, P_a = none"""
        comm, m = self.comm, self.model
        h_a = h_m = None
        have_a = have_m = False
        for i, layer in enumerate(m.layers):
            if i in ladder:
                comm.wait(h_a)
                self._norm(layer.attention_norm.weight, rows, add1=self.part_a if have_a else None)
                self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a)
                h_a = comm.all_reduce_async(self.part_a, rows)
                comm.wait(h_m)
                self._norm(layer.ffn_norm.weight, rows, add1=self.part_m if have_m else None)
                self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m)
                h_m = comm.all_reduce_async(self.part_m, rows)
                have_a = have_m = True
            else:
                comm.wait(h_a)
                comm.wait(h_m)
                self._norm(layer.attention_norm.weight, rows, add1=self.part_a if have_a else None,
                           add2=self.part_m if have_m else None)
                self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a)
                comm.all_reduce(self.part_a, rows)
                self._norm(layer.ffn_norm.weight, rows, add1=self.part_a)
                self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m)
                h_a, h_m = None, comm.all_reduce_async(self.part_m, rows)
                have_a, have_m = False, True
        comm.wait(h_a)
        comm.wait(h_m)
        self._norm(m.norm.weight, rows, add1=self.part_a if have_a else None, add2=self.part_m if have_m else None,
                   write_residual=False)

    def _reduce_now(self, buf, rows, channel, split):
        """All-reduce consumed by the very next norm: pushed (and gathered there) or done in-stream."""
        if not split:
            self.comm.all_reduce(buf, rows)

    def _run_dense(self, rows, B, S, pos):
        comm, m = self.comm, self.model
        ca, cm, pa, pm, split = self._reduce_plan(rows)
        pending = None
        for layer in m.layers:
            self._norm(layer.attention_norm.weight, rows, add1=pending, ch1=cm)
            self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a, push=pa)
            self._reduce_now(self.part_a, rows, 1, split)
            self._norm(layer.ffn_norm.weight, rows, add1=self.part_a, ch1=ca)
            self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m, push=pm)
            self._reduce_now(self.part_m, rows, 2, split)
            pending = self.part_m
        self._norm(m.norm.weight, rows, add1=pending, write_residual=False, ch1=cm)

    def _run_parallel(self, rows, B, S, pos):
        comm, m = self.comm, self.model
        _, cm, _, pm, split = self._reduce_plan(rows)
        pending = None
        for layer in m.layers:
            att = layer.attention
            self._norm(layer.attention_norm.weight, rows, add1=pending, ch1=cm)
            w = att.wqkv1.weight
            nqkv = att.qkv_rows
            self._attention(att, w[:nqkv], rows, B, S, pos, self.part_a)
            self._mlp(w[nqkv:], att.w2.weight, rows, self.part_m, addend=self.part_a, push=pm)
            self._reduce_now(self.part_m, rows, 2, split)
            pending = self.part_m
        self._norm(m.norm.weight, rows, add1=pending, write_residual=False, ch1=cm)

    def _run_desync(self, rows, B, S, pos):
        comm, m = self.comm, self.model
        t = comm.world
        pending = None  # a partial that still has to be added to the rank-local residual

        def fold_and_reduce(partial):
            # residual = all_reduce(partial + residual / t)
            self.ops.add_rmsnorm(self.resid, partial, None, None, self.cfg.norm_eps, self.resid, None, rows, 1.0 / t)
            comm.all_reduce(self.resid, rows)

        for layer in m.layers:
            self._norm(layer.attention_norm.weight, rows, add1=pending)
            self._attention(layer.attention, layer.attention.wqkv.weight, rows, B, S, pos, self.part_a)
            if layer.do_attention_all_reduce:
                fold_and_reduce(self.part_a)
                pending = None
            else:
                pending = self.part_a
            self._norm(layer.ffn_norm.weight, rows, add1=pending)
            self._mlp(layer.feed_forward.w1.weight, layer.feed_forward.w2.weight, rows, self.part_m)
            if layer.do_mlp_all_reduce:
                fold_and_reduce(self.part_m)
                pending = None
            else:
                pending = self.part_m
        self._norm(m.norm.weight, rows, add1=pending, write_residual=False)
