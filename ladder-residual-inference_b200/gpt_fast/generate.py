"""Device-side greedy decode loop.

The reference decodes one token per host iteration: `decode_n_tokens` calls the model, clones the
token, bumps `input_pos` from Python (benchmark.py:95-115), and `generate_using_cuda_graphs` replays
one graph per token with `copy_` of the inputs in between (benchmark.py:167-225).  Once a decode step
takes a few hundred microseconds that host work is a visible share of it.

`DeviceLoop` keeps the whole feedback on the device: the next token is written straight into the
token buffer the next step reads, the position tensor is incremented by a kernel, and `steps_per_replay`
consecutive steps are captured into ONE CUDA graph.  The host replays a graph every `steps_per_replay`
tokens and reads the tokens back once at the end.
"""
from typing import Optional

import torch


class DeviceLoop:
    def __init__(self, model, batch_size: int, steps_per_replay: int = 8, head: str = "replicated"):
        """model: a GPT* of this package with caches set up for at least `batch_size`.
        head: "replicated" (arg-max of model(...) logits, the reference's scheme) or "vocab-parallel"
        (model.decode_greedy)."""
        assert head in ("replicated", "vocab-parallel")
        assert steps_per_replay >= 1
        self.model, self.k, self.head = model, steps_per_replay, head
        dev = model.output.weight.device
        self.tok = torch.zeros(batch_size, 1, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.zeros(batch_size, steps_per_replay, dtype=torch.int32, device=dev)
        self._graphs = {}

    def _steps(self, n: int):
        with torch.no_grad():
            for s in range(n):
                if self.head == "vocab-parallel":
                    nxt = self.model.decode_greedy(self.tok, self.pos)
                else:
                    nxt = torch.argmax(self.model(self.tok, self.pos)[:, -1], dim=-1, keepdim=True).to(torch.int32)
                self.out[:, s:s + 1].copy_(nxt)
                self.tok.copy_(nxt)
                self.pos.add_(1)

    def _graph(self, n: int) -> torch.cuda.CUDAGraph:
        """Graph of n consecutive steps; captured once (the warm-up steps advance the position, which
        the caller's start() sets afterwards)."""
        if n not in self._graphs:
            tok0, pos0 = self.tok.clone(), self.pos.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._steps(1)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.tok.copy_(tok0)
            self.pos.copy_(pos0)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._steps(n)
            # the capture executed nothing: token and position are still the caller's
            self._graphs[n] = g
        return self._graphs[n]

    def start(self, first_token: torch.Tensor, position: int) -> None:
        """first_token [B, 1]: the token to feed at `position` (e.g. the arg-max of the prompt pass)."""
        self.tok.copy_(first_token.to(torch.int32))
        self.pos.fill_(position)

    def run(self, n_new: int, max_position: Optional[int] = None) -> torch.Tensor:
        """Decodes n_new tokens after start(); returns them as int32 [B, n_new] on the device.
        max_position: size of the KV cache (defaults to the model's max_seq_length); a replay of
        steps_per_replay steps is only used while it stays inside the cache."""
        limit = self.model.max_seq_length if max_position is None else max_position
        hist = torch.empty(self.tok.shape[0], n_new, dtype=torch.int32, device=self.tok.device)
        # graphs are captured before the loop so that capture never interleaves with replays
        done = 0
        pos = int(self.pos.item())
        assert pos + n_new <= limit, "the KV cache is too short for this many tokens"
        plan = []
        while done < n_new:
            n = self.k if n_new - done >= self.k else 1
            plan.append(n)
            done += n
        for n in set(plan):
            self._graph(n)
        done = 0
        for n in plan:
            self._graphs[n].replay()
            hist[:, done:done + n].copy_(self.out[:, :n])
            done += n
        return hist
