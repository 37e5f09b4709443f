"""Per-operation device timing of an engine step (a debugging and measurement aid).

`trace_engine(engine)` wraps the engine's device ops and its communicator so that every call is
bracketed by CUDA events on the stream it runs on and by host clock readings; `report()` synchronises and
returns, per operation name, the number of calls, the summed device time and the summed host time of the
calls (a step whose host time exceeds its device time is bound by the launching thread, not by the GPU).  The events serialise nothing, but the step must
run eagerly (not inside a CUDA graph capture), and time spent waiting on another stream shows up in
the operation that waited.  The reference has no counterpart; its benchmark driver times whole
generations (benchmark.py:140-159)."""
import time

import torch


class _Timed:
    def __init__(self, target, names, log, prefix=""):
        self._target, self._names, self._log, self._prefix = target, set(names), log, prefix

    def __getattr__(self, name):
        attr = getattr(self._target, name)
        if name not in self._names or not callable(attr):
            return attr

        def call(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            t0 = time.perf_counter()
            out = attr(*a, **kw)
            host = time.perf_counter() - t0
            e1.record()
            self._log.append((self._prefix + name, e0, e1, host))
            return out

        return call


class EngineTrace:
    OPS = ("embedding", "add_rmsnorm", "linear", "qkv_rope_kvcache", "gateup_swiglu", "attention", "lm_head_argmax")
    COMM = ("all_reduce", "all_reduce_async", "wait", "linear_push", "add_rmsnorm_gather")

    def __init__(self, engine):
        self.engine, self.log = engine, []
        self._ops, self._comm = engine.ops, engine.comm
        engine.ops = _Timed(engine.ops, self.OPS, self.log)
        engine.comm = _Timed(engine.comm, self.COMM, self.log, prefix="comm.")

    def stop(self):
        self.engine.ops, self.engine.comm = self._ops, self._comm

    def report(self):
        """{name: (calls, device milliseconds, host milliseconds)} over everything recorded so far."""
        torch.cuda.synchronize()
        out = {}
        for name, e0, e1, host in self.log:
            n, ms, hs = out.get(name, (0, 0.0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1), hs + host * 1e3)
        return out


def trace_engine(engine):
    return EngineTrace(engine)
