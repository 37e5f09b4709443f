"""All-reduce back ends for the row-parallel partial sums (one process per GPU).

`all_reduce_async(t)` starts an in-place SUM over the TP group and returns a handle;
`wait(handle)` makes the CURRENT stream wait for it (a stream dependency, not a host sync).
Issuing and waiting are separate because the ladder schedule consumes a sublayer's all-reduce
one sublayer later (the reference: gpt_fast/gpt_ladder_TP.py:323-356 with
gpt_fast/utils.py:390-397).

  NoComm       world size 1.
  TorchComm    torch.distributed all_reduce(async_op=True): NCCL runs on c10d's own stream (the
               dedicated communication stream), gloo in CPU tests.
  P2PComm      the hand-written one-shot NVLink all-reduce (lri_allreduce) on a dedicated
               high-priority stream with event fork/join, for messages up to `max_elems`;
               larger messages go to TorchComm.
`make_comm()` picks by the LRI_COMM environment variable: "nccl", "p2p" or "auto" (default;
p2p for small messages when peers are reachable, else nccl).
"""
import ctypes
import os

import torch
import torch.distributed as dist

P2P_MAX_BYTES_DEFAULT = 2 * 1024 * 1024


def p2p_max_bytes(world):
    """Largest message the peer all-reduce kernels take before NCCL does, from the measured latency table
    (`bench.py --mode comm` on one 8 x B200 host): with 2 ranks the one-shot kernel wins up to the 8 MiB
    measured (30.9 vs 42.8 us at 4 MiB), with 8 ranks every rank pushes 7 copies and NCCL wins from 2 MiB
    on (45.6 vs 37.9 us) while the kernel wins at 1 MiB (31.6 vs 34.6 us); 4 ranks take the value between."""
    return {2: 8 << 20, 3: 4 << 20, 4: 2 << 20}.get(world, 1 << 20 if world > 4 else 8 << 20)


class NoComm:
    world = 1
    rank = 0
    name = "none"

    def can_split(self, count, rows=1, hidden=False):
        return False

    def reduce_mode(self, count, rows=1, hidden=False):
        return "kernel"

    def all_reduce_async(self, t, rows=None):
        return None

    def wait(self, handle):
        return None

    def all_reduce(self, t, rows=None):
        return None

    def status(self):
        return None


class ElidedComm(NoComm):
    """The tensor-parallel group with every collective left out: same interface, all-reduces are
    no-ops, so the engine launches exactly the kernels of a step minus the communication.  For
    timing only (the step with communication minus this one is the exposed all-reduce time, the
    reference's "upper bound" notion, gpt_fast/gpt_desync_TP.py:165-176); the logits are those of
    unreduced partial sums."""
    name = "elided"

    def __init__(self, world, rank, like=None):
        self.world, self.rank = world, rank
        # the greedy head's (value, index) exchange is not an all-reduce and stays as it is
        self.handle = getattr(like, "handle", None)
        self.timeout_ms = getattr(like, "timeout_ms", 2000)


class TorchComm:
    name = "torch.distributed"

    def can_split(self, count, rows=1, hidden=False):
        return False

    def reduce_mode(self, count, rows=1, hidden=False):
        return "kernel"

    def __init__(self):
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()

    def all_reduce_async(self, t, rows=None):
        if rows is not None and rows != t.shape[0]:
            t = t[:rows]
        return dist.all_reduce(t, async_op=True)

    def wait(self, handle):
        if handle is not None:
            handle.wait()

    def all_reduce(self, t, rows=None):
        """In-stream all-reduce: later work on the current stream sees the sum."""
        if rows is not None and rows != t.shape[0]:
            t = t[:rows]
        dist.all_reduce(t)

    def status(self):
        return None


class _P2PHandle:
    __slots__ = ("event",)

    def __init__(self, event):
        self.event = event


class P2PComm:
    name = "p2p-oneshot"

    def __init__(self, max_bytes=P2P_MAX_BYTES_DEFAULT, timeout_ms=2000):
        from . import _C
        self._C = _C
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.timeout_ms = timeout_ms
        self.max_elems = max_bytes // 2
        self.fallback = TorchComm()
        handle = ctypes.c_void_p()
        ipc = ctypes.create_string_buffer(64)
        rc = _C.lib.lri_comm_create(self.rank, self.world, self.max_elems, ctypes.byref(handle), ipc)
        err = _C.lib.lri_last_error().decode() if rc < 0 else ""
        self.handle = handle if rc == 0 else None
        # every step that can fail on one rank alone is followed by an exchange of the outcome,
        # so that all ranks take the same decision and nobody waits in a collective alone
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (rc, bytes(ipc.raw)))
        if any(g[0] != 0 for g in gathered):
            self.close()
            raise RuntimeError(f"P2P all-reduce set-up failed on a rank (local status {rc} {err})")
        rc = _C.lib.lri_comm_connect(self.handle, b"".join(g[1] for g in gathered))
        err = _C.lib.lri_last_error().decode() if rc < 0 else ""
        outcomes = [None] * self.world
        dist.all_gather_object(outcomes, rc)
        if any(o != 0 for o in outcomes):
            self.close()
            raise RuntimeError(f"P2P all-reduce peer mapping failed on a rank (local status {rc} {err})")
        # events are created up front: torch records into an existing event during graph capture
        self.stream = torch.cuda.Stream(priority=-1)
        self._ready = [torch.cuda.Event() for _ in range(4)]
        self._done = [torch.cuda.Event() for _ in range(4)]
        self._n = 0
        self._push_max = _C.lib.lri_comm_push_max_elems()
        self.split_mode = os.environ.get("LRI_SPLIT_AR", "auto")

    def all_reduce_async(self, t, rows=None):
        if rows is not None and rows != t.shape[0]:
            t = t[:rows]
        count = t.numel()
        if count > self.max_elems or count % 8 != 0:
            return self.fallback.all_reduce_async(t)
        i = self._n % 4
        self._n += 1
        ready, done = self._ready[i], self._done[i]
        ready.record()  # on the current (compute) stream: the partial is complete
        self.stream.wait_event(ready)
        self._C.check(self._C.lib.lri_allreduce(self.handle, self._C.dtype_code(t.dtype), t.data_ptr(), t.data_ptr(),
                                                 count, self.timeout_ms, self.stream.cuda_stream))
        done.record(self.stream)
        return _P2PHandle(done)

    def wait(self, handle):
        if handle is None:
            return
        if isinstance(handle, _P2PHandle):
            torch.cuda.current_stream().wait_event(handle.event)
        else:
            handle.wait()

    def all_reduce(self, t, rows=None):
        """In-stream all-reduce for schedules that consume the sum at once (dense, parallel,
        desync): the kernel runs on the current stream, so there is no event fork/join to pay."""
        if rows is not None and rows != t.shape[0]:
            t = t[:rows]
        count = t.numel()
        if count > self.max_elems or count % 8 != 0:
            dist.all_reduce(t)
            return
        self._C.check(self._C.lib.lri_allreduce(self.handle, self._C.dtype_code(t.dtype), t.data_ptr(), t.data_ptr(),
                                                 count, self.timeout_ms, torch.cuda.current_stream().cuda_stream))

    # ---- split all-reduce: push now, reduce inside the consuming add + RMSNorm ----------------
    def can_split(self, count, rows=1, hidden=False):
        """True when the partial of a row-parallel projection takes the split path: pushed from the
        projection's epilogue and reduced inside the consuming add + RMSNorm.  Used for single-row
        decode steps, where the fused push exists; larger steps use the all-reduce kernel.
        `hidden` says that the schedule consumes the sum a sublayer later (ladder): there the
        stand-alone kernel on the communication stream is already off the critical path and
        measured faster (2 ranks: slightly; 8 ranks: 1262 against 900 tokens/s).  The gathering norm
        polls its peers one after the other, so its cost grows with the number of ranks: with
        LRI_SPLIT_AR=auto the split path is taken only by the schedules that consume the sum at once
        and only at 2 ranks, where it was measured faster than kernel + norm; =1 forces it everywhere
        it exists, =0 turns it off, =fused selects the one-kernel form (see reduce_mode)."""
        if self.split_mode in ("0", "fused") or (self.split_mode == "auto" and (hidden or self.world > 2)):
            return False
        return rows == 1 and count % 8 == 0 and count <= self._push_max

    def reduce_mode(self, count, rows=1, hidden=False):
        """How the partial of a row-parallel projection of `count` elements becomes a sum:
        "kernel"  the all-reduce kernel (on the communication stream when the schedule hides it),
        "split"   pushed from the projection's epilogue, reduced inside the consuming add + RMSNorm,
        "fused"   pushed AND reduced inside the consuming add + RMSNorm (one launch, no stream hop;
                  any number of rows while the message fits a push channel).
        LRI_SPLIT_AR = auto | 0 | 1 | fused selects; every rank must use the same value."""
        if self.split_mode == "fused":
            return "fused" if (count % 8 == 0 and count <= self._push_max) else "kernel"
        return "split" if self.can_split(count, rows, hidden) else "kernel"

    def linear_push(self, x, w, out, rows, channel, addend=None):
        """out = x W^T (+ addend) with the result also pushed to the peers on `channel`."""
        C = self._C
        n, k = w.shape
        C.check(C.lib.lri_linear_push(self.handle, channel, C.dtype_code(x.dtype), x.data_ptr(), w.data_ptr(),
                                      C.ptr(addend), out.data_ptr(), rows, n, k,
                                      torch.cuda.current_stream().cuda_stream))

    def push(self, t, rows, channel):
        """Store rows [0, rows) of `t` into every peer's inbox on push channel 1 or 2 (current stream)."""
        count = rows * t.shape[1]
        self._C.check(self._C.lib.lri_comm_push(self.handle, channel, self._C.dtype_code(t.dtype), t.data_ptr(), count,
                                                torch.cuda.current_stream().cuda_stream))

    def add_rmsnorm_gather(self, residual, ch1, add1, ch2, add2, weight, eps, residual_out, normed_out, rows, scale=1.0,
                           self_push=False):
        """lri_add_rmsnorm with addends summed over the ranks' messages on a channel (> 0): messages
        pushed beforehand, or with self_push stored to the peers by the same kernel."""
        C = self._C
        fn = C.lib.lri_add_rmsnorm_allreduce if self_push else C.lib.lri_add_rmsnorm_gather
        C.check(fn(self.handle, C.dtype_code(residual.dtype), residual.data_ptr(), ch1, C.ptr(add1), ch2, C.ptr(add2),
                   float(scale), C.ptr(weight), float(eps), C.ptr(residual_out), C.ptr(normed_out), rows,
                   residual.shape[-1], self.timeout_ms, torch.cuda.current_stream().cuda_stream))

    def status(self):
        """Raises if a bounded peer wait gave up since the last check.  Waits for the compute stream
        (gathering norms and in-stream all-reduces run there) and for the communication stream."""
        torch.cuda.current_stream().synchronize()
        self._C.check(self._C.lib.lri_comm_status(self.handle, self.stream.cuda_stream))

    def close(self):
        if self.handle:
            self._C.lib.lri_comm_destroy(self.handle)
            self.handle = None


_COMM = None


def make_comm():
    """The process-wide communicator for the TP group (created once)."""
    global _COMM
    if _COMM is not None:
        return _COMM
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        _COMM = NoComm()
        return _COMM
    mode = os.environ.get("LRI_COMM", "auto").lower()
    if mode not in ("auto", "nccl", "p2p"):
        raise ValueError(f"LRI_COMM={mode!r}: expected auto, nccl or p2p")
    use_p2p = mode in ("auto", "p2p") and torch.cuda.is_available() and dist.get_backend() == "nccl" and world <= 8
    if use_p2p:
        try:
            _COMM = P2PComm(max_bytes=int(os.environ.get("LRI_P2P_MAX_BYTES", p2p_max_bytes(world))))
        except RuntimeError:
            if mode == "p2p":
                raise
            _COMM = TorchComm()
    else:
        _COMM = TorchComm()
    return _COMM


def reset_comm():
    global _COMM
    if isinstance(_COMM, P2PComm):
        _COMM.close()
    _COMM = None
