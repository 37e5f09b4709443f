"""Process-group bootstrap: torchrun environment -> one process per GPU, world == TP group.

Same contract as the reference's gpt_fast/tp.py:14-63: ranks and sizes come from LOCAL_RANK,
RANK, LOCAL_WORLD_SIZE and WORLD_SIZE; when no process group exists yet the CUDA device
LOCAL_RANK is selected and an NCCL group with a 600 s timeout is created; when the caller has
already created a group (any backend) it is left alone, which is how CPU tests substitute gloo.
Two additions: a single process started without torchrun gets a loop-back rendezvous address
instead of failing, and on a machine without a GPU the group falls back to gloo so that host
logic (presets, sharded module shapes, schedule bookkeeping) can be tested.
"""
import os
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist


def _env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, str(default)))


def local_rank() -> int:
    return _env_int("LOCAL_RANK", 0)


def is_local() -> bool:
    return local_rank() == 0


def local_break() -> None:
    """Debug helper of the reference (tp.py:34-37): breakpoint on local rank 0, barrier elsewhere."""
    if is_local():
        breakpoint()
    dist.barrier()


def maybe_init_dist() -> Optional[int]:
    rank = local_rank()
    global_rank = _env_int("RANK", 0)
    world = _env_int("LOCAL_WORLD_SIZE", 1)
    global_world = _env_int("WORLD_SIZE", 1)
    if dist.is_initialized():
        return rank
    if global_world == 1 and world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29400 + os.getpid() % 1000))
    has_gpu = torch.cuda.is_available()
    if has_gpu:
        torch.cuda.set_device(rank)
    backend = "nccl" if has_gpu else "gloo"
    if global_world > 1:
        dist.init_process_group(backend=backend, rank=global_rank, world_size=global_world,
                                timeout=timedelta(seconds=600))
    else:
        dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=timedelta(seconds=600))
    return rank
