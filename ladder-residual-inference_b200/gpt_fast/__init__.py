"""Drop-in `gpt_fast` package: the reference's model classes backed by sm_100a kernels.

Importing the package initialises the process group when none exists (one process per GPU,
torchrun environment), as the reference does at import time.
"""
from .gpt_dense_TP import GPTDense
from .gpt_desync_TP import GPTDesync
from .gpt_ladder_TP import GPTLadder
from .gpt_parallel_TP import GPTParallel
from .tp import maybe_init_dist

__all__ = ["GPTDense", "GPTDesync", "GPTLadder", "GPTParallel", "maybe_init_dist"]
