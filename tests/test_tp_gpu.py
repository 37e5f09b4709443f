"""Tensor-parallel tests on 2 GPUs (skipped on a single-GPU box): the one-shot peer all-reduce,
whole-model parity at TP = 2 against the reference's fixtures under both communication back ends,
graph capture with the communication stream, and the bounded wait of the all-reduce."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_worker():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29811", os.path.join(ROOT, "tests", "tp_gpu_worker.py")]
    # NVLS off: a rank that leaves while its memory is bound to an NVLink switch-reduction object can fault its peers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    sys.stdout.write(r.stdout[-4000:])
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    assert "TP-GPU-OK" in r.stdout
