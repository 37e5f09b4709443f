"""Tensor-parallel tests on 2, 4 and 8 GPUs (each skipped when the box has fewer): the one-shot peer
all-reduce, whole-model parity of an 8-KV-head model against the oracle at the same number of ranks
and against the one-rank oracle, rank agreement, both communication back ends, graph capture with the
communication stream; at 2 ranks also the reference's TP = 2 fixtures and the bounded wait."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_worker(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29811 + world), os.path.join(ROOT, "tests", "tp_gpu_worker.py")]
    # NVLS off: a rank that leaves while its memory is bound to an NVLink switch-reduction object can fault its peers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1200, env=env)
    sys.stdout.write(r.stdout[-4000:])
    failures = "\n".join(line for line in (r.stdout + r.stderr).splitlines() if "TP-GPU-FAIL" in line)[:4000]
    assert r.returncode == 0, failures + "\n" + r.stdout[-2000:] + r.stderr[-2000:]
    assert f"TP-GPU-OK world={world}" in r.stdout
