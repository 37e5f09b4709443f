"""pytest configuration: the `gpu` marker, import paths for the product package and the oracle, and
a build of the C-ABI library when it is not there yet (nvcc cross-compiles without a GPU)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ladder-residual-inference_b200")
for p in (ROOT, PKG, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    if not os.path.exists(os.path.join(PKG, "liblri_b200.so")):
        subprocess.run([sys.executable, os.path.join(PKG, "build.py")], check=True)
