"""The one-SM GEMM kernels are the fallback when CTA pairs are not wanted (AXM_GEMM_2SM=0) or
cannot be scheduled.  The switch is read once per process, so the forward and backward GEMM
tests are run again in a child process with the switch set."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_gemm_tests_pass_on_the_one_sm_kernels(cuda_device):
    env = dict(os.environ, AXM_GEMM_2SM="0")
    r = subprocess.run(
        [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
         os.path.join(HERE, "test_ffn_gpu.py"), os.path.join(HERE, "test_ffn_backward_gpu.py")],
        env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
