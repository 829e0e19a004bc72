"""Builds tests/cabi_host.cpp (plain C++ host over the C ABI, no Python in the data
path) against the shared library and runs it on the GPU."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_cpp_host_program(axm, tmp_path, cuda_device):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available to build the host program")
    libdir = os.path.dirname(axm.LIB_PATH)
    exe = str(tmp_path / "cabi_host")
    subprocess.run([nvcc, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), "-o", exe,
                    os.path.join(HERE, "cabi_host.cpp"), "-L" + libdir, "-laxm_moe", "-cudart", "shared",
                    "-Xlinker", "-rpath=" + libdir], check=True)
    env = dict(os.environ)
    import torch
    cudart_dir = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia", "cuda_runtime", "lib")
    env["LD_LIBRARY_PATH"] = cudart_dir + ":/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=120)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "OK" in r.stdout and "histogram_sum=512" in r.stdout
