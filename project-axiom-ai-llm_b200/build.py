"""Builds the CUDA libraries of this package in-tree with nvcc for sm_100a.

  libaxm_moe.so         the layer behind include/axm_moe.h
  libaxm_moe_dropin.so  the three symbols of the reference engine's MoE interface

Run as a script or call build().  Nothing is installed outside this directory.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaxm_moe.so")
DROPIN = os.path.join(HERE, "libaxm_moe_dropin.so")

CORE_SOURCES = ["moe_api.cu", "router.cu", "router_tc.cu", "permute.cu", "grouped_ffn.cu", "noalloc.cu",
                "ep_exchange.cu", "ep_layer.cu", "ep_train.cu", "grouped_bwd.cu", "backward.cu",
                "grouped_ffn_2sm.cu", "grouped_bwd_2sm.cu", "checkpoint.cu"]
DROPIN_SOURCES = ["dropin.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    deps = list(sources) + headers + [os.path.join(HERE, "..", "include", "axm_moe.h"), __file__]
    return any(os.path.getmtime(s) > t for s in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def _compile_objects(sources, extra, force, verbose):
    """One object per source under csrc/build/, compiled in parallel; an object is
    rebuilt when its source, a header or this script is newer."""
    from concurrent.futures import ThreadPoolExecutor
    obj_dir = os.path.join(CSRC, "build")
    os.makedirs(obj_dir, exist_ok=True)
    objs, jobs = [], []
    for src in sources:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src]):
            jobs.append([_nvcc()] + NVCC_FLAGS + extra + ["-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    return objs, bool(jobs)


def build(force=False, verbose=True, ptxas_info=False):
    core = [os.path.join(CSRC, s) for s in CORE_SOURCES]
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    if force or _stale(LIB, core):
        objs, _ = _compile_objects(core, extra, force, verbose)
        _run([_nvcc()] + NVCC_FLAGS + ["-shared", "-o", LIB] + objs + ["-cudart", "shared"], verbose)
    drop = [os.path.join(CSRC, s) for s in DROPIN_SOURCES]
    if all(os.path.exists(s) for s in drop) and (force or _stale(DROPIN, drop + [LIB])):
        _run([_nvcc()] + NVCC_FLAGS + ["-shared", "-o", DROPIN] + drop +
             ["-L" + HERE, "-laxm_moe", "-Xlinker", "-rpath=$ORIGIN", "-cudart", "shared", "-ldl"], verbose)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
