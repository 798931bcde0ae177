"""Builds libirontensor_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m irontensor_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_OUT = os.path.join(_HERE, "libirontensor_b200.so")
_INC = os.path.join(os.path.dirname(_HERE), "include")


def _sources():
    deps = [os.path.join(_CSRC, f) for f in sorted(os.listdir(_CSRC)) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(_INC, "irontensor_b200.h"))
    return deps


def up_to_date():
    if not os.path.exists(_OUT):
        return False
    t = os.path.getmtime(_OUT)
    return all(os.path.getmtime(s) <= t for s in _sources())


def build(force=False, verbose=False):
    if not force and up_to_date():
        return _OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-o", _OUT, os.path.join(_CSRC, "it_capi.cu")]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    subprocess.run(cmd, check=True)
    return _OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(_OUT)
