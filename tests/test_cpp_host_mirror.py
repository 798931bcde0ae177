"""The C++ host mirror (include/irontensor_b200.hpp): it must compile and link against the C ABI
everywhere, and its test program (tests/cpp/host_mirror_test.cpp, modelled on the reference's own
unit tests) must pass on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
LIBDIR = os.path.join(ROOT, "irontensor_b200")


def build(out):
    from irontensor_b200 import _lib
    _lib.load()   # makes sure the shared library exists
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), SRC, "-L", LIBDIR,
                    "-lirontensor_b200", f"-Wl,-rpath,{LIBDIR}", "-o", out], check=True)


def test_cpp_host_mirror_compiles_and_links(tmp_path):
    build(str(tmp_path / "host_mirror_test"))


@pytest.mark.gpu
def test_cpp_host_mirror_runs(tmp_path):
    exe = str(tmp_path / "host_mirror_test")
    build(exe)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all checks passed" in out.stdout
