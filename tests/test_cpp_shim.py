"""Builds the C++ nt:: host surface tests against libntb200.so (CPU: compile + link only) and runs them on the
GPU.  The binary mirrors the reference's own test cases for this path and reads its golden .npy vectors."""
import os
import subprocess

import pytest

from conftest import REF_GOLDEN, ROOT

BIN = os.path.join(ROOT, "tests", "cpp", "_build", "test_nt_shim")


def build_binary():
    from neurotensor_b200 import _lib
    _lib.lib()
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    src = os.path.join(ROOT, "tests", "cpp", "test_nt_shim.cpp")
    pkg = os.path.join(ROOT, "neurotensor_b200")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"), "-I", pkg, src, "-o", BIN,
           "-L", pkg, "-lntb200", "-Wl,-rpath," + pkg, "-pthread"]
    subprocess.check_call(cmd)
    return BIN


def test_cpp_shim_compiles_and_links():
    assert os.path.exists(build_binary())


@pytest.mark.gpu
def test_cpp_shim_cases_pass_on_gpu():
    build_binary()   # always against the current header and library: a stale binary would speak an old ABI
    r = subprocess.run([BIN, REF_GOLDEN], capture_output=True, text=True, timeout=600)
    print(r.stdout[-4000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "0 of" in r.stdout
