"""Builds and runs the C++ mirror of the reference's tests/test_linear_sumcheck.rs
(tests/host_cpp/test_linear_sumcheck.cpp) against libzkb200.so on the GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_mirror_linear_sumcheck():
    src = os.path.join(ROOT, "tests", "host_cpp", "test_linear_sumcheck.cpp")
    exe = os.path.join(ROOT, "tests", "host_cpp", "test_linear_sumcheck.bin")
    libdir = os.path.join(ROOT, "zkes_b200")
    subprocess.run(["g++", "-O1", "-std=c++17", "-x", "c++", src, "-o", exe, f"-L{libdir}", "-lzkb200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failure(s)" in r.stdout
