"""The host-side field inversion of the commitments' affine form (zkes_b200/csrc/msm.hpp: inverse_host, 64-bit limbs)
against the shared field code, compiled and run on the CPU (no GPU call is made; nvcc is only the compiler)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_inverse_host_matches_shared_field_code(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    exe = str(tmp_path / "host_field_check")
    cmd = [nvcc, "-O2", "-std=c++17", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "zkes_b200", "csrc"), "-o", exe, os.path.join(ROOT, "tests", "host_field_check.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr
