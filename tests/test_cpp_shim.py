"""The header-compatible C++ surface (include/lutGEMM): a program written like the reference's own
benchmark compiles and links against it (CPU check) and reproduces a host fp32 evaluation (GPU check)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "shim_check.cu")
EXE = os.path.join(ROOT, "tests", "cpp", "shim_check")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def build_shim_check():
    from lutgemm_b200 import _build
    _build.build()
    cmd = [NVCC, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"), SRC,
           "-L" + os.path.join(ROOT, "lutgemm_b200"), "-llutgemm_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../lutgemm_b200", "-o", EXE]
    subprocess.check_call(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return EXE


@pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not available")
def test_reference_style_program_compiles_and_links():
    exe = build_shim_check()
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_reference_style_program_runs():
    if not os.path.exists(EXE) or (os.path.exists(NVCC) and os.path.getmtime(EXE) < os.path.getmtime(SRC)):
        if not os.path.exists(NVCC):
            pytest.skip("shim_check was not built")
        build_shim_check()
    out = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "shim ok" in out.stdout
    assert "fields 512 1024 3 8 128" in out.stdout
