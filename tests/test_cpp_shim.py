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
    assert "fields 512 1024 3 8 128" in out.stdout and " wx " in out.stdout


# ---- the reference's own benchmark translation unit, unmodified, against this library ----
from oracle import oracle as _oracle  # noqa: E402  (the one place that knows where the reference tree lies: oracle/Makefile)
REF = os.environ.get("LUTGEMM_REFERENCE") or _oracle._makefile_default_ref()
REF_TU = os.path.join(REF, "tests", "opt", "fp16", "int3_col_wise_matmul_fp16.cu")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "ref_layer175b_test")


@pytest.mark.skipif(not (os.path.exists(NVCC) and os.path.exists(REF_TU)), reason="needs nvcc and the reference tree")
def test_reference_benchmark_tu_compiles_and_links_unchanged():
    """tests/opt/fp16/int3_col_wise_matmul_fp16.cu + tests/main.cc + tests/src/custom_random.cpp + the vendored gtest,
    compiled where they lie with -I include (this library's lutGEMM header) and linked with liblutgemm_b200.so and the
    cublas_gemm_ex definition of tests/cpp/ (the symbol the translation unit declares at :25-27)."""
    from lutgemm_b200 import _build
    _build.build()
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "-B", "ref_tu", "REF=" + REF])
    assert os.path.exists(REF_EXE)
    out = subprocess.run([REF_EXE, "--gtest_list_tests"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0 and "int3_col_wise_matmul_fp16" in out.stdout and "layer_175b" in out.stdout, out.stdout + out.stderr


@pytest.mark.gpu
def test_reference_benchmark_tu_runs_against_this_library():
    """TEST(int3_col_wise_matmul_fp16, layer_175b) (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:293-314): six
    instantiations at M = 1, N = 28672, K = 7168 (cuBLAS, the 3-bit uniform kernel and LUT-GEMM at 8 / 4 / 3 planes), whose
    host loops fill several GB with rand() first: minutes of CPU time.  The binary is built where the reference tree is
    (oracle/Makefile ref_tu) and travels with the repository."""
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/ref_layer175b_test was not built (no reference tree at build time)")
    out = subprocess.run([REF_EXE], capture_output=True, text=True, timeout=1500)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "[  PASSED  ] 1 test" in out.stdout
    assert out.stdout.count("latency min") == 8           # 3 in the warm-up instantiation + the 5 reported rows
