"""include/q38rt_cuda_b200.hpp compiles as one translation unit: against the reference's own declarations when the
reference checkout is present (its signatures must match definition for definition), and standalone."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("Q38RT_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
CUDA_INC = "/usr/local/cuda/include"


def _compile(extra, tmp_path):
    src = os.path.join(ROOT, "tests", "shim", "shim_probe.cpp")
    obj = str(tmp_path / "probe.o")
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-Wno-unused-function", "-c", src, "-o", obj, "-I", os.path.join(ROOT, "include"), "-I", CUDA_INC] + extra
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    syms = subprocess.run(["nm", "-C", "--defined-only", obj], capture_output=True, text=True).stdout
    for name in ("q38rt::cuda::gemv_q8n(", "q38rt::cuda::gemv_q8(", "q38rt::cuda::quantize_act_q8(", "q38rt::cuda::gemv_q8_supported(",
                 "q38rt::cuda::dequant_rows_f16(", "q38rt::cuda::gemm_f16(", "q38rt::cuda::cublas_create(", "q38rt::cuda::cublas_bind(",
                 "q38rt::cuda::cublas_destroy("):
        assert any(name in l and " T " in l for l in syms.splitlines()), f"{name} is not defined with external linkage"


@pytest.mark.skipif(not os.path.isdir(CUDA_INC), reason="CUDA headers not installed")
def test_shim_compiles_standalone(tmp_path):
    _compile([], tmp_path)


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "src", "cuda", "gemv.cuh")), reason="reference checkout not present")
def test_shim_matches_the_reference_declarations(tmp_path):
    """With the reference's include path the header takes ActQ8, QuantFormat and the function declarations from
    src/cuda/gemv.cuh; a definition whose signature differed from its declaration would be an overload, and the calls in
    the probe (written like engine.cpp's) would not find the defaults or would be ambiguous."""
    _compile(["-I", os.path.join(REF, "src"), "-I", os.path.join(REF, "include"), "-DQ38RT_B200_EXPECT_REFERENCE"], tmp_path)
