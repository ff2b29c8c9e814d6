"""The reference runtime's entry points (namespace q38rt::cuda) through include/q38rt_cuda_b200.hpp on a GPU: a probe
library written like engine.cpp's call sites (tests/shim/shim_probe.cpp) is compiled against the header and linked with
libq38b200.so; decode goes quantize_act_q8 -> gemv_q8 / gemv_q8n, prefill goes dequant_rows_f16 -> gemm_f16 in row
blocks through one fp16 scratch, as Engine::gemm_split does."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle
from qwengine_b200 import build, formats as F, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def probe(tmp_path_factory, ctx):
    lib = build.build()
    so = str(tmp_path_factory.mktemp("shim") / "libshim_probe.so")
    cuda = "/usr/local/cuda"
    subprocess.run(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", os.path.join(ROOT, "tests", "shim", "shim_probe.cpp"), "-o", so,
                    "-I", os.path.join(ROOT, "include"), "-I", cuda + "/include", lib, "-L", cuda + "/lib64", "-lcudart",
                    "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    p = C.CDLL(so)
    vp = C.c_void_p
    p.probe_decode.argtypes = [C.c_uint32, vp, C.c_size_t, C.c_int, C.c_int, vp, C.c_int, vp, vp, vp, vp]
    p.probe_prefill.argtypes = [C.c_uint32, vp, C.c_size_t, C.c_int, C.c_int, vp, vp, C.c_int, C.c_int, vp, C.c_int]
    return p


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ4_XS", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("nb", [1, 4])
def test_decode_call_sites(probe, name, nb):
    f = F.get(name)
    M, K = 520, 5120
    w = synth.make_weights(f, M, K, seed=61, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = synth.make_activations(nb, K, seed=62)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    q = torch.empty((nb, K), dtype=torch.int8, device="cuda")
    d = torch.empty((nb, K // 32), device="cuda")
    s = torch.empty_like(d)
    y = torch.empty((nb, M), device="cuda")
    assert probe.probe_decode(f.type_id, wd.data_ptr(), wd.stride(0), K, M, xd.data_ptr(), nb, q.data_ptr(), d.data_ptr(), s.data_ptr(),
                              y.data_ptr()) == 0
    torch.cuda.synchronize()
    oq, od, osum = oracle.quantize_act_q8(x)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy().view(np.uint32), osum.view(np.uint32))
    want, mag = oracle.port.matmul_ref(f.type_id, w, oracle.act_q8_dequant(oq, od), K)
    err = np.abs(y.cpu().numpy().astype(np.float64) - want) / np.where(mag == 0, 1, mag)
    assert err.max() < 1e-3      # the bound of the path; the kernels stay below 2e-6 (tests/test_gpu_act_q8.py)


def test_unsupported_format_returns_false(probe):
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert probe.probe_decode(11, t.data_ptr(), 110, 256, 1, t.data_ptr(), 1, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr()) == 1   # Q3_K: no kernel


@pytest.mark.parametrize("name", ["IQ3_XXS", "Q4_K"])
def test_prefill_call_site(probe, name):
    f = F.get(name)
    M, K, B = 700, 5120, 130
    w = synth.make_weights(f, M, K, seed=63, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    wd = torch.from_numpy(w).cuda()
    x = torch.randn((B, K), device="cuda", dtype=torch.float16)
    scratch = torch.zeros(((M + 1) // 2, K), device="cuda", dtype=torch.float16)
    y = torch.empty((B, M), device="cuda")
    assert probe.probe_prefill(f.type_id, wd.data_ptr(), wd.stride(0), K, M, scratch.data_ptr(), x.data_ptr(), K, B, y.data_ptr(), M) == 0
    torch.cuda.synchronize()
    want, mag = oracle.port.matmul_ref(f.type_id, w, x.float().cpu().numpy(), K)
    err = np.abs(y.cpu().numpy().astype(np.float64) - want) / np.where(mag == 0, 1, mag)
    assert err.max() < 1e-2
