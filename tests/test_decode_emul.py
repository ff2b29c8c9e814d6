"""GPU-free check of the tensor-core fragment builders (qwengine_b200/csrc/q38b_decode.cuh): the header is
compiled for the host with 32 threads playing the lanes of a warp (tests/host_emul/emul_decode.cpp) and a 16-row
tile is compared with the oracle."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle
from qwengine_b200 import formats as F, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def emul(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("emul") / "libemul.so")
    src = os.path.join(ROOT, "tests", "host_emul", "emul_decode.cpp")
    subprocess.run(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-o", so, src, "-lpthread"], check=True)
    lib = C.CDLL(so)
    u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    lib.emul_tile.argtypes = [C.c_int, C.c_int, u8p, u8p, C.c_int, C.c_int, C.c_int, f32p]
    return lib


@pytest.mark.parametrize("name", list(F.FORMATS))
@pytest.mark.parametrize("nb,addr_lo,rep_log2", [(1, 0, 5), (7, 8, 3), (8, 2, 0)])
def test_tile_matches_oracle(emul, name, nb, addr_lo, rep_log2):
    f = F.get(name)
    if addr_lo % {"Q4_K": 16, "Q5_K": 16, "IQ4_XS": 8}.get(name, 2):
        addr_lo = 0   # the format's loads need this alignment (the C ABI rejects anything else)
    K = 768
    w = synth.make_weights(f, 16, K, seed=3, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = synth.make_activations(nb, K, seed=4) * (np.arange(nb, dtype=np.float32)[:, None] + 1)
    xq = oracle.port.quantize_q8k(x)
    y = np.zeros((16, 8), np.float32)
    assert emul.emul_tile(f.type_id, K, w.reshape(-1), xq.reshape(-1), nb, addr_lo, rep_log2, y.reshape(-1)) == 0
    for c in range(nb):
        ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[c], K)
        assert np.max(np.abs(y[:, c] - ref) / mag) < 1e-6
    assert not y[:, nb:].any()


@pytest.mark.parametrize("name", list(F.FORMATS) + list(F.ONE_COLUMN))
@pytest.mark.parametrize("K,addr_lo,rep_log2", [(1024, 0, 5), (1280, 8, 3), (2048, 2, 0)])
def test_single_column_granules_match_oracle(emul, name, K, addr_lo, rep_log2):
    """The dp4a granule decoders of the nb = 1 kernel (q38b_decode1.cuh), lane by lane on the host."""
    f = F.get(name)
    if addr_lo % {"Q4_K": 16, "Q5_K": 16, "IQ4_XS": 8, "Q2_K": 4}.get(name, 2):
        addr_lo = 0
    u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    emul.emul_gemv1.argtypes = [C.c_int, C.c_int, u8p, C.c_int, u8p, C.c_int, C.c_int, f32p]
    M = 6
    w = synth.make_weights(f, M, K, seed=13, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    xq = oracle.port.quantize_q8k(synth.make_activations(1, K, seed=14))
    y = np.zeros(M, np.float32)
    assert emul.emul_gemv1(f.type_id, K, w.reshape(-1), M, xq.reshape(-1), addr_lo, rep_log2, y) == 0
    ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
    assert np.max(np.abs(y - ref) / mag) < 1e-6


@pytest.mark.parametrize("K,row_pad,addr_lo", [(1024, 0, 0), (5120, 0, 8), (1280, 6, 0), (2304, 6, 8)])
def test_row_group_decoder_matches_oracle(emul, K, row_pad, addr_lo):
    """The eight-lanes-per-row IQ3_XXS decoder (GranR) with every field fetched by its widest aligned load: the host
    loaders abort on a misaligned access, so this also proves the alignment rules for 8-byte aligned rows."""
    f = F.get("IQ3_XXS")
    u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    emul.emul_gemv1_rowgroup.argtypes = [C.c_int, C.c_int, u8p, C.c_int, C.c_int, u8p, C.c_int, f32p]
    M = 9
    w = synth.make_weights(f, M, K, seed=23, scale=2e-4)
    rb = f.row_bytes(K) + row_pad
    assert rb % 8 == 0
    wpad = np.zeros((M, rb), np.uint8)
    wpad[:, :f.row_bytes(K)] = w
    xq = oracle.port.quantize_q8k(synth.make_activations(1, K, seed=24))
    y = np.zeros(M, np.float32)
    assert emul.emul_gemv1_rowgroup(f.type_id, K, wpad.reshape(-1), rb, M, xq.reshape(-1), addr_lo, y) == 0
    ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
    assert np.max(np.abs(y - ref) / mag) < 1e-6


@pytest.mark.parametrize("name", list(F.FORMATS) + list(F.ONE_COLUMN))
@pytest.mark.parametrize("K,addr_lo", [(1024, 0), (1280, 8)])
def test_single_column_granules_with_per32_activations(emul, name, K, addr_lo):
    """The same decoders fed with the reference GPU path's activation format (int8 values, one scale per 32): the
    result is the exact dot of the dequantized weights with d[k / 32] * q[k]."""
    f = F.get(name)
    if addr_lo % {"Q4_K": 16, "Q5_K": 16, "IQ4_XS": 8, "Q2_K": 4}.get(name, 2):
        addr_lo = 0
    u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    emul.emul_gemv1_act32.argtypes = [C.c_int, C.c_int, u8p, C.c_int, i8p, f32p, C.c_int, f32p]
    M = 5
    w = synth.make_weights(f, M, K, seed=33, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = synth.make_activations(1, K, seed=34) * np.linspace(0.1, 3.0, K, dtype=np.float32)   # scales differ from block to block
    q8, d32, _ = oracle.quantize_act_q8(x)
    y = np.zeros(M, np.float32)
    assert emul.emul_gemv1_act32(f.type_id, K, w.reshape(-1), M, q8.reshape(-1), d32.reshape(-1), addr_lo, y) == 0
    want, mag = oracle.port.matmul_ref(f.type_id, w, oracle.act_q8_dequant(q8, d32), K)
    assert np.max(np.abs(y - want[0]) / mag[0]) < 1e-6
