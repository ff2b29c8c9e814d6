"""The CPU oracle (oracle/oracle_port.c) against the reference: its compiled sources (oracle/_ref, when
built), the committed vectors generated from them, and gguf-py's independent dequantizers."""
import numpy as np
import pytest

import oracle
from qwengine_b200 import formats as F, synth

ALL = list(F.FORMATS)
WITH_REF_DOT = ["IQ3_XXS", "IQ3_S", "IQ4_XS", "Q4_K", "Q6_K"]   # get_vec_dot returns nullptr for Q5_K and Q8_0
EXTRA = list(F.ONE_COLUMN)                                      # the reference's other six matvec formats


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("name", ALL)
def test_dequant_matches_golden(golden, name):
    f = F.get(name)
    dq = oracle.port.dequantize(f.type_id, golden[f"w_{name}"])
    assert np.array_equal(bits(dq), bits(golden[f"dq_{name}"]))


@pytest.mark.parametrize("name", WITH_REF_DOT)
def test_dot_matches_golden_bitwise(golden, name):
    f = F.get(name)
    K = golden["x"].shape[1]
    for nb in (1, 2, 3):
        y = oracle.port.gemv(f.type_id, golden[f"w_{name}"], golden["xq"][:nb], K)
        assert np.array_equal(bits(y), bits(golden[f"y{nb}_{name}"]))


def test_q8k_matches_golden(golden):
    assert np.array_equal(oracle.port.quantize_q8k(golden["x"]), golden["xq"])
    assert np.array_equal(oracle.port.quantize_q8k(golden["x_edge"]), golden["xq_edge"])
    # all-zero row -> all-zero blocks
    zero_row = np.where(~golden["x_edge"].any(axis=1))[0][0]
    assert not golden["xq_edge"][zero_row].any()


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (no reference checkout)")
@pytest.mark.parametrize("name", ALL)
def test_port_equals_compiled_reference(name):
    f = F.get(name)
    K = 1024
    w = synth.make_weights(f, 40, K, seed=5 + f.type_id, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    if name != "Q5_K":
        assert np.array_equal(bits(oracle.port.dequantize(f.type_id, w)), bits(oracle.ref.dequantize(f.type_id, w, K)))
    x = synth.make_activations(8, K, seed=9) * (np.arange(8, dtype=np.float32)[:, None] + 1)
    xq = oracle.port.quantize_q8k(x)
    assert np.array_equal(xq, oracle.ref.quantize_q8k(x))
    assert np.array_equal(xq, oracle.ref.quantize_q8k(x, avx2=True))
    if name in WITH_REF_DOT:
        assert oracle.ref.has_vec_dot(f.type_id)
        for nb in (1, 4, 7, 8):
            y_ref, _ = oracle.ref.gemv(f.type_id, w, xq[:nb], K, threads=2)
            assert np.array_equal(bits(oracle.port.gemv(f.type_id, w, xq[:nb], K)), bits(y_ref))
    else:
        assert not oracle.ref.has_vec_dot(f.type_id)


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (no reference checkout)")
@pytest.mark.parametrize("name", EXTRA)
def test_port_equals_compiled_reference_other_formats(name):
    """IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S, IQ1_M and Q2_K: dequantized values and dot products of the restatement are the bits of
    the reference's own quant_ref.cpp / cpu_kernels.cpp."""
    f = F.get(name)
    K = 1024
    w = synth.make_weights(f, 40, K, seed=5 + f.type_id, scale=1e-3)
    assert np.array_equal(bits(oracle.port.dequantize(f.type_id, w)), bits(oracle.ref.dequantize(f.type_id, w, K)))
    xq = oracle.port.quantize_q8k(synth.make_activations(8, K, seed=9) * (np.arange(8, dtype=np.float32)[:, None] + 1))
    assert oracle.ref.has_vec_dot(f.type_id)
    for nb in (1, 4, 7, 8):
        y_ref, _ = oracle.ref.gemv(f.type_id, w, xq[:nb], K, threads=2)
        assert np.array_equal(bits(oracle.port.gemv(f.type_id, w, xq[:nb], K)), bits(y_ref))


@pytest.mark.parametrize("name", ALL + EXTRA)
def test_dequant_matches_gguf_py(name):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    f = F.get(name)
    w = synth.make_weights(f, 16, 512, seed=21 + f.type_id)
    ours = oracle.port.dequantize(f.type_id, w)
    theirs = quants.dequantize(w, getattr(gguf.GGMLQuantizationType, name)).astype(np.float32)
    assert np.array_equal(bits(ours), bits(theirs))


@pytest.mark.parametrize("name", ALL)
def test_dot_close_to_exact_sum(name):
    """The reference tests' own metric (tests/kernels/test_cpu_gemv.cpp:100-125): |y - exact| / sum|w*x| < 1e-6."""
    f = F.get(name)
    K = 2048
    w = synth.make_weights(f, 64, K, seed=31)
    xq = oracle.port.quantize_q8k(synth.make_activations(1, K, seed=32))
    y = oracle.port.gemv(f.type_id, w, xq, K)[0]
    ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
    assert np.max(np.abs(y - ref) / mag) < 1e-6


def test_columns_bit_identical_to_single_column():
    f = F.get("Q6_K")
    K = 512
    w = synth.make_weights(f, 8, K, seed=41)
    xq = oracle.port.quantize_q8k(synth.make_activations(8, K, seed=42))
    y8 = oracle.port.gemv(f.type_id, w, xq, K)
    for c in range(8):
        assert np.array_equal(bits(y8[c]), bits(oracle.port.gemv(f.type_id, w, xq[c:c + 1], K)[0]))


def test_fp16_conversion_exhaustive():
    lib = oracle.port.lib
    h = np.arange(65536, dtype=np.uint16)
    ours = np.array([lib.q38o_fp16_to_fp32(int(v)) for v in h], np.float32)
    theirs = h.view(np.float16).astype(np.float32)
    ok = np.isnan(theirs) | (bits(ours) == bits(theirs))
    assert ok.all()
    finite = np.isfinite(theirs)
    back = np.array([lib.q38o_fp32_to_fp16(float(v)) for v in theirs[finite]], np.uint16)
    assert np.array_equal(back, h[finite])


def test_topk_order():
    """oracle.topk: values descending, equal values by ascending position, NaN last, (NaN, -1) past the end."""
    x = np.array([[1.0, 5.0, 5.0, np.nan, -np.inf, 0.0, -0.0, 7.0]], np.float32)
    v, i = oracle.topk(x, 10, index_offset=100)
    assert i[0].tolist() == [107, 101, 102, 100, 105, 106, 104, 103, -1, -1]
    assert v[0, 0] == 7.0 and np.isnan(v[0, 7]) and np.isnan(v[0, 9])
