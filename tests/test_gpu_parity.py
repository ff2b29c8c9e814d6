"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the committed reference vectors.

Tolerances: integer / byte outputs bit-exact; matvec rows within 2e-6 of the exact sum relative to sum|w*x|
(the reference's own GPU bound, tests/kernels/test_gemv.cu:101), far inside the 1e-3 the path is required to meet."""
import numpy as np
import pytest
import torch

import oracle
from qwengine_b200 import api, formats as F, synth

pytestmark = pytest.mark.gpu
ALL = list(F.FORMATS)
REL_TOL = 2e-6
HARD_BAR = 1e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def scale_for(name):
    return 2e-4 if name == "IQ3_XXS" else 1e-3


def rel_err(y, w, xq, f, K):
    """max over rows and columns of |y - exact| / sum|w*x| (y: [nb, M])."""
    worst = 0.0
    for c in range(xq.shape[0]):
        ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[c], K)
        mag = np.where(mag == 0, 1.0, mag)
        worst = max(worst, float(np.max(np.abs(y[c] - ref) / mag)))
    return worst


# ---------------------------------------------------------------------------------------------
def test_q8k_quantizer_bit_exact(ctx, golden):
    for key in ("x", "x_edge"):
        out = ctx.quantize_q8k(dev(golden[key])).cpu().numpy()
        assert np.array_equal(out, golden["xq" if key == "x" else "xq_edge"])
    x = synth.make_activations(7, 17408, seed=11) * np.float32(3.0)
    assert np.array_equal(ctx.quantize_q8k(dev(x)).cpu().numpy(), oracle.port.quantize_q8k(x))
    ctx.check()


def test_q8k_quantizer_strided_input(ctx):
    x = synth.make_activations(3, 1024, seed=12)
    big = torch.zeros((3, 1536), dtype=torch.float32, device="cuda")
    big[:, :1024] = dev(x)
    out = ctx.quantize_q8k(big[:, :1024]).cpu().numpy()
    assert np.array_equal(out, oracle.port.quantize_q8k(x))


@pytest.mark.parametrize("name", ALL)
def test_dequant_bit_exact(ctx, golden, name):
    f = F.get(name)
    w = golden[f"w_{name}"]
    K = golden["x"].shape[1]
    got = ctx.dequant_rows(f, dev(w), K, api.OUT_F32).cpu().numpy()
    assert np.array_equal(bits(got), bits(golden[f"dq_{name}"]))
    w2 = synth.make_weights(f, 37, 1280, seed=50 + f.type_id, scale=scale_for(name))
    want = oracle.port.dequantize(f.type_id, w2)
    got = ctx.dequant_rows(f, dev(w2), 1280, api.OUT_F32).cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    h = ctx.dequant_rows(f, dev(w2), 1280, api.OUT_F16).cpu().numpy()
    assert np.array_equal(h.view(np.uint16), want.astype(np.float16).view(np.uint16))
    b = ctx.dequant_rows(f, dev(w2), 1280, api.OUT_BF16).cpu()
    assert torch.equal(b, torch.from_numpy(want).to(torch.bfloat16))


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ3_S", "IQ4_XS", "Q4_K", "Q6_K"])
def test_gemv_matches_reference_vectors(ctx, golden, name):
    """Against the outputs of the reference's AVX2 kernels on the same blocks and Q8_K activations."""
    f = F.get(name)
    w, xq = golden[f"w_{name}"], golden["xq"]
    K = golden["x"].shape[1]
    for nb in (1, 2, 3):
        y = ctx.gemv(f, dev(w), dev(xq[:nb]), K).cpu().numpy()
        ref_y = golden[f"y{nb}_{name}"]
        for c in range(nb):
            _, mag = oracle.port.row_ref_mag(f.type_id, w, xq[c], K)
            assert np.max(np.abs(y[c] - ref_y[c]) / mag) < REL_TOL
    ctx.check()


SHAPES = [(1, 256), (15, 512), (33, 768), (257, 2048), (1024, 5120), (48, 6144), (40, 17408)]


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("M,K", SHAPES)
def test_gemv_against_oracle(ctx, name, M, K):
    f = F.get(name)
    w = synth.make_weights(f, M, K, seed=100 + M, scale=scale_for(name))
    x = synth.make_activations(8, K, seed=200 + K) * (np.arange(8, dtype=np.float32)[:, None] + 1)
    xq = oracle.port.quantize_q8k(x)
    wd, xd = dev(w), dev(xq)
    for nb in (1, 2, 4, 7, 8):
        y = ctx.gemv(f, wd, xd[:nb], K).cpu().numpy()
        err = rel_err(y, w, xq[:nb], f, K)
        assert err < REL_TOL, (name, M, K, nb, err)
        assert err < HARD_BAR
    ctx.check()


@pytest.mark.parametrize("M,K,pad", [(1000, 5120, 0), (37, 1024, 0), (64, 1280, 6), (300, 17408, 0), (129, 2304, 22)])
def test_row_group_mapping_against_lane_per_granule(ctx, M, K, pad):
    """IQ3_XXS rows that are a multiple of 8 bytes apart take the row-group mapping of the one-column kernel (eight
    lanes per row, widest aligned loads); both mappings form the same exact integer sums, so they agree with the oracle
    and with each other to float rounding.  Rows padded to a multiple of 8 bytes (K not a multiple of 1024) and ragged
    row counts included."""
    f = F.IQ3_XXS
    w = synth.make_weights(f, M, K, seed=700 + M, scale=scale_for("IQ3_XXS"))
    rb = f.row_bytes(K) + pad
    assert rb % 8 == 0
    wp = np.zeros((M, rb), np.uint8)
    wp[:, :f.row_bytes(K)] = w
    xq = oracle.port.quantize_q8k(synth.make_activations(1, K, seed=701))
    wd, xd = dev(wp), dev(xq)
    y_rg = ctx.gemv(f, wd, xd, K).cpu().numpy()
    ctx.debug_set_rowgroup(False)
    try:
        y_lane = ctx.gemv(f, wd, xd, K).cpu().numpy()
    finally:
        ctx.debug_set_rowgroup(True)
    ctx.check()
    ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
    mag = np.where(mag == 0, 1.0, mag)
    assert np.max(np.abs(y_rg[0] - ref) / mag) < REL_TOL
    assert np.max(np.abs(y_lane[0] - ref) / mag) < REL_TOL
    assert np.max(np.abs(y_rg[0] - y_lane[0]) / mag) < REL_TOL


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("M,K", [(5120, 1024), (2999, 1024), (8 * 296 + 8 * 40 + 3, 512), (700, 5120), (5120, 17408)])
def test_one_and_two_ctas_per_sm_give_the_same_bits(ctx, name, M, K):
    """The one-column kernel exists for two CTAs per SM (eight consumer warps each) and for one (sixteen warps, larger
    tiles for the row-group mapping); a row's arithmetic does not depend on the tile it sits in or the warp that takes
    it, so both give the same bits.  (Compared with the row-group mapping off: which shapes it takes differs between the
    two variants, and it sums a row in another order than the lane-per-granule mapping.)"""
    f = F.get(name)
    w = dev(synth.make_weights(f, M, K, seed=800 + M % 97, scale=scale_for(name)))
    xq = dev(oracle.port.quantize_q8k(synth.make_activations(1, K, seed=801)))
    ys = {}
    try:
        for rg in (False, True):
            ctx.debug_set_rowgroup(rg)
            for mode in (0, 2):
                ctx.debug_set_one_cta(mode)
                ys[rg, mode] = ctx.gemv(f, w, xq, K)
    finally:
        ctx.debug_set_one_cta(1)
        ctx.debug_set_rowgroup(True)
    ctx.check()
    assert torch.equal(ys[False, 0].view(torch.int32), ys[False, 2].view(torch.int32))
    scale = float(ys[False, 0].abs().max())
    for mode in (0, 2):
        assert float((ys[True, mode] - ys[False, 0]).abs().max()) <= 1e-5 * scale


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("M", [6144, 12288])
def test_verify_sweep_row_counts(ctx, name, M):
    """The speculative-verify sweep's middle row counts (M = 6144 and 12288 at K = 5120; 1024 and 17408 are covered by
    the shape list above and the full-size test) for 1, 2, 4 and 7 columns, every row against the oracle."""
    f = F.get(name)
    K = 5120
    w = synth.make_weights(f, M, K, seed=600 + M, scale=scale_for(name))
    x = synth.make_activations(7, K, seed=601) * (np.arange(7, dtype=np.float32)[:, None] + 1)
    xq = oracle.port.quantize_q8k(x)
    wd, xd = dev(w), dev(xq)
    refs = [oracle.port.row_ref_mag(f.type_id, w, xq[c], K) for c in range(7)]
    for nb in (1, 2, 4, 7):
        y = ctx.gemv(f, wd, xd[:nb], K).cpu().numpy()
        for c in range(nb):
            ref, mag = refs[c]
            err = float(np.max(np.abs(y[c] - ref) / np.where(mag == 0, 1.0, mag)))
            assert err < REL_TOL, (name, M, nb, c, err)
    ctx.check()


@pytest.mark.parametrize("name", ALL)
def test_columns_bit_identical_to_single_column(ctx, name):
    """gemv_q8n's promise (src/cuda/gemv.cuh:31-34): every column equals the one-column call.  Holds across all nb
    with the uniform-columns option (nb = 1 then runs the tensor-core kernel too); without it the dedicated nb = 1
    kernel sums in another order and agrees to rounding, while columns of nb >= 2 calls never depend on nb."""
    f = F.get(name)
    M, K = 200, 5120
    wn = synth.make_weights(f, M, K, seed=7, scale=scale_for(name))
    w = dev(wn)
    xqn = oracle.port.quantize_q8k(synth.make_activations(8, K, seed=8))
    xq = dev(xqn)
    ctx.set_uniform_columns(True)
    try:
        singles = [ctx.gemv(f, w, xq[c:c + 1], K)[0] for c in range(8)]
    finally:
        ctx.set_uniform_columns(False)
    for nb in (2, 3, 5, 7, 8):
        y = ctx.gemv(f, w, xq[:nb], K)
        for c in range(nb):
            assert torch.equal(y[c].view(torch.int32), singles[c].view(torch.int32)), (name, nb, c)
    fast = ctx.gemv(f, w, xq[:1], K)[0].cpu().numpy()
    _, mag = oracle.port.row_ref_mag(f.type_id, wn, xqn[0], K)
    assert np.max(np.abs(fast - singles[0].cpu().numpy()) / mag) < REL_TOL


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ3_S", "IQ4_XS", "Q4_K", "Q5_K", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("M,K", [(1, 8448), (37, 17408), (531, 8448), (531, 17408)])
def test_long_rows_in_k_parts(ctx, name, M, K):
    """Rows longer than 8192 on the multi-column kernel: the row is cut into K-parts that different CTAs compute and the
    last one adds up.  The sums match the oracle, do not depend on the column count, the row count of the call or on
    which launch it is, and accumulate / strided outputs work as for short rows."""
    f = F.get(name)
    wn = synth.make_weights(f, M, K, seed=131, scale=scale_for(name))
    w = dev(wn)
    xqn = oracle.port.quantize_q8k(synth.make_activations(8, K, seed=132))
    xq = dev(xqn)
    y8 = ctx.gemv(f, w, xq, K)
    assert rel_err(y8.cpu().numpy(), wn, xqn, f, K) < REL_TOL
    for nb in (2, 7):
        y = ctx.gemv(f, w, xq[:nb], K)
        assert torch.equal(y.view(torch.int32), y8[:nb].view(torch.int32)), (name, nb)
        assert torch.equal(ctx.gemv(f, w, xq[:nb], K), y)          # the tile counters are back at zero
    if M > 100:
        cut = 16 * 9 + 5                                            # shards that do not end on a tile boundary
        top = ctx.gemv(f, dev(wn[:cut]), xq[:7], K)
        rest = ctx.gemv(f, dev(wn[cut:]), xq[:7], K)
        assert torch.equal(torch.cat([top, rest], dim=1), y8[:7])
    buf = torch.full((3, M + 12), 2.0, dtype=torch.float32, device="cuda")
    ctx.gemv(f, w, xq[:3], K, out=buf[:, :M], accumulate=True)
    assert torch.equal(buf[:, :M], y8[:3] + 2.0)
    assert torch.all(buf[:, M:] == 2.0)
    if M > 100:
        # a matrix with more (tile, part) sums than the scratch area holds runs as one launch per block of rows
        ctx.debug_set_gemv_part_items(64)
        try:
            assert torch.equal(ctx.gemv(f, w, xq[:7], K), y8[:7])
        finally:
            ctx.debug_set_gemv_part_items(0)
    ctx.check()


@pytest.mark.parametrize("name", ["IQ3_XXS", "Q4_K", "Q6_K", "Q8_0"])
def test_accumulate_and_output_stride(ctx, name):
    f = F.get(name)
    M, K, nb = 100, 1024, 3
    w = dev(synth.make_weights(f, M, K, seed=17, scale=scale_for(name)))
    xq = dev(oracle.port.quantize_q8k(synth.make_activations(nb, K, seed=18)))
    y = ctx.gemv(f, w, xq, K)
    buf = torch.full((nb, M + 28), 3.0, dtype=torch.float32, device="cuda")   # y_ld > M, canary beyond M
    view = buf[:, :M]
    ctx.gemv(f, w, xq, K, out=view, accumulate=True)
    assert torch.equal(view, y + 3.0)
    assert torch.all(buf[:, M:] == 3.0)


@pytest.mark.parametrize("name", ["IQ3_XXS", "IQ3_S", "Q6_K", "Q8_0", "IQ4_XS", "Q4_K"])
def test_row_stride_and_shards(ctx, name):
    """Rows `row_bytes` apart (a column-split or padded layout) and row shards give the same rows bit for bit."""
    f = F.get(name)
    M, K = 96, 1024
    rb = f.row_bytes(K)
    pad = 48 if rb % 16 == 0 else 40      # keeps the format's alignment (16 for the K-quants, 8 for the 2-byte formats)
    w = synth.make_weights(f, M, K, seed=27, scale=scale_for(name))
    xq = dev(oracle.port.quantize_q8k(synth.make_activations(2, K, seed=28)))
    full = ctx.gemv(f, dev(w), xq, K)
    wide = torch.zeros((M, rb + pad), dtype=torch.uint8, device="cuda")
    wide[:, :rb] = dev(w)
    assert torch.equal(ctx.gemv(f, wide[:, :rb], xq, K), full)
    for shards in (2, 4, 8):
        rows = M // shards
        parts = [ctx.gemv(f, dev(w[i * rows:(i + 1) * rows]), xq, K) for i in range(shards)]
        assert torch.equal(torch.cat(parts, dim=1), full)


@pytest.mark.parametrize("name", ["IQ3_XXS", "Q4_K", "IQ4_XS", "Q8_0"])
def test_gemv_from_fp32_activations(ctx, name):
    """q38b_gemv_f32 = quantize into caller scratch + matvec: the same bits as the two calls made separately."""
    f = F.get(name)
    M, K = 300, 2048
    w = dev(synth.make_weights(f, M, K, seed=91, scale=scale_for(name)))
    for nb in (1, 4):
        x = dev(synth.make_activations(nb, K, seed=92 + nb))
        y = ctx.gemv_f32(f, w, x, K)
        assert torch.equal(y, ctx.gemv(f, w, ctx.quantize_q8k(x), K))
    small = torch.empty(100, dtype=torch.uint8, device="cuda")
    with pytest.raises(api.Q38BError):
        ctx.gemv_f32(f, w, x, K, scratch=small)
    ctx.check()


def test_argument_errors(ctx):
    f = F.IQ3_XXS
    K, M = 512, 16
    w = dev(synth.make_weights(f, M, K, seed=1))
    xq = dev(oracle.port.quantize_q8k(synth.make_activations(1, K, seed=2)))
    y = torch.zeros((8, M), dtype=torch.float32, device="cuda")
    rb = f.row_bytes(K)
    call = lambda **kw: ctx.gemv_raw(**{**dict(type_id=18, W_ptr=w.data_ptr(), row_bytes=rb, K=K, M=M, xq_ptr=xq.data_ptr(),
                                               x_stride=K // 256, nb=1, y_ptr=y.data_ptr(), y_ld=M), **kw})
    assert call() == 0
    assert call(type_id=11) == -2          # Q3_K: no kernel here
    assert call(nb=9) == -1 and call(nb=0) == -1
    assert call(K=500) == -1
    assert call(W_ptr=w.data_ptr() + 2) == -3
    assert call(row_bytes=rb - 2) == -1
    assert call(y_ld=M - 1) == -1
    ctx.check()


# ---------------------------------------------------------------------------------------------
# Full benchmark sizes
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_full_size_gemv(ctx, name):
    """17408 x 5120 (the single-matvec configuration): all rows against the oracle, plus exact properties."""
    f = F.get(name)
    M, K = 17408, 5120
    w = synth.make_weights(f, M, K, seed=4242, scale=scale_for(name))
    x = synth.make_activations(7, K, seed=4243)
    xq = oracle.port.quantize_q8k(x)
    wd, xd = dev(w), dev(xq)
    y1 = ctx.gemv(f, wd, xd[:1], K)
    y7 = ctx.gemv(f, wd, xd, K)
    ctx.check()
    ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
    bad = np.where(np.abs(y1[0].cpu().numpy() - ref) / mag >= REL_TOL)[0]
    assert bad.size == 0, (bad.size, bad[:32])
    y_cpu = oracle.port.gemv(f.type_id, w, xq[:1], K)[0]
    assert np.max(np.abs(y1[0].cpu().numpy() - y_cpu) / mag) < REL_TOL
    assert np.max(np.abs(y7[0].cpu().numpy() - ref) / mag) < REL_TOL
    ctx.set_uniform_columns(True)
    try:
        assert torch.equal(y7[0].view(torch.int32), ctx.gemv(f, wd, xd[:1], K)[0].view(torch.int32))
    finally:
        ctx.set_uniform_columns(False)
    # row permutation commutes with the matvec, bit for bit
    perm = torch.randperm(M, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    assert torch.equal(ctx.gemv(f, wd[perm].contiguous(), xd[:1], K)[0], y1[0][perm])
    # zero activations give exact zeros
    z = ctx.quantize_q8k(torch.zeros((1, K), dtype=torch.float32, device="cuda"))
    assert not ctx.gemv(f, wd, z, K).any()


def test_swiglu_and_requantisation(ctx):
    n = 17408
    g = synth.make_activations(2, n, seed=61) * np.float32(2.0)
    u = synth.make_activations(2, n, seed=62)
    h, q = ctx.swiglu_q8k(dev(g), dev(u))
    h = h.cpu().numpy()
    want = oracle.port.swiglu(g, u).reshape(2, n)
    assert np.max(np.abs(h - want)) <= 1e-6 * np.max(np.abs(want))      # expf differs in the last bit at most
    # the blocks are exactly the Q8_K quantisation of the h this kernel produced
    assert np.array_equal(q.cpu().numpy(), oracle.port.quantize_q8k(h))


def test_ffn_block_full_size(ctx):
    """gate, up 17408 x 5120 in Q4_K, SwiGLU, down 5120 x 17408 in Q6_K, one token."""
    H, FF = 5120, 17408
    gate = synth.make_weights(F.Q4_K, FF, H, seed=71)
    up = synth.make_weights(F.Q4_K, FF, H, seed=72)
    down = synth.make_weights(F.Q6_K, H, FF, seed=73)
    x = synth.make_activations(1, H, seed=74)
    xq = ctx.quantize_q8k(dev(x))
    g = ctx.gemv(F.Q4_K, dev(gate), xq, H)
    u = ctx.gemv(F.Q4_K, dev(up), xq, H)
    _, hq = ctx.swiglu_q8k(g, u, want_h=False)
    y = ctx.gemv(F.Q6_K, dev(down), hq, FF)[0].cpu().numpy()
    ctx.check()
    # oracle chain
    xq_o = oracle.port.quantize_q8k(x)
    g_o = oracle.port.gemv(F.Q4_K.type_id, gate, xq_o, H)
    u_o = oracle.port.gemv(F.Q4_K.type_id, up, xq_o, H)
    hq_o = oracle.port.quantize_q8k(oracle.port.swiglu(g_o, u_o).reshape(1, FF))
    y_o = oracle.port.gemv(F.Q6_K.type_id, down, hq_o, FF)[0]
    _, mag = oracle.port.row_ref_mag(F.Q6_K.type_id, down, hq_o[0], FF)
    assert np.max(np.abs(y - y_o) / mag) < HARD_BAR


def test_one_column_kernels_are_resident_as_planned(ctx):
    """Every one-column launch plans its shared memory for two CTAs per SM (or one, for the 16-warp variant); a launch
    whose CTA turned out too large (for instance by static shared memory the plan did not count) would silently run at
    half the occupancy."""
    ctx.lib.q38b_debug_occupancy_shortfalls(ctx.h, 1)
    try:
        for name in ALL:
            f = F.get(name)
            for M, K in [(64, 256), (128, 1024), (512, 5120), (64, 6144), (40, 17408)]:
                w = dev(synth.make_weights(f, M, K, seed=1))
                xq = dev(oracle.port.quantize_q8k(synth.make_activations(1, K, seed=2)))
                for mode in (0, 2):
                    ctx.debug_set_one_cta(mode)
                    ctx.gemv(f, w, xq, K)
        ctx.check()
    finally:
        ctx.debug_set_one_cta(1)
        n = ctx.lib.q38b_debug_occupancy_shortfalls(ctx.h, 0)
    assert n == 0
