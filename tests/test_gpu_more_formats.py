"""The reference's other six matvec formats (IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S, IQ1_M, Q2_K) on the GPU: exact dequantizer,
one-column matvec (and several columns, run one after the other), per-32 activations, grouped launches and the prefill
GEMM, against the CPU oracle, which is bit-identical to the compiled reference for these formats (tests/test_oracle.py)."""
import numpy as np
import pytest
import torch

import oracle
import qwengine_b200 as q
from qwengine_b200 import api, formats as F, synth

pytestmark = pytest.mark.gpu
NAMES = list(F.ONE_COLUMN)
REL_TOL = 2e-6


@pytest.mark.parametrize("name", NAMES)
def test_dequant_rows_bit_exact(ctx, name):
    f = F.get(name)
    w = synth.make_weights(f, 33, 1280, seed=3 + f.type_id)
    wd = torch.from_numpy(w).cuda()
    want = oracle.port.dequantize(f.type_id, w)
    got = ctx.dequant_rows(f, wd, 1280, api.OUT_F32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    h = ctx.dequant_rows(f, wd, 1280, api.OUT_F16).cpu().numpy()
    assert np.array_equal(h.view(np.uint16), want.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("M,K", [(1, 256), (33, 768), (1000, 5120), (40, 17408), (17408, 5120)])
def test_gemv_against_oracle(ctx, name, M, K):
    f = F.get(name)
    w = synth.make_weights(f, M, K, seed=100 + M)
    x = synth.make_activations(7, K, seed=200 + K) * (np.arange(7, dtype=np.float32)[:, None] + 1)
    xq = oracle.port.quantize_q8k(x)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(xq).cuda()
    refs = [oracle.port.row_ref_mag(f.type_id, w, xq[c], K) for c in range(7)]
    singles = None
    for nb in (1, 3, 7) if M < 10000 else (1,):
        y = ctx.gemv(f, wd, xd[:nb], K)
        yn = y.cpu().numpy()
        for c in range(nb):
            ref, mag = refs[c]
            assert np.max(np.abs(yn[c] - ref) / np.where(mag == 0, 1.0, mag)) < REL_TOL, (name, M, K, nb, c)
        if nb == 7:
            singles = y
    if singles is not None:      # columns of a wider call are the one-column results (src/cuda/gemv.cuh:31-34)
        for c in (0, 6):
            one = ctx.gemv(f, wd, xd[c:c + 1], K)
            assert torch.equal(one[0].view(torch.int32), singles[c].view(torch.int32))
    # close to the reference's own AVX2 results too (another summation order of the same integers)
    cpu = oracle.port.gemv(f.type_id, w, xq[:1], K)
    _, mag = refs[0]
    assert np.max(np.abs(ctx.gemv(f, wd, xd[:1], K).cpu().numpy()[0] - cpu[0]) / np.where(mag == 0, 1.0, mag)) < 1e-5
    ctx.check()


@pytest.mark.parametrize("name", NAMES)
def test_act_q8_and_groups(ctx, name):
    f = F.get(name)
    K = 5120
    Ms = [700, 9, 2051]
    ws = [synth.make_weights(f, M, K, seed=40 + i) for i, M in enumerate(Ms)]
    wds = [torch.from_numpy(w).cuda() for w in ws]
    x = synth.make_activations(2, K, seed=8)
    xd = torch.from_numpy(x).cuda()
    # per-32 activations (the reference GPU path's format)
    q8, d32, _ = oracle.quantize_act_q8(x)
    want, mag = oracle.port.matmul_ref(f.type_id, ws[0], oracle.act_q8_dequant(q8, d32), K)
    y = ctx.gemv_act_q8(f, wds[0], torch.from_numpy(q8).cuda(), torch.from_numpy(d32).cuda(), K)
    assert (np.abs(y.cpu().numpy() - want) / np.where(mag == 0, 1, mag)).max() < REL_TOL
    # three matrices on one column in one launch, from floats: the bits of quantize + one call per matrix
    xq = ctx.quantize_q8k(xd[:1])
    want1 = [ctx.gemv(f, w, xq, K)[0] for w in wds]
    got = ctx.gemv_group(f, wds, K, x_f32=xd[0])
    for a, b in zip(got, want1):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    ctx.check()


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill(ctx, name, dtype):
    f = F.get(name)
    M, K, B = 200, 1024, 300
    w = synth.make_weights(f, M, K, seed=400 + f.type_id)
    x = torch.randn((B, K), generator=torch.Generator().manual_seed(B)).to(dtype)
    y = ctx.gemm_prefill(f, torch.from_numpy(w).cuda(), x.cuda(), K)
    ctx.check()
    want, mag = oracle.port.matmul_ref(f.type_id, w, x.float().numpy(), K)
    err = np.abs(y.cpu().numpy().astype(np.float64) - want) / np.where(mag == 0, 1, mag)
    assert err.max() < 1e-2


def test_recorded_pass_with_the_other_formats(ctx):
    """A recorded pass over all six formats for 1 and 3 columns equals the direct calls bit for bit."""
    K = 1024
    ps = q.Pass(ctx, max_nb=3)
    xin, xq = ps.buffer_f32(K), ps.buffer_q8k(K)
    ps.quantize(xin, 0, K, xq)
    items = []
    for i, name in enumerate(NAMES):
        w = synth.make_weights(name, 100 + 8 * i, K, seed=70 + i)
        yb = ps.buffer_f32(100 + 8 * i)
        ps.gemv(ps.matrix_upload(name, w, K), xq, yb, 0)
        items.append((name, w, yb))
    x = torch.from_numpy(synth.make_activations(3, K, seed=5)).cuda()
    for nb in (1, 3):
        ps.buffer_tensor(xin)[:nb].copy_(x[:nb])
        ps.run(nb)
        torch.cuda.synchronize()
        xqd = ctx.quantize_q8k(x[:nb])
        for name, w, yb in items:
            want = ctx.gemv(name, torch.from_numpy(w).cuda(), xqd, K)
            assert torch.equal(ps.buffer_tensor(yb)[:nb].view(torch.int32), want.view(torch.int32)), (name, nb)
    ctx.check()
    ps.close()
