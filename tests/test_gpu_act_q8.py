"""The reference GPU path's activation format (ActQ8: int8 values, one scale per 32) through the C ABI: the quantizer
bit for bit against its numpy restatement (oracle.quantize_act_q8), the matvec against the double-precision dot of the
exactly dequantized weights with d[k / 32] * q[k]."""
import numpy as np
import pytest
import torch

import oracle
from qwengine_b200 import formats as F, synth

pytestmark = pytest.mark.gpu
REL_TOL = 2e-6   # of sum |w x| per row (the reference's own bound for its GPU kernels, tests/kernels/test_gemv.cu:101)


def test_act_q8_quantizer_bit_exact(ctx):
    x = synth.make_activations(5, 5120, seed=41) * np.logspace(-4, 4, 5, dtype=np.float32)[:, None]
    x[1, 64:96] = 0.0                      # an all-zero block stays zero
    x[2, 32:64] = 1e-30
    x[3, 7] = -5.0
    q, d, s = ctx.quantize_act_q8(torch.from_numpy(x).cuda())
    wq, wd, ws = oracle.quantize_act_q8(x)
    assert np.array_equal(q.cpu().numpy(), wq)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), wd.view(np.uint32))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))


@pytest.mark.parametrize("name", list(F.FORMATS))
@pytest.mark.parametrize("M,K", [(333, 5120), (64, 17408), (17, 256), (1000, 1280)])
def test_gemv_act_q8_against_oracle(ctx, name, M, K):
    f = F.get(name)
    w = synth.make_weights(f, M, K, seed=900 + M, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = synth.make_activations(7, K, seed=901) * np.linspace(0.2, 4.0, K, dtype=np.float32)
    q, d, _ = oracle.quantize_act_q8(x)
    want, mag = oracle.port.matmul_ref(f.type_id, w, oracle.act_q8_dequant(q, d), K)
    wd, qd, dd = torch.from_numpy(w).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(d).cuda()
    singles = []
    for nb in (1, 3, 7):
        y = ctx.gemv_act_q8(f, wd, qd[:nb], dd[:nb], K)
        err = np.abs(y.cpu().numpy().astype(np.float64) - want[:nb]) / np.where(mag[:nb] == 0, 1, mag[:nb])
        assert err.max() < REL_TOL, (name, M, K, nb, err.max())
        singles.append(y)
    # every column is the single-column result (src/cuda/gemv.cuh:31-34)
    for c in range(7):
        one = ctx.gemv_act_q8(f, wd, qd[c:c + 1], dd[c:c + 1], K)
        assert torch.equal(one[0].view(torch.int32), singles[2][c].view(torch.int32))
    ctx.check()


def test_gemv_act_q8_accumulate_and_strides(ctx):
    f = F.Q4_K
    M, K = 100, 1024
    w = torch.from_numpy(synth.make_weights(f, M, K, seed=77)).cuda()
    x = torch.from_numpy(synth.make_activations(2, K, seed=78)).cuda()
    q, d, _ = ctx.quantize_act_q8(x)
    base = ctx.gemv_act_q8(f, w, q, d, K)
    out = torch.full((2, M + 5), 3.0, device="cuda")
    ctx.gemv_act_q8(f, w, q, d, K, out=out[:, :M], accumulate=True)
    assert torch.equal(out[:, M:], torch.full((2, 5), 3.0, device="cuda"))
    assert torch.allclose(out[:, :M] - 3.0, base, rtol=0, atol=1e-5)
    ctx.check()
