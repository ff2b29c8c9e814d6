"""The two dense helpers that complete a layer's linear algebra: the bf16 matvec of the small per-layer projections and
the prefill SwiGLU written in place as 16-bit floats."""
import numpy as np
import pytest
import torch

from qwengine_b200 import api

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(48, 5120), (1, 8), (7, 17408)])
def test_gemv_bf16(ctx, N, K):
    g = torch.Generator(device="cuda").manual_seed(N)
    W = torch.randn((N, K), device="cuda", generator=g).to(torch.bfloat16)
    x = torch.randn(K, device="cuda", generator=g)
    y = ctx.gemv_bf16(W, x)
    ref = W.double() @ x.double()
    mag = W.double().abs() @ x.double().abs()
    assert float(((y.double() - ref).abs() / mag).max()) < 1e-5      # fp32 accumulation against the exact dot
    ctx.check()


@pytest.mark.parametrize("kind,dtype", [(api.OUT_F16, torch.float16), (api.OUT_BF16, torch.bfloat16)])
@pytest.mark.parametrize("B,n,ld", [(5, 17408, 17408), (3, 256, 300), (2, 8, 8)])
def test_swiglu_rows_inplace(ctx, kind, dtype, B, n, ld):
    g = torch.Generator(device="cuda").manual_seed(n)
    G = torch.randn((B, ld), device="cuda", generator=g) * 3
    U = torch.randn((B, ld), device="cuda", generator=g)
    want = (G[:, :n].double() / (1 + torch.exp(-G[:, :n].double())) * U[:, :n].double())
    tail = G[:, n:].clone()
    ctx.swiglu_rows_inplace(G, U, n, kind)
    torch.cuda.synchronize()
    got = G.view(dtype)[:, :n]                  # the 16-bit matrix the next GEMM reads: row stride 2 ld
    eps = 2.0 ** (-11 if dtype == torch.float16 else -8)
    # one rounding to the 16-bit type (plus the fast exponential's few fp32 ulps; fp16 results below 6e-5 are subnormal)
    assert bool(((got.double() - want).abs() <= 1.1 * eps * want.abs() + 1e-7).all())
    assert torch.equal(G[:, n:], tail)          # the halves end at float n / 2: the rest of the row is untouched
    ctx.check()


@pytest.mark.parametrize("rows,n,with_a,with_b", [(1, 5120, True, False), (7, 5120, True, True), (3, 256, False, False), (2, 8192, True, False)])
def test_add_rmsnorm_q8k(ctx, rows, n, with_a, with_b):
    """Residual add + RMSNorm + Q8_K in one kernel: the residual stream is the exact float sum, the normed row agrees with
    the double-precision formula, and the Q8_K blocks are exactly the quantizer's output on that normed row."""
    import oracle
    g = torch.Generator(device="cuda").manual_seed(rows * n)
    x = torch.randn((rows, n), device="cuda", generator=g) * 2
    a = torch.randn((rows, n), device="cuda", generator=g) if with_a else None
    b = torch.randn((rows, n), device="cuda", generator=g) if with_b else None
    w = torch.rand(n, device="cuda", generator=g) + 0.5
    want_x = x.clone()
    if with_a:
        want_x = want_x + a
    if with_b:
        want_x = want_x + b
    eps = 1e-6
    xn, q8 = ctx.add_rmsnorm_q8k(x, w, a, b, eps)
    torch.cuda.synchronize()
    assert torch.equal(x, want_x)                                  # float adds in the reference's order: x + a, then + b
    xd = want_x.double()
    ref = xd * torch.rsqrt((xd * xd).mean(dim=1, keepdim=True) + eps) * w.double()
    assert float(((xn.double() - ref).abs() / ref.abs().clamp_min(1e-3)).max()) < 1e-5
    assert np.array_equal(q8.cpu().numpy(), oracle.port.quantize_q8k(xn.cpu().numpy()))
    ctx.check()
