"""Prefill GEMM (tcgen05, weights dequantized on the fly to bf16) against the fp32/double oracle.

Tolerance: |Y - exact| <= 1e-2 * sum_k |w x| per output (the bound set for the bf16 path; the only rounding besides
fp32 accumulation is one bf16 rounding per weight, 2^-9 relative)."""
import numpy as np
import pytest
import torch

import oracle
from qwengine_b200 import formats as F, synth

pytestmark = pytest.mark.gpu
TOL = 1e-2


def check(ctx, name, M, K, B, accumulate=False):
    f = F.get(name)
    w = synth.make_weights(f, M, K, seed=400 + M + B, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = torch.randn((B, K), generator=torch.Generator().manual_seed(B)).to(torch.bfloat16)
    wd, xd = torch.from_numpy(w).cuda(), x.cuda()
    if accumulate:
        y = torch.full((B, M), 2.0, dtype=torch.float32, device="cuda")
        ctx.gemm_prefill(f, wd, xd, K, out=y, accumulate=True)
        y = y - 2.0
    else:
        y = ctx.gemm_prefill(f, wd, xd, K)
    ctx.check()
    want, mag = oracle.port.matmul_ref(f.type_id, w, x.float().numpy(), K)
    err = np.abs(y.cpu().numpy().astype(np.float64) - want) / np.where(mag == 0, 1, mag)
    assert err.max() < TOL, (name, M, K, B, err.max())
    return err.max()


@pytest.mark.parametrize("name", list(F.FORMATS))
def test_prefill_small_all_formats(ctx, name):
    check(ctx, name, 128, 512, 64)


@pytest.mark.parametrize("M,K,B", [(128, 256, 1), (200, 1024, 300), (384, 2048, 256), (130, 768, 700), (256, 5120, 1024)])
def test_prefill_shapes(ctx, M, K, B):
    check(ctx, "IQ3_XXS", M, K, B)
    check(ctx, "Q4_K", M, K, B)


@pytest.mark.parametrize("name", ["IQ3_XXS", "Q4_K"])
@pytest.mark.parametrize("M,K", [(17408, 5120), (5120, 17408)])
def test_prefill_full_size_1024_tokens(ctx, name, M, K):
    """The prefill chunk at its stated size: 1024 tokens against the 17408 x 5120 up projection and the 5120 x 17408
    down projection.  All tokens of 192 sampled rows (first and last row tiles, and rows spread over the rest) are held
    to the bound against the double-precision oracle; the remaining rows are checked for finiteness and, through a
    second run on a row-permuted copy of the weights, for the same bits wherever a row lands."""
    f = F.get(name)
    B = 1024
    w = synth.make_weights(f, M, K, seed=500 + M, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    x = torch.randn((B, K), generator=torch.Generator().manual_seed(K)).to(torch.bfloat16)
    wd, xd = torch.from_numpy(w).cuda(), x.cuda()
    y = ctx.gemm_prefill(f, wd, xd, K)
    ctx.check()
    assert bool(torch.isfinite(y).all())
    rng = np.random.default_rng(M + K)
    rows = np.unique(np.concatenate([np.arange(64), np.arange(M - 64, M), rng.choice(M, 64, replace=False)]))
    want, mag = oracle.port.matmul_ref(f.type_id, np.ascontiguousarray(w[rows]), x.float().numpy(), K)
    got = y[:, torch.from_numpy(rows).cuda()].cpu().numpy().astype(np.float64)
    err = np.abs(got - want) / np.where(mag == 0, 1, mag)
    assert err.max() < TOL, (name, M, K, err.max())
    perm = torch.from_numpy(rng.permutation(M)).cuda()
    y2 = ctx.gemm_prefill(f, wd[perm].contiguous(), xd, K)
    ctx.check()
    assert torch.equal(y2.view(torch.int32), y[:, perm].view(torch.int32))


def test_prefill_accumulate_and_stride(ctx):
    check(ctx, "Q6_K", 128, 512, 40, accumulate=True)


@pytest.mark.parametrize("name,bound", [("IQ3_XXS", 1e-5), ("IQ4_XS", 1e-5), ("Q4_K", 4e-3), ("Q5_K", 4e-3), ("Q6_K", 4e-3)])
def test_prefill_equals_bf16_reference_gemm(ctx, name, bound):
    """Against torch: bf16(exactly dequantized weights) x bf16 activations with fp32 accumulation.  For the codebook
    formats the kernel multiplies the same operands, so only the summation order differs.  The K-quants take the packed
    bf16 dequantizer, which rounds scale and minimum to bf16 before the multiplication instead of the product after
    it: each weight may differ from bf16(exact) by 2^-8 of its magnitude."""
    from qwengine_b200 import api
    f = F.get(name)
    M, K, B = 512, 5120, 512
    w = torch.from_numpy(synth.make_weights(f, M, K, seed=77)).cuda()
    x = torch.randn((B, K), device="cuda", dtype=torch.bfloat16)
    y = ctx.gemm_prefill(f, w, x, K)
    wb = ctx.dequant_rows(f, w, K, api.OUT_BF16)
    ref = (x.float() @ wb.float().t())
    mag = (x.float().abs() @ wb.float().abs().t())
    assert float(((y - ref).abs() / mag).max()) < bound


@pytest.mark.parametrize("name,bound", [("Q8_0", 1e-5), ("IQ3_XXS", 1e-5), ("IQ3_S", 1e-5), ("IQ4_XS", 1e-5), ("Q4_K", 1e-3), ("Q5_K", 1e-3), ("Q6_K", 1e-3)])
def test_prefill_fp16_operands_equal_the_reference_path(ctx, name, bound):
    """fp16 operands: what the reference's prefill path multiplies (dequant_rows_f16 + gemm_f16, src/cuda/prefill.cu:
    802-851).  Against torch on the fp16 dequantized weights (q38b_dequant_rows, bit-exact to dequant_rows_f16's
    arithmetic) with fp32 accumulation: the same operands for the codebook formats and Q8_0 (only the summation order
    differs); the K-quants round scale and minimum to fp16 before the multiplication (2^-11 per weight).  And against
    the double-precision oracle at the path's 1e-2 bound."""
    from qwengine_b200 import api
    f = F.get(name)
    M, K, B = 384, 5120, 300
    wn = synth.make_weights(f, M, K, seed=91, scale=2e-4 if name == "IQ3_XXS" else 1e-3)
    w = torch.from_numpy(wn).cuda()
    x = torch.randn((B, K), device="cuda", dtype=torch.float16)
    y = ctx.gemm_prefill(f, w, x, K)
    ctx.check()
    wh = ctx.dequant_rows(f, w, K, api.OUT_F16)
    ref = x.float() @ wh.float().t()
    mag = x.float().abs() @ wh.float().abs().t()
    assert float(((y - ref).abs() / mag).max()) < bound
    want, omag = oracle.port.matmul_ref(f.type_id, wn, x.float().cpu().numpy(), K)
    err = np.abs(y.cpu().numpy().astype(np.float64) - want) / np.where(omag == 0, 1, omag)
    assert err.max() < TOL
