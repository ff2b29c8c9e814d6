"""q38b_gemv_f32_static: the matvec for hosts that cannot allocate device memory on the decode path (a runtime with
a fixed arena, code under stream capture).  Its Q8_K scratch is an array built into the library; results must equal
q38b_gemv_f32, which takes the scratch from the caller.  Collected last on purpose: a failure here leaves every other
test already run."""
import numpy as np
import pytest
import torch

from qwengine_b200 import api, formats as F, synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_caller_scratch_twice(ctx):
    f = F.IQ4_XS
    M, K = 520, 17408                      # the largest K of the model; 8 columns fill the built-in scratch exactly
    w = torch.from_numpy(synth.make_weights(f, M, K, seed=501)).cuda()
    assert ctx.lib.q38b_gemv_f32_static_capacity() == 8 * (K // 256) * 292
    for call, nb in enumerate((8, 3)):     # two calls in a row; the second leaves stale blocks of the first behind it
        x = torch.from_numpy(synth.make_activations(nb, K, seed=600 + call)).cuda()
        want = ctx.gemv_f32(f, w, x, K)
        got = torch.full((nb, M), float("nan"), device="cuda")
        ctx.gemv_f32_static(f, w, x, K, out=got)
        ctx.check()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # single column (the other kernel family) and another format
    f2 = F.Q4_K
    w2 = torch.from_numpy(synth.make_weights(f2, 300, 5120, seed=502)).cuda()
    x2 = torch.from_numpy(synth.make_activations(1, 5120, seed=503)).cuda()
    got2 = torch.empty((1, 300), device="cuda")
    ctx.gemv_f32_static(f2, w2, x2, 5120, out=got2)
    assert torch.equal(got2, ctx.gemv_f32(f2, w2, x2, 5120))


def test_static_scratch_rejects_oversize(ctx):
    f = F.Q8_0
    K = 17408 + 256                        # 8 columns of this K need more than the built-in 158,848 bytes
    w = torch.zeros((16, f.row_bytes(K)), dtype=torch.uint8, device="cuda")
    x = torch.zeros((8, K), device="cuda")
    y = torch.empty((8, 16), device="cuda")
    with pytest.raises(api.Q38BError) as e:
        ctx.gemv_f32_static(f, w, x, K, out=y)
    assert e.value.status == -6            # Q38B_ERR_NOMEM
    ctx.gemv_f32_static(f, w, x[:7], K, out=y[:7])   # 7 columns fit
    ctx.check()
