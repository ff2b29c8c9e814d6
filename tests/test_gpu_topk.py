"""Top-k of the head's logits (q38b_topk, the pass step q38b_pass_op_topk) against the oracle's ordering: values
descending, equal values by ascending position.  Sizes and k follow the reference's test (tests/kernels/test_ops.cu:425-447
of the reference project: n = 248320, 100000, 4096, 1000; k = 1, 20, 32; positions offset by 1000), plus ties, NaN,
infinities, several rows, k = 64 and k > n."""
import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import qwengine_b200 as q   # noqa: E402


@pytest.fixture(scope="module")
def ctx():
    c = q.Context(0)
    yield c
    c.close()


def check(ctx, x, k, off=0):
    vals, idx = ctx.topk(torch.from_numpy(x).cuda(), k, off)
    ctx.check()
    want_v, want_i = oracle.topk(x, k, off)
    assert np.array_equal(idx.cpu().numpy(), want_i)
    assert np.array_equal(vals.cpu().numpy().view(np.uint32), want_v.view(np.uint32))


@pytest.mark.parametrize("n", [248320, 100000, 4096, 1000])
@pytest.mark.parametrize("k", [1, 20, 32, 64])
def test_topk_sizes_of_the_reference_test(ctx, n, k):
    rng = np.random.default_rng(n + k)
    check(ctx, (rng.standard_normal((1, n)) * 4).astype(np.float32), k, 1000)


def test_topk_ties_go_to_the_lower_position(ctx):
    rng = np.random.default_rng(3)
    x = rng.integers(-3, 4, size=(2, 50000)).astype(np.float32)   # seven distinct values: nothing but ties
    check(ctx, x, 64)
    check(ctx, np.zeros((1, 5000), np.float32), 40)
    check(ctx, np.where(rng.random((1, 3000)) < 0.5, np.float32(0.0), np.float32(-0.0)).astype(np.float32), 10)


def test_topk_special_values_and_short_vectors(ctx):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((3, 70001)) * 10).astype(np.float32)
    x[0, [5, 40000, 70000]] = np.inf
    x[0, [6, 7]] = -np.inf
    x[1, ::3] = np.nan
    x[2, :] = np.nan
    x[2, 123] = -np.inf
    check(ctx, x, 33)
    check(ctx, rng.standard_normal((1, 10)).astype(np.float32), 64)      # k > n: the rest is (NaN, -1)
    check(ctx, rng.standard_normal((8, 1025)).astype(np.float32), 5)


def test_topk_as_a_step_of_the_recorded_pass(ctx):
    """A head matvec followed by the top-k step: the run returns 2 k words per column instead of all logits."""
    from qwengine_b200 import formats as F, synth
    K, V, k = 1024, 5000, 16
    w = synth.make_weights("Q6_K", V, K, seed=77)
    x = synth.make_activations(3, K, seed=78)
    ps = q.Pass(ctx, max_nb=3)
    xin, xq, logits, best = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(V), ps.buffer_f32(2 * k)
    ps.quantize(xin, 0, K, xq)
    ps.gemv(ps.matrix_upload("Q6_K", w, K), xq, logits, 0)
    ps.topk(logits, 0, V, k, best)
    for nb in (1, 3):
        y = np.empty((nb, 2 * k), np.float32)
        ps.run_host(nb, xin, x[:nb], best, 0, y)
        ctx.check()
        full = ps.buffer_tensor(logits)[:nb].cpu().numpy()
        want_v, want_i = oracle.topk(full, k)
        assert np.array_equal(y[:, k:].view(np.int32), want_i)
        assert np.array_equal(y[:, :k].view(np.uint32), want_v.view(np.uint32))
        ref = oracle.port.gemv(F.Q6_K.type_id, w, oracle.port.quantize_q8k(x[:nb]), K)
        assert np.array_equal(want_i[:, 0], np.argmax(ref, axis=1).astype(np.int32)) or np.allclose(full, ref, rtol=0, atol=1e-4 * np.abs(ref).max())
    ps.close()
