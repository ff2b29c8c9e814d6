"""The planner's recorded pass (C++ q38b_pass, CUDA-graph replay) against the CPU oracle chain."""
import numpy as np
import pytest
import torch

import oracle
import qwengine_b200 as q
from qwengine_b200 import decode_pass as dp, formats as F, synth

pytestmark = pytest.mark.gpu


def small_weights(n_layers, head_rows):
    ws = {}
    for i, s in enumerate(dp.all_specs(n_layers, head=False)):
        ws[s.name] = synth.make_weights(s.fmt, s.M, s.K, seed=300 + i, scale=dp.UNIT_GAIN_SCALE[s.fmt], zero_mean=True)
    return ws


@pytest.mark.parametrize("nb", [1, 3])
def test_pass_replay_equals_step_by_step_calls(ctx, nb):
    """The recorded pass (CUDA graph, programmatic dependent launch) gives the bits of the same steps called one by one,
    and stays close to the CPU oracle chain.  Two chains of re-quantised matvecs can only be compared loosely end to
    end: a last-bit difference in one fp32 output flips an int8 rounding of the next Q8_K block, which moves later
    outputs by about one quantisation step; every single step is held to 2e-6 / bit-exactness in test_gpu_parity.py."""
    n_layers = 4   # three DeltaNet-shaped layers and one attention-shaped layer
    ws = small_weights(n_layers, 0)
    ps = q.Pass(ctx, max_nb=nb)
    io = dp.build(ps, lambda spec, rows: ps.matrix_upload(spec.fmt, ws[spec.name], spec.K), n_layers=n_layers, head=False)
    x = synth.make_activations(nb, dp.HIDDEN, seed=5)
    y = np.empty((nb, dp.HIDDEN), np.float32)
    ps.run_host(nb, io["in_buf"], x, io["out_buf"], 0, y)
    ctx.check()
    # the same chain with individual calls on the default stream
    wd = {k: torch.from_numpy(v).cuda() for k, v in ws.items()}
    xe = torch.from_numpy(x).cuda()
    for il in range(n_layers):
        attn, mats = dp.layer_specs(il)
        big = ctx.gemv(mats[0].fmt, wd[mats[0].name], ctx.quantize_q8k(xe), dp.HIDDEN)
        proj = mats[3] if attn else mats[1]
        xe = ctx.gemv(proj.fmt, wd[proj.name], ctx.quantize_q8k(big[:, :dp.INNER]), dp.INNER)
        xq = ctx.quantize_q8k(xe)
        g = ctx.gemv(mats[-3].fmt, wd[mats[-3].name], xq, dp.HIDDEN)
        u = ctx.gemv(mats[-2].fmt, wd[mats[-2].name], xq, dp.HIDDEN)
        _, hq = ctx.swiglu_q8k(g, u, want_h=False)
        ffn = ctx.gemv(mats[-1].fmt, wd[mats[-1].name], hq, dp.FF)
        if il == n_layers - 1:
            xe = ffn
    assert np.array_equal(y.view(np.uint32), xe.cpu().numpy().view(np.uint32))
    # replaying the graph gives the same bits
    y2 = np.empty_like(y)
    ps.run_host(nb, io["in_buf"], x, io["out_buf"], 0, y2)
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))
    want = dp.oracle_forward(oracle.port, ws, x, n_layers, head=False)
    assert np.linalg.norm(y - want) < 0.15 * np.linalg.norm(want)
    assert ps.weight_bytes == dp.total_weight_bytes(n_layers, head=False)
    ps.close()


def test_upload_shards_cover_all_rows(ctx):
    """Row shards uploaded by the planner reproduce the unsharded matvec bit for bit."""
    f = F.IQ3_XXS
    M, K = 64, 1024
    w = synth.make_weights(f, M, K, seed=9)
    x = synth.make_activations(1, K, seed=10)
    full = ctx.gemv(f, torch.from_numpy(w).cuda(), ctx.quantize_q8k(torch.from_numpy(x).cuda()), K).cpu().numpy()
    for shards in (2, 4, 8):
        out = np.zeros((1, M), np.float32)
        for g in range(shards):
            ps = q.Pass(ctx, max_nb=1)
            xin, xq, yb = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(M)
            mid = ps.matrix_upload(f, w, K, shard=g, n_shards=shards)
            ps.quantize(xin, 0, K, xq)
            ps.gemv(mid, xq, yb, g * (M // shards))
            y = np.empty((1, M), np.float32)
            ps.run_host(1, xin, x, yb, 0, y)
            rows = slice(g * (M // shards), (g + 1) * (M // shards))
            out[0, rows] = y[0, rows]
            ps.close()
        assert np.array_equal(out.view(np.uint32), full.view(np.uint32))


def _mixed_cases(ctx, cases):
    ps = q.Pass(ctx, max_nb=1)
    xin, xq = ps.buffer_f32(5120), ps.buffer_q8k(5120)
    xin2, xq2 = ps.buffer_f32(17408), ps.buffer_q8k(17408)
    ps.quantize(xin, 0, 5120, xq)
    ps.quantize(xin2, 0, 17408, xq2)
    ybufs, wts = [], []
    for i, (fmt, M, K) in enumerate(cases):
        w = synth.make_weights(fmt, M, K, seed=900 + i)
        wts.append(w)
        yb = ps.buffer_f32(M)
        ybufs.append(yb)
        ps.gemv(ps.matrix_upload(fmt, w, K), xq if K == 5120 else xq2, yb, 0)
    x1 = torch.from_numpy(synth.make_activations(1, 5120, seed=3)).cuda()
    x2 = torch.from_numpy(synth.make_activations(1, 17408, seed=4)).cuda()
    ps.buffer_tensor(xin).copy_(x1)
    ps.buffer_tensor(xin2).copy_(x2)
    ps.run(1)
    torch.cuda.synchronize()
    ctx.check()
    q1, q2 = ctx.quantize_q8k(x1), ctx.quantize_q8k(x2)
    for (fmt, M, K), w, yb in zip(cases, wts, ybufs):
        want = ctx.gemv(fmt, torch.from_numpy(w).cuda(), q1 if K == 5120 else q2, K)
        got = ps.buffer_tensor(yb)
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (fmt, M, K)
    ps.close()


def test_recorded_pass_all_formats(ctx):
    """One quantize step feeding matvecs of every format (ragged row counts) as a recorded pass, against the same
    matvecs called one by one."""
    _mixed_cases(ctx, [("IQ3_XXS", 1000, 5120), ("IQ3_S", 333, 5120), ("IQ4_XS", 1024, 5120), ("Q4_K", 2051, 5120),
                       ("Q5_K", 515, 5120), ("Q6_K", 777, 5120), ("Q8_0", 130, 5120), ("Q4_K", 7, 5120)])


def test_recorded_pass_long_rows(ctx):
    """Rows too long for eight- or four-row tiles take two-row tiles; mixed with short rows and a second input vector."""
    _mixed_cases(ctx, [("IQ3_XXS", 1000, 5120), ("IQ4_XS", 517, 17408), ("Q4_K", 2051, 5120), ("IQ3_XXS", 64, 17408),
                       ("Q4_K", 100, 17408), ("Q5_K", 33, 17408), ("Q6_K", 777, 5120), ("Q8_0", 130, 5120)])


@pytest.mark.parametrize("fmt", ["IQ3_XXS", "IQ4_XS", "Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_gemv_group_equals_separate_calls(ctx, fmt):
    """Three matrices on one column in one launch, from Q8_K blocks and from floats (quantized inside the kernel), give
    the bits of quantize + one matvec call per matrix."""
    K = 5120
    Ms = [1000, 7, 2051]
    ws = [torch.from_numpy(synth.make_weights(fmt, M, K, seed=40 + i)).cuda() for i, M in enumerate(Ms)]
    x = torch.from_numpy(synth.make_activations(1, K, seed=8)).cuda()
    xq = ctx.quantize_q8k(x)
    want = [ctx.gemv(fmt, w, xq, K)[0] for w in ws]
    for kwargs in (dict(xq=xq), dict(x_f32=x)):
        got = ctx.gemv_group(fmt, ws, K, **kwargs)
        torch.cuda.synchronize()
        ctx.check()
        for g, w_ in zip(got, want):
            assert torch.equal(g.view(torch.int32), w_.view(torch.int32)), (fmt, list(kwargs))
    # a zero column quantizes to all-zero blocks
    got = ctx.gemv_group(fmt, ws[:2], K, x_f32=torch.zeros(K, device="cuda"))
    assert all(float(g.abs().max()) == 0.0 for g in got)


@pytest.mark.parametrize("fmt", ["IQ4_XS", "IQ3_XXS", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("nb", [2, 7])
def test_long_rows_merged_launches_equal_single_ones(ctx, fmt, nb):
    """Rows of 17408 on several columns (the K-part path of the multi-column kernel): three matrices behind one quantize
    step, merged into one launch with the quantize folded in, give the bits of one kernel per step; replays agree."""
    K = 17408
    Ms = [200, 7, 531]
    ws = [synth.make_weights(fmt, M, K, seed=70 + i, scale=dp.UNIT_GAIN_SCALE.get(fmt, 1e-4), zero_mean=True) for i, M in enumerate(Ms)]
    x = synth.make_activations(nb, K, seed=9)
    outs = []
    for merge in (True, False):
        ps = q.Pass(ctx, max_nb=nb)
        ps.set_merge(merge)
        src, xq, dst = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(1024)
        ps.quantize(src, 0, K, xq)
        off = 0
        for M, w in zip(Ms, ws):
            ps.gemv(ps.matrix_upload(fmt, w, K), xq, dst, off)
            off += M
        y = np.empty((nb, off), np.float32)
        for _ in range(2):
            ps.run_host(nb, src, x, dst, 0, y)
            ctx.check()
            outs.append(y.copy())
        ps.close()
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint32), outs[0].view(np.uint32))
    assert np.all(np.isfinite(outs[0])) and float(np.abs(outs[0]).max()) > 0


def test_merged_replay_equals_one_kernel_per_step(ctx):
    """Shared launches and folded quantize steps change nothing in the results, and fewer kernels run."""
    n_layers = 4
    ws = small_weights(n_layers, 0)
    x = synth.make_activations(1, dp.HIDDEN, seed=12)
    outs, counts = [], []
    for merge in (True, False):
        ps = q.Pass(ctx, max_nb=1)
        ps.set_merge(merge)
        io = dp.build(ps, lambda spec, rows: ps.matrix_upload(spec.fmt, ws[spec.name], spec.K), n_layers=n_layers, head=False)
        y = np.empty((1, dp.HIDDEN), np.float32)
        ps.run_host(1, io["in_buf"], x, io["out_buf"], 0, y)
        ctx.check()
        outs.append(y.copy())
        counts.append(ps.kernel_count)
        ps.close()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert counts[0] < counts[1]


@pytest.mark.parametrize("seed,nb", [(0, 1), (1, 1), (2, 1), (3, 1), (4, 3), (5, 7)])
def test_random_passes_merge_invariant(ctx, seed, nb):
    """Random recorded passes (mixed formats, matvecs sharing and not sharing a column, quantize steps whose output is
    or is not read again later, SwiGLU, outputs at offsets) give the same bits with and without merged launches."""
    rng = np.random.default_rng(seed)
    fmts = ["IQ3_XXS", "IQ4_XS", "Q4_K", "Q6_K", "IQ3_S", "Q8_0", "Q5_K"]
    K = 1024
    n_mats = 10
    mats = [(fmts[int(rng.integers(len(fmts)))], int(rng.choice([256, 264, 512, 1000]))) for _ in range(n_mats)]
    ws = [synth.make_weights(f, M, K, seed=1000 + 17 * seed + i, scale=dp.UNIT_GAIN_SCALE.get(f, 1e-4), zero_mean=True) for i, (f, M) in enumerate(mats)]
    # a fixed program of steps drawn once, replayed on two passes
    steps = []
    for _ in range(14):
        kind = rng.choice(["quant", "gemv", "gemv", "gemv", "swiglu"])
        if kind == "quant":
            steps.append(("quant", int(rng.integers(2)), int(rng.integers(2))))                  # source buffer, Q8_K buffer
        elif kind == "gemv":
            steps.append(("gemv", int(rng.integers(n_mats)), int(rng.integers(2)), int(rng.integers(3)), int(rng.choice([0, 8, 1024]))))
        else:
            steps.append(("swiglu", int(rng.integers(3)), int(rng.integers(3)), int(rng.integers(2))))
    x = synth.make_activations(nb, K, seed=50 + seed)
    results = []
    for merge in (True, False):
        ps = q.Pass(ctx, max_nb=nb)
        ps.set_merge(merge)
        src = [ps.buffer_f32(K), ps.buffer_f32(K)]
        qb = [ps.buffer_q8k(K), ps.buffer_q8k(K)]
        outs = [ps.buffer_f32(2048 + 1024) for _ in range(3)]
        mids = [ps.matrix_upload(f, w, K) for (f, _), w in zip(mats, ws)]
        ps.quantize(src[0], 0, K, qb[0])
        ps.quantize(src[1], 0, K, qb[1])
        for st in steps:
            if st[0] == "quant":
                ps.quantize(src[st[1]], 0, K, qb[st[2]])
            elif st[0] == "gemv":
                ps.gemv(mids[st[1]], qb[st[2]], outs[st[3]], st[4])
            else:
                ps.swiglu(outs[st[1]], 0, outs[st[2]], 1024, K, qb[st[3]])
        for b in src:
            ps.buffer_tensor(b).copy_(torch.from_numpy(x).cuda())
        for _ in range(2):
            ps.run(nb)
        torch.cuda.synchronize()
        ctx.check()
        results.append([ps.buffer_tensor(o).cpu().numpy().copy() for o in outs])
        ps.close()
    for a, b in zip(*results):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_recorded_graph_follows_later_changes(ctx):
    """A pass that has already been replayed picks up steps appended afterwards and context options switched afterwards
    (the recorded graph is captured again when what it was captured with has changed)."""
    f, K, M = F.IQ3_XXS, 1024, 96
    w1 = synth.make_weights(f, M, K, seed=71)
    w2 = synth.make_weights(f, M, K, seed=72)
    x = torch.from_numpy(synth.make_activations(1, K, seed=73)).cuda()
    ps = q.Pass(ctx, max_nb=1)
    xin, xq, y1, y2 = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(M), ps.buffer_f32(M)
    ps.quantize(xin, 0, K, xq)
    ps.gemv(ps.matrix_upload(f, w1, K), xq, y1, 0)
    ps.buffer_tensor(xin).copy_(x)
    ps.run(1)
    torch.cuda.synchronize()
    assert not ps.buffer_tensor(y2).any()
    ps.gemv(ps.matrix_upload(f, w2, K), xq, y2, 0)      # appended after the first replay
    ps.run(1)
    torch.cuda.synchronize()
    xq_t = ctx.quantize_q8k(x)
    want2 = ctx.gemv(f, torch.from_numpy(w2).cuda(), xq_t, K)
    assert torch.equal(ps.buffer_tensor(y2).view(torch.int32), want2.view(torch.int32))
    # a context option that picks another kernel: the replay must now give the bits of that kernel
    ctx.set_uniform_columns(True)
    try:
        ps.run(1)
        torch.cuda.synchronize()
        want_u = ctx.gemv(f, torch.from_numpy(w1).cuda(), xq_t, K)
        assert torch.equal(ps.buffer_tensor(y1).view(torch.int32), want_u.view(torch.int32))
    finally:
        ctx.set_uniform_columns(False)
    ctx.check()
    ps.close()


def test_pass_from_gguf_file(ctx, tmp_path):
    """Weights read from a GGUF file (written here with gguf-py) and row-sharded by the planner give the bits of the same
    bytes uploaded directly."""
    gguf = pytest.importorskip("gguf")
    f, M, K = F.IQ4_XS, 64, 1024
    w = synth.make_weights(f, M, K, seed=90)
    path = str(tmp_path / "one.gguf")
    wr = gguf.GGUFWriter(path, "qwen35")
    wr.add_tensor("blk.0.ffn_down.weight", w, raw_shape=w.shape, raw_dtype=gguf.GGMLQuantizationType(f.type_id))
    wr.write_header_to_file(); wr.write_kv_data_to_file(); wr.write_tensors_to_file(); wr.close()
    x = synth.make_activations(1, K, seed=91)
    want = ctx.gemv(f, torch.from_numpy(w).cuda(), ctx.quantize_q8k(torch.from_numpy(x).cuda()), K).cpu().numpy()
    g = q.GgufFile(path)
    out = np.zeros((1, M), np.float32)
    for shard in range(2):
        ps = q.Pass(ctx, max_nb=1)
        xin, xq, yb = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(M)
        ps.quantize(xin, 0, K, xq)
        ps.gemv(ps.matrix_from_gguf(g, "blk.0.ffn_down.weight", shard, 2), xq, yb, shard * (M // 2))
        y = np.empty((1, M), np.float32)
        ps.run_host(1, xin, x, yb, 0, y)
        out[0, shard * (M // 2):(shard + 1) * (M // 2)] = y[0, shard * (M // 2):(shard + 1) * (M // 2)]
        ps.close()
    g.close()
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    with pytest.raises(KeyError):
        g2 = q.GgufFile(path)
        try:
            q.Pass(ctx).matrix_from_gguf(g2, "missing")
        finally:
            g2.close()


def test_local_matvec_step_equals_the_plain_one(ctx):
    """q38b_pass_op_gemv_local (a matrix every rank holds whole: no peer stores) is the plain matvec step on one GPU, and
    local and pushed steps on one column still share nothing they should not: same bits, merged or not."""
    K, M = 1024, 520
    w = [synth.make_weights("Q4_K", M, K, seed=90 + i) for i in range(3)]
    x = synth.make_activations(1, K, seed=93)
    outs = []
    for local in (False, True):
        for merge in (True, False):
            ps = q.Pass(ctx, max_nb=1)
            ps.set_merge(merge)
            xin, xq, y = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(3 * M)
            ps.quantize(xin, 0, K, xq)
            for i in range(3):
                ps.gemv(ps.matrix_upload("Q4_K", w[i], K), xq, y, i * M, local=local and i != 1)
            out = np.empty((1, 3 * M), np.float32)
            ps.run_host(1, xin, x, y, 0, out)
            ctx.check()
            outs.append(out.copy())
            ps.close()
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint32), outs[0].view(np.uint32))
