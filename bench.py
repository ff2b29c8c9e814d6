#!/usr/bin/env python3
"""Benchmark of the decode weight pass (27B-shaped, 64 layers + output head, 12.5 GB of GGUF blocks).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one full pass over all 353 weight matrices for one token (nb = 1): Q8_K quantisation, matvec,
SwiGLU, matvec ..., replayed as a CUDA graph by the C++ planner.  `value` is weight bytes streamed per second
summed over all ranks (the pass is row-sharded over the ranks and the output slices are all-gathered, so the
total work is fixed: strong scaling).  Synthetic seeded weights stand in for the model file.
The single JSON line also carries the nb = 7 pass, the end-to-end number through the host-buffer C ABI, a live
roofline measurement of the dominant kernel and the reference's AVX2 kernels timed on this box's host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_weight_pass_stream_bandwidth"
UNIT = "GB/s"
HBM_NOMINAL_GBS = 8000.0
# dram__bytes_read of one IQ3_XXS one-column launch divided by its GGUF bytes, from an ncu capture of the kernel on
# THREE 17408 x 5120 matrices per launch (102.44 MB read for 102.36 MB of blocks); the launch timed below has two, and
# traffic grows in proportion to the rows, so it is scaled by the launch's bytes
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0008


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own AVX2 kernels (oracle/_ref) on a bounded sample of the same pass
# ---------------------------------------------------------------------------------------------------------------
def cpu_sample_specs():
    from qwengine_b200 import decode_pass as dp
    specs = dp.all_specs(n_layers=4, head=False)                      # 3 DeltaNet layers + 1 attention layer
    specs.append(dp.MatSpec("lm_head_slice", "Q6_K", dp.VOCAB // 16, dp.HIDDEN))
    return specs


def cpu_run(seconds_budget=None, steps=None, warmup=1):
    """Times the reference CPU kernels; returns dict(value GB/s, cores, kind, sample, ms_per_step, steps)."""
    import oracle
    from qwengine_b200 import formats as F, synth
    cores = len(os.sched_getaffinity(0))
    impl = oracle.ref if oracle.ref is not None else None
    kind = "reference" if impl is not None else "port"
    specs = cpu_sample_specs()
    rng = np.random.Generator(np.random.PCG64(99))
    mats = []
    for s in specs:
        f = F.get(s.fmt)
        w = rng.integers(0, 256, size=(s.M, f.row_bytes(s.K)), dtype=np.uint8)   # timing does not depend on the values
        xq = oracle.port.quantize_q8k(synth.make_activations(1, s.K, seed=s.K))
        mats.append((f, w, xq, s.K))
    nbytes = sum(m[1].nbytes for m in mats)

    def one_pass():
        t = 0.0
        for f, w, xq, K in mats:
            if impl is not None:
                t += impl.gemv(f.type_id, w, xq, K, threads=cores)[1]
            else:
                t0 = time.perf_counter()
                oracle.port.gemv(f.type_id, w, xq, K)
                t += time.perf_counter() - t0
        return t

    # the reference's pool spins its threads up lazily and the weights are first touched here: at least a second of
    # untimed passes, so that a short timed run measures the steady state
    t_warm = time.perf_counter()
    n_warm = 0
    while n_warm < max(1, warmup) or time.perf_counter() - t_warm < 1.0:
        one_pass()
        n_warm += 1
    times = []
    t_start = time.perf_counter()
    while True:
        times.append(one_pass())
        if steps is not None and len(times) >= steps:
            break
        if steps is None and time.perf_counter() - t_start > seconds_budget:
            break
    sec = sum(times) / len(times)
    return {"value": round(nbytes / sec / 1e9, 2), "unit": UNIT, "cores": cores, "kind": kind, "sample_bytes": nbytes,
            "sample": f"layers 0-3 (8 Q4_K, 8 IQ3_XXS, 4 IQ4_XS matrices) + 1/16 of the Q6_K head = {nbytes / 1e6:.0f} MB per "
                      f"pass, nb=1, {len(times)} timed passes",
            "ms_per_step": sec * 1e3, "steps": len(times)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from qwengine_b200 import decode_pass as dp
    r = cpu_run(steps=max(1, args.steps), warmup=max(1, args.warmup))
    total_bytes = dp.total_weight_bytes(args.layers, True)
    line = {"metric": METRIC, "value": r["value"], "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": r["steps"],
            "warmup": args.warmup, "ms_per_step": round(r["ms_per_step"], 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": run_config(args.layers, args.gpus, args.gather),
            "sample_fraction": round(r["sample_bytes"] / total_bytes, 5),
            "arm": "the reference's AVX2 CPU kernels on this box's host cores; each step = one pass over a bounded sample of the workload's matrices (same format mix)",
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_config(n_layers, world, gather):
    """The `config` object of both arms: the workload BASELINE.json's configs[4] names."""
    from qwengine_b200 import decode_pass as dp
    cfg = {"workload": "decode_weight_pass_27b_shape", "layers": n_layers, "matrices": len(dp.all_specs(n_layers)),
           "weight_bytes": dp.total_weight_bytes(n_layers, True), "nb": 1,
           "parallelism": f"row-shard x{world}" + (f" (FFN and head; attention-side projections whole on every rank) + {gather} gather" if world > 1 else ""),
           "cache": "12.5 GB of weights per pass, far larger than L2; no flush needed"}
    return cfg


# ---------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------
_FP16_FIELDS = {"Q8_0": (0,), "Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,), "IQ3_XXS": (0,), "IQ3_S": (0,), "IQ4_XS": (0,)}


def device_weights(torch, spec, rows, seed, scale):
    """Random valid blocks generated on the device: uniform bytes, fp16 super-scales |N(0,1)| * scale."""
    from qwengine_b200 import formats as F
    f = F.get(spec.fmt)
    g = torch.Generator(device="cuda").manual_seed(seed)
    nblk = spec.K // f.block_elems
    w = torch.randint(0, 256, (rows, nblk, f.block_bytes), dtype=torch.uint8, device="cuda", generator=g)
    from qwengine_b200 import synth
    d0 = None
    for off in _FP16_FIELDS[f.name]:
        d = torch.randn((rows, nblk), device="cuda", generator=g).abs() * scale
        if off == 2 and f.name in synth.ZERO_MEAN_DMIN:
            d = d0 * synth.ZERO_MEAN_DMIN[f.name]          # zero-mean weights: see synth.ZERO_MEAN_DMIN
        d0 = d
        w[:, :, off:off + 2] = d.to(torch.float16).view(torch.uint8).view(rows, nblk, 2)
    return w.view(rows, nblk * f.block_bytes)


def time_pass(torch, ps, nb, reps, warm=2):
    for _ in range(warm):
        ps.run(nb)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        ps.run(nb)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def per_format_table(torch, q, ctx, peak):
    """Every format at 17408 x 5120, one matrix per launch, cycling over distinct resident matrices of more than 1 GB in
    all (far beyond L2), for 1 and 7 activation columns: us per matvec, GB/s of GGUF bytes, fraction of the HBM peak."""
    from qwengine_b200 import decode_pass as dp, formats as F
    M, K = dp.FF, dp.HIDDEN
    out = {}
    for name in F.FORMATS:
        f = F.get(name)
        nbytes = M * f.row_bytes(K)
        copies = int(1.1e9 // nbytes) + 1
        ps = q.Pass(ctx, max_nb=7)
        ps.set_merge(False)                      # one launch per matrix
        xin, xq, yb = ps.buffer_f32(K), ps.buffer_q8k(K), ps.buffer_f32(M)
        ps.quantize(xin, 0, K, xq)
        g = torch.Generator(device="cuda").manual_seed(F.get(name).type_id)
        for _ in range(copies):
            w = torch.randint(0, 256, (M, f.row_bytes(K)), dtype=torch.uint8, device="cuda", generator=g)
            ps.gemv(ps.matrix_device(f, w, K), xq, yb, 0)
        ps.buffer_tensor(xin).normal_(generator=g)
        row = {"bytes_per_matvec": nbytes, "distinct_matrices": copies}
        for nb in (1, 7):
            us = time_pass(torch, ps, nb, 3) * 1e3 / copies
            gbs = nbytes / us / 1e3
            row[f"nb{nb}"] = {"us": round(us, 2), "GBps": round(gbs, 1), "frac": round(gbs / peak, 4)}
        row["nb7_vs_nb1"] = round(row["nb7"]["us"] / row["nb1"]["us"], 3)
        out[name] = row
        ps.close()
    return out


def ffn_block_time(torch, q, ctx):
    """The decode FFN block: gate and up 17408 x 5120 in Q4_K, SwiGLU, down 5120 x 17408 in Q6_K, one column; eight
    distinct blocks (1.4 GB) per replay."""
    from qwengine_b200 import decode_pass as dp, formats as F
    ps = q.Pass(ctx, max_nb=1)
    x, xq, gu, hq = ps.buffer_f32(dp.HIDDEN), ps.buffer_q8k(dp.HIDDEN), ps.buffer_f32(2 * dp.FF), ps.buffer_q8k(dp.FF)
    g = torch.Generator(device="cuda").manual_seed(4242)
    n = 8
    nbytes = 0
    for _ in range(n):
        ps.quantize(x, 0, dp.HIDDEN, xq)
        for off in (0, dp.FF):
            w = torch.randint(0, 256, (dp.FF, F.Q4_K.row_bytes(dp.HIDDEN)), dtype=torch.uint8, device="cuda", generator=g)
            w[:, 0::144] = 0; w[:, 1::144] = 0; w[:, 2::144] = 0; w[:, 3::144] = 0      # d = dmin = 0: the chain stays finite
            ps.gemv(ps.matrix_device(F.Q4_K, w, dp.HIDDEN), xq, gu, off)
            nbytes += w.numel()
        ps.swiglu(gu, 0, gu, dp.FF, dp.FF, hq)
        w = torch.randint(0, 256, (dp.HIDDEN, F.Q6_K.row_bytes(dp.FF)), dtype=torch.uint8, device="cuda", generator=g)
        w[:, 208::210] = 0; w[:, 209::210] = 0
        ps.gemv(ps.matrix_device(F.Q6_K, w, dp.FF), hq, x, 0)
        nbytes += w.numel()
    us = time_pass(torch, ps, 1, 5) * 1e3 / n
    ps.close()
    return {"us_per_block": round(us, 2), "bytes_per_block": nbytes // n, "GBps": round(nbytes / n / us / 1e3, 1), "kernels_per_block": 3}


def prefill_table(torch, ctx):
    """The prefill chunk GEMM: 1024 bf16 tokens against 17408 x 5120 and 5120 x 17408 weights in IQ3_XXS and Q4_K."""
    from qwengine_b200 import formats as F
    peak, kind = measured_tensor_peak()
    out = {"tokens": 1024, "peak_TFLOPs": peak, "peak_source": kind + " cuBLAS bf16 burst", "cases": {}}
    g = torch.Generator(device="cuda").manual_seed(99)
    best = 0.0
    for name in ("IQ3_XXS", "Q4_K"):
        f = F.get(name)
        for M, K in ((17408, 5120), (5120, 17408)):
            w = torch.randint(0, 256, (M, f.row_bytes(K)), dtype=torch.uint8, device="cuda", generator=g)
            x = torch.randn((1024, K), device="cuda", generator=g).to(torch.bfloat16)
            y = torch.empty((1024, M), device="cuda")
            for _ in range(2):
                ctx.gemm_prefill(f, w, x, K, out=y)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                ctx.gemm_prefill(f, w, x, K, out=y)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            tf = 2.0 * 1024 * M * K / ms / 1e9
            best = max(best, tf)
            out["cases"][f"{name}_{M}x{K}"] = {"ms": round(ms, 4), "TFLOPs": round(tf, 1), "frac": round(tf / peak, 4)}
    out["roofline"] = {"bound": "tensor", "achieved": round(best, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(best / peak, 4)}
    return out


def sharded_equals_single(torch, dist, q, ctx, rank, world, gather):
    """Correctness of the row-sharded pass at this world size: a 4-layer + head pass on seeded weights, sharded over the
    ranks, against the same pass unsharded on rank 0's GPU (a context of its own), bit for bit, for 1 and 7 columns."""
    from qwengine_b200 import decode_pass as dp, formats as F
    n_layers = 4

    def weights(spec, rows_from, rows):
        # the whole matrix from a seed that does not depend on the rank, then this rank's rows
        w = device_weights(torch, spec, spec.M, seed=777 + sum(map(ord, spec.name)), scale=dp.UNIT_GAIN_SCALE.get(spec.fmt, 1e-3))
        return w[rows_from:rows_from + rows].contiguous()

    x0 = torch.randn((7, dp.HIDDEN), device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    ps = q.Pass(ctx, max_nb=7)
    io = dp.build(ps, lambda spec, rows, replicated=False: ps.matrix_device(spec.fmt, weights(spec, 0 if replicated else rank * rows, rows), spec.K),
                  n_layers=n_layers, head=True, rank=rank, world=world, gather=gather)
    outs = {}
    for nb in (1, 7):
        ps.buffer_tensor(io["in_buf"]).copy_(x0)
        ps.run(nb)
        torch.cuda.synchronize()
        dist.barrier()
        outs[nb] = ps.buffer_tensor(io["out_buf"])[:nb].clone()
    ok = True
    if rank == 0:
        c1 = q.Context(torch.cuda.current_device())
        p1 = q.Pass(c1, max_nb=7)
        io1 = dp.build(p1, lambda spec, rows: p1.matrix_device(spec.fmt, weights(spec, 0, rows), spec.K), n_layers=n_layers, head=True)
        for nb in (1, 7):
            p1.buffer_tensor(io1["in_buf"]).copy_(x0)
            p1.run(nb)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(p1.buffer_tensor(io1["out_buf"])[:nb].view(torch.int32), outs[nb].view(torch.int32)))
        c1.check()
        p1.close()
        c1.close()
    ps.close()
    dist.barrier()
    return ok


def run_ours(args):
    import torch
    import torch.distributed as dist
    import qwengine_b200 as q
    from qwengine_b200 import build as qbuild, decode_pass as dp, formats as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        qbuild.build()
    if world > 1:
        dist.barrier()
    ctx = q.Context(local)
    if world > 1:
        idbuf = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            import ctypes as C
            raw = (C.c_ubyte * 128)()
            ctx._rc(ctx.lib.q38b_comm_unique_id(raw), "q38b_comm_unique_id")
            idbuf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
        dist.broadcast(idbuf, 0)
        host_id = bytes(idbuf.cpu().tolist())
        ctx._rc(ctx.lib.q38b_comm_init(ctx.h, world, rank, host_id), "q38b_comm_init")

    def exchange(handle):
        """All ranks' 64-byte IPC handles, in rank order."""
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
        out = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(out, mine)
        return [bytes(t.cpu().tolist()) for t in out]

    if world > 1 and args.gather == "peer":
        ctx.peer_connect(world, rank, exchange(ctx.peer_arena_create()))

    shard_ok = None
    if world > 1:
        shard_ok = sharded_equals_single(torch, dist, q, ctx, rank, world, args.gather)

    n_layers = args.layers
    ps = q.Pass(ctx, max_nb=7)
    counter = [0]
    made = []   # the weight tensors in the order the pass asked for them

    def make_matrix(spec, rows, replicated=False):
        counter[0] += 1   # a replicated matrix has the same bytes on every rank
        w = device_weights(torch, spec, rows, seed=1000 * counter[0] + (0 if replicated else rank), scale=dp.UNIT_GAIN_SCALE.get(spec.fmt, 1e-3))
        made.append(w)
        return ps.matrix_device(spec.fmt, w, spec.K)

    io = dp.build(ps, make_matrix, n_layers=n_layers, head=True, rank=rank, world=world, gather=args.gather)
    local_bytes = ps.weight_bytes
    total_bytes = dp.total_weight_bytes(n_layers, True)
    xin = ps.buffer_tensor(io["in_buf"])
    x0 = torch.randn((7, dp.HIDDEN), device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(nb, steps, warmup):
        for _ in range(warmup):
            xin.copy_(x0)
            ps.run(nb)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            ps.run(nb)
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    warm = max(3, args.warmup)
    with ClockSampler(local) as clocks:
        ms1 = timed(1, args.steps, warm)
    ms7 = timed(7, max(3, args.steps // 2), 3)
    ctx.check()
    # What the cross-GPU exchanges cost: the same pass on the same weights with no exchange recorded (no peer stores, no
    # barriers: every rank's share of the work alone; its results are incomplete and are not used).
    exchange = None
    if world > 1:
        it = iter(made)
        ps_alone = q.Pass(ctx, max_nb=1)
        dp.build(ps_alone, lambda spec, rows, replicated=False: ps_alone.matrix_device(spec.fmt, next(it), spec.K), n_layers=n_layers, head=True,
                 rank=rank, world=world, gather="none")
        t_alone = torch.tensor([time_pass(torch, ps_alone, 1, max(3, args.steps // 2), warm=3)], device="cuda")
        dist.all_reduce(t_alone, op=dist.ReduceOp.MAX)
        ps_alone.close()
        exchange = {"ms_per_step_without_exchange": round(float(t_alone.item()), 4), "share_of_step": round(1.0 - float(t_alone.item()) / ms1, 4)}
    logits = ps.buffer_tensor(io["out_buf"])
    finite = bool(torch.isfinite(logits[:7]).all().item())

    # end to end through the host-buffer entry point: pinned staging, H2D of the token's hidden state, the pass,
    # D2H of the step's result (the head's top-k values and positions, what the sampler reads), synchronise -- every step
    xh = np.ascontiguousarray(x0[:1].cpu().numpy())
    yh = np.empty((1, 2 * io["topk_k"]), np.float32)
    for _ in range(3):
        ps.run_host(1, io["in_buf"], xh, io["topk_buf"], 0, yh)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ps.run_host(1, io["in_buf"], xh, io["topk_buf"], 0, yh)
    sync_all()
    e2e_elapsed = time.perf_counter() - t0
    # the returned candidates are the logits' largest (checked once, outside the timed region)
    k_ = io["topk_k"]
    top_v, top_i = torch.topk(logits[0], k_)
    topk_ok = bool(np.array_equal(np.sort(yh[0, k_:].view(np.int32)), np.sort(top_i.cpu().numpy().astype(np.int32)))) if finite else None
    e2e_ms = torch.tensor([e2e_elapsed * 1e3 / args.steps], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())

    # Roofline of the dominant kernel, measured live: the launch the pass makes for every layer's gate + up projections
    # (gemv1_kernel<IQ3_XXS>: two 17408 x 5120 matrices on one column, the column quantized inside the kernel; 35 % of the
    # pass's bytes).  32 launches on 64 distinct resident matrices (2.2 GB at one GPU: far larger than L2), recorded as a
    # pass and replayed as a CUDA graph so that the host's launch rate does not enter; CUDA events on the stream.
    spec = dp.MatSpec("roof", "IQ3_XXS", dp.FF, dp.HIDDEN)
    rows = spec.M // world
    f = F.get(spec.fmt)
    n_pairs = max(4, 32 // world)
    mats = [device_weights(torch, spec, rows, seed=50000 + i, scale=1.4e-4) for i in range(2 * n_pairs)]
    rp = q.Pass(ctx, max_nb=1)
    r_in, r_xq = rp.buffer_f32(spec.K), rp.buffer_q8k(spec.K)
    r_ya, r_yb = rp.buffer_f32(rows), rp.buffer_f32(rows)
    for i in range(n_pairs):
        rp.quantize(r_in, 0, spec.K, r_xq)           # folded into the launch of the two matvecs after it
        rp.gemv(rp.matrix_device(f, mats[2 * i], spec.K), r_xq, r_ya, 0)
        rp.gemv(rp.matrix_device(f, mats[2 * i + 1], spec.K), r_xq, r_yb, 0)
    assert rp.kernel_count == n_pairs, rp.kernel_count
    rp.buffer_tensor(r_in).copy_(x0[0])
    for _ in range(3):
        rp.run(1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 4
    e0.record()
    for _ in range(reps):
        rp.run(1)
    e1.record()
    torch.cuda.synchronize()
    ctx.check()
    kern_us = e0.elapsed_time(e1) * 1e3 / (reps * n_pairs)
    alg_bytes = 2 * rows * f.row_bytes(spec.K)
    peak, peak_kind = measured_peak()
    achieved = alg_bytes / kern_us / 1e3
    roofline = {"bound": "hbm", "kernel": "gemv1_kernel<IQ3_XXS>, gate + up (2 x 17408x5120/%d) in one launch, nb=1" % world, "achieved": round(achieved, 1),
                "peak": peak, "peak_source": peak_kind + " copy bandwidth", "unit": UNIT, "frac": round(achieved / peak, 4),
                "frac_of_nominal_8TBps": round(achieved / HBM_NOMINAL_GBS, 4), "us_per_launch": round(kern_us, 2),
                "algorithmic_bytes_per_launch": alg_bytes,
                "traffic": int(alg_bytes * DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE),
                "traffic_source": "scaled from the dram bytes of an ncu capture of the same kernel with three matrices per launch on one GPU, by the launch's GGUF bytes"}
    rp.close()
    del mats
    extras = {}
    if rank == 0 and world == 1 and not args.no_extras:
        torch.cuda.empty_cache()
        extras["per_format_17408x5120"] = per_format_table(torch, q, ctx, peak)
        extras["ffn_block"] = ffn_block_time(torch, q, ctx)
        extras["prefill_1024_tokens"] = prefill_table(torch, ctx)
        ctx.check()

    line = None
    if rank == 0:
        value = total_bytes / ms1 / 1e6
        cpu = cpu_run(seconds_budget=12.0) if (world == 1 and not args.no_cpu) else None
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": round(ms1, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": run_config(n_layers, world, args.gather),
            "checks": {"outputs_finite": finite, "topk_matches_logits": topk_ok, "sharded_bits_equal_single": shard_ok},
            "exchange": exchange,
            "tokens_per_s": round(1e3 / ms1, 1),
            "frac_of_nominal_8TBps": round(value / world / HBM_NOMINAL_GBS, 4),
            "nb7": {"ms_per_step": round(ms7, 4), "value": round(total_bytes / ms7 / 1e6, 1), "tokens_per_s": round(7e3 / ms7, 1),
                    "time_vs_nb1": round(ms7 / ms1, 3)},
            "e2e": {"value": round(total_bytes / e2e_ms / 1e6, 1), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": int(xh.nbytes), "d2h_bytes_per_step": int(yh.nbytes)},
            "gpu_launches": ps.kernel_count * args.steps,
            "roofline": roofline,
            "clocks": clocks.summary(),
        }
        line.update(extras)
        if "prefill_1024_tokens" in extras:
            line["roofline_prefill"] = extras["prefill_1024_tokens"]["roofline"]
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    ps.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64, help="number of layers of the pass (64 = the benchmark configuration)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"], help="multi-GPU output exchange: fused peer stores or NCCL")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-format, FFN-block and prefill legs (one GPU only)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
