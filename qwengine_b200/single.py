"""Times one matvec (or prefill GEMM) shape on cuda:0 and prints one JSON line; also the command ncu profiles.

    python -m qwengine_b200.single --fmt IQ3_XXS --M 17408 --K 5120 --nb 1 [--copies 8] [--reps 5] [--no-pdl]
    python -m qwengine_b200.single --op prefill --fmt Q4_K --M 17408 --K 5120 --tokens 1024

Matvec: `copies` distinct resident matrices (random valid blocks; by default enough to exceed 1.5 GB, far beyond L2)
are recorded as one pass and replayed as a CUDA graph, so host launch overhead does not count.
"""
import argparse
import json

import torch

from . import Context, Pass, formats as F


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemv", choices=["gemv", "prefill"])
    ap.add_argument("--fmt", default="IQ3_XXS")
    ap.add_argument("--M", type=int, default=17408)
    ap.add_argument("--K", type=int, default=5120)
    ap.add_argument("--nb", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--no-pdl", action="store_true")
    a = ap.parse_args()
    ctx = Context(0)
    ctx.set_pdl(not a.no_pdl)
    f = F.get(a.fmt)
    rb = f.row_bytes(a.K)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.op == "gemv":
        copies = a.copies or max(4, int(1.5e9 // (a.M * rb)) + 1)
        ps = Pass(ctx, max_nb=a.nb)
        xin, xq, yb = ps.buffer_f32(a.K), ps.buffer_q8k(a.K), ps.buffer_f32(a.M)
        ps.quantize(xin, 0, a.K, xq)
        for _ in range(copies):
            w = torch.randint(0, 256, (a.M, rb), dtype=torch.uint8, device="cuda")
            ps.gemv(ps.matrix_device(f, w, a.K), xq, yb, 0)
        ps.buffer_tensor(xin).normal_()
        for _ in range(2):
            ps.run(a.nb)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.reps):
            ps.run(a.nb)
        e1.record()
        torch.cuda.synchronize()
        ctx.check()
        us = e0.elapsed_time(e1) * 1e3 / (a.reps * copies)
        print(json.dumps({"op": "gemv", "fmt": f.name, "M": a.M, "K": a.K, "nb": a.nb, "copies": copies, "us_per_launch": round(us, 2),
                          "weight_GBps": round(a.M * rb / us / 1e3, 1)}))
    else:
        w = torch.randint(0, 256, (a.M, rb), dtype=torch.uint8, device="cuda")
        x = torch.randn((a.tokens, a.K), device="cuda", dtype=torch.bfloat16)
        y = torch.empty((a.tokens, a.M), device="cuda")
        for _ in range(2):
            ctx.gemm_prefill(f, w, x, a.K, out=y)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.reps):
            ctx.gemm_prefill(f, w, x, a.K, out=y)
        e1.record()
        torch.cuda.synchronize()
        ctx.check()
        ms = e0.elapsed_time(e1) / a.reps
        print(json.dumps({"op": "prefill", "fmt": f.name, "M": a.M, "K": a.K, "tokens": a.tokens, "ms": round(ms, 4),
                          "TFLOPs": round(2.0 * a.tokens * a.M * a.K / ms / 1e9, 1)}))


if __name__ == "__main__":
    main()
