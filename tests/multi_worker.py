"""Worker of the multi-rank tests (launched with torch.distributed.run).

mode "cpu":  gloo ranks; every rank computes its row shard of a small pass with the CPU oracle and the slices are
             all-gathered -- checks the sharding arithmetic of qwengine_b200.decode_pass (rows, offsets) without a GPU.
mode "gpu":  one rank per GPU; the recorded pass with the peer-store gather (and with NCCL) must reproduce the bits
             of the unsharded pass run by every rank on its own.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import oracle                                                   # noqa: E402
from qwengine_b200 import decode_pass as dp, formats as F, synth   # noqa: E402

N_LAYERS = 4


def weights():
    return {s.name: synth.make_weights(s.fmt, s.M, s.K, seed=300 + i, scale=dp.UNIT_GAIN_SCALE[s.fmt], zero_mean=True)
            for i, s in enumerate(dp.all_specs(N_LAYERS, head=False))}


class OracleRecorder:
    """Stands in for qwengine_b200.Pass: executes the recorded steps at once with the oracle and a gloo all-gather."""

    def __init__(self, ws, nb, world):
        self.ws, self.nb, self.world, self.bufs, self.mats = ws, nb, world, [], []

    def buffer_f32(self, n):
        self.bufs.append(np.zeros((self.nb, n), np.float32)); return len(self.bufs) - 1

    def buffer_q8k(self, K):
        self.bufs.append(None); return len(self.bufs) - 1

    def quantize(self, src, off, K, dst):
        self.bufs[dst] = oracle.port.quantize_q8k(np.ascontiguousarray(self.bufs[src][:, off:off + K]))

    def gemv(self, mat, src_q, dst, off, local=False):
        spec, w = self.mats[mat]
        y = oracle.port.gemv(F.get(spec.fmt).type_id, w, self.bufs[src_q], spec.K)
        self.bufs[dst][:, off:off + w.shape[0]] = y

    def swiglu(self, g, g_off, u, u_off, n, dst):
        h = oracle.port.swiglu(np.ascontiguousarray(self.bufs[g][:, g_off:g_off + n]),
                               np.ascontiguousarray(self.bufs[u][:, u_off:u_off + n])).reshape(self.nb, n)
        self.bufs[dst] = oracle.port.quantize_q8k(h)

    def allgather(self, buf, off, count):
        mine = torch.from_numpy(np.ascontiguousarray(self.bufs[buf][:, off + dist.get_rank() * count: off + (dist.get_rank() + 1) * count]))
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        for r, t in enumerate(parts):
            self.bufs[buf][:, off + r * count: off + (r + 1) * count] = t.numpy()


def run_cpu():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ws = weights()
    x = synth.make_activations(2, dp.HIDDEN, seed=5)
    rec = OracleRecorder(ws, 2, world)

    def make(spec, rows, replicated=False):
        rec.mats.append((spec, ws[spec.name] if replicated else ws[spec.name][rank * rows:(rank + 1) * rows]))
        return len(rec.mats) - 1

    # record with the in-buffer filled: buffer 0 is the input
    orig = rec.buffer_f32

    def first_buffer(n, _done=[False]):
        i = orig(n)
        if not _done[0]:
            rec.bufs[i][:] = x
            _done[0] = True
        return i
    rec.buffer_f32 = first_buffer
    io = dp.build(rec, make, n_layers=N_LAYERS, head=False, rank=rank, world=world, gather="nccl")
    got = rec.bufs[io["out_buf"]]
    want = dp.oracle_forward(oracle.port, ws, x, N_LAYERS, head=False)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "sharded oracle pass differs from the unsharded one"
    dist.barrier()
    if rank == 0:
        print("MULTI_CPU_OK")
    dist.destroy_process_group()


def run_gpu():
    import qwengine_b200 as q
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    ctx = q.Context(local)

    def exchange(handle):
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
        out = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(out, mine)
        return [bytes(t.cpu().tolist()) for t in out]

    import ctypes as C
    idbuf = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        raw = (C.c_ubyte * 128)()
        ctx._rc(ctx.lib.q38b_comm_unique_id(raw), "q38b_comm_unique_id")
        idbuf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
    dist.broadcast(idbuf, 0)
    ctx._rc(ctx.lib.q38b_comm_init(ctx.h, world, rank, bytes(idbuf.cpu().tolist())), "q38b_comm_init")
    ctx.peer_connect(world, rank, exchange(ctx.peer_arena_create()))
    ws = weights()
    outs = {}
    for nb in (1, 3):
        x = synth.make_activations(nb, dp.HIDDEN, seed=5)
        for mode in ("single", "peer", "peer_all_sharded", "nccl"):
            ps = q.Pass(ctx, max_nb=nb)
            w_, r_ = (1, 0) if mode == "single" else (world, rank)
            # "peer_all_sharded": every matrix row-sharded; the other sharded modes keep the attention-side projections whole
            io = dp.build(ps, lambda spec, rows, replicated=False: ps.matrix_upload(spec.fmt, ws[spec.name], spec.K, shard=0 if replicated else r_,
                                                                                      n_shards=1 if replicated else w_),
                          n_layers=N_LAYERS, head=False, rank=r_, world=w_, gather="peer" if mode.startswith("peer") else mode,
                          replicate_small=mode != "peer_all_sharded")
            y = np.empty((nb, dp.HIDDEN), np.float32)
            for _ in range(3):      # replays reuse the flags and the buffers
                ps.run_host(nb, io["in_buf"], x, io["out_buf"], 0, y)
            ctx.check()
            outs[(nb, mode)] = y.copy()
            dist.barrier()
            ps.close()
        assert np.array_equal(outs[(nb, "peer")].view(np.uint32), outs[(nb, "single")].view(np.uint32)), "peer gather differs"
        assert np.array_equal(outs[(nb, "peer_all_sharded")].view(np.uint32), outs[(nb, "single")].view(np.uint32)), "peer gather (all sharded) differs"
        assert np.array_equal(outs[(nb, "nccl")].view(np.uint32), outs[(nb, "single")].view(np.uint32)), "nccl gather differs"
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    run_cpu() if sys.argv[1] == "cpu" else run_gpu()
