"""A device-side wait that runs out: the cross-GPU barrier of the peer-store gather waits (bounded) for flags that the
other ranks write.  Here a context is told, through a test hook, that it is rank 0 of 2 with a peer that never
signals; with a budget of a few milliseconds the barrier kernel gives up, returns, and the host reads
Q38B_ERR_DEVICE_WAIT from q38b_ctx_check.  Nothing faults or spins without limit, and the context works afterwards."""
import numpy as np
import pytest
import torch

import oracle
import qwengine_b200 as q
from qwengine_b200 import api, formats as F, synth

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_the_context_stays_usable():
    ctx = q.Context(0)     # a context of its own: the fake peer state must not leak into other tests
    try:
        ctx.set_wait_budget_cycles(5_000_000)            # about 2.5 ms at 2 GHz
        ctx._rc(ctx.lib.q38b_debug_fake_silent_peer(ctx.h, 1), "fake peer")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        ctx._rc(ctx.lib.q38b_peer_barrier(ctx.h, api._stream()), "q38b_peer_barrier")
        ev1.record()
        torch.cuda.synchronize()
        assert ev0.elapsed_time(ev1) < 500.0             # the kernel returned by itself, in milliseconds
        with pytest.raises(api.Q38BError) as e:
            ctx.check()
        assert e.value.status == -5                      # Q38B_ERR_DEVICE_WAIT
        ctx.check()                                      # reading the status cleared it
        ctx._rc(ctx.lib.q38b_debug_fake_silent_peer(ctx.h, 0), "fake peer off")
        # an ordinary matvec on the same context is still right
        f, M, K = F.Q4_K, 300, 1024
        w = synth.make_weights(f, M, K, seed=5)
        xq = oracle.port.quantize_q8k(synth.make_activations(1, K, seed=6))
        y = ctx.gemv(f, torch.from_numpy(w).cuda(), torch.from_numpy(xq).cuda(), K).cpu().numpy()
        ref, mag = oracle.port.row_ref_mag(f.type_id, w, xq[0], K)
        assert np.max(np.abs(y[0] - ref) / np.where(mag == 0, 1, mag)) < 2e-6
        ctx.check()
    finally:
        ctx.close()
