"""The 27B-shaped decode weight pass: every matvec of one token step of the reference model, in order.

Shapes follow the reference model (docs/gguf_inventory.md:58-80 of the reference project; the forward order is
Engine::decode_batch, src/runtime/engine.cpp:1770-1849): 64 layers of hidden size 5120, three of every four a
Gated-DeltaNet layer (in_proj 16384 x 5120, out 5120 x 6144), every fourth a gated-attention layer (q+gate
12288 x 5120, k and v 1024 x 5120, o 5120 x 6144), each followed by the FFN (gate, up 17408 x 5120, SwiGLU, down
5120 x 17408), then the 248320 x 5120 output head.  The recurrence / attention between the projections is not
part of this path: the first 6144 outputs of the input projection stand in for its result, so that every matvec
still consumes data produced by the step before it.  The FFN output of the last layer feeds the head; the other
layers' FFN outputs end in a buffer of their own (see build).

Sharding (one process per GPU): rank g of G owns rows [g*M/G, (g+1)*M/G) of every matrix and the fp32 output
slices are all-gathered so that each rank holds the full vector for the next matvec.
"""
from dataclasses import dataclass

import numpy as np

from . import formats as F

HIDDEN, FF, INNER, VOCAB = 5120, 17408, 6144, 248320
N_LAYERS = 64
TOPK = 32          # candidates the sampler takes from the head (TK of the reference, src/cuda/ops.cu:821)
# fp16 super-scale magnitudes at which a matvec of uniformly random (zero-mean, see synth.ZERO_MEAN_DMIN) blocks has
# a gain near 1, so that the 64 chained layers of the synthetic pass stay inside the fp32 range
UNIT_GAIN_SCALE = {"Q4_K": 5.0e-5, "IQ3_XXS": 1.4e-4, "IQ4_XS": 5.5e-6, "Q6_K": 1.0e-5}


@dataclass(frozen=True)
class MatSpec:
    name: str
    fmt: str
    M: int
    K: int

    @property
    def nbytes(self):
        return self.M * F.get(self.fmt).row_bytes(self.K)


def layer_specs(il):
    attn = il % 4 == 3
    if attn:
        mats = [MatSpec(f"l{il}.q_gate", "Q4_K", 12288, HIDDEN), MatSpec(f"l{il}.k", "Q4_K", 1024, HIDDEN),
                MatSpec(f"l{il}.v", "Q4_K", 1024, HIDDEN), MatSpec(f"l{il}.o", "Q4_K", HIDDEN, INNER)]
    else:
        mats = [MatSpec(f"l{il}.in_proj", "Q4_K", 16384, HIDDEN), MatSpec(f"l{il}.out", "Q4_K", HIDDEN, INNER)]
    mats += [MatSpec(f"l{il}.gate", "IQ3_XXS", FF, HIDDEN), MatSpec(f"l{il}.up", "IQ3_XXS", FF, HIDDEN),
             MatSpec(f"l{il}.down", "IQ4_XS", HIDDEN, FF)]
    return attn, mats


def all_specs(n_layers=N_LAYERS, head=True):
    out = []
    for il in range(n_layers):
        out += layer_specs(il)[1]
    if head:
        out.append(MatSpec("lm_head", "Q6_K", VOCAB, HIDDEN))
    return out


def total_weight_bytes(n_layers=N_LAYERS, head=True):
    return sum(m.nbytes for m in all_specs(n_layers, head))


def build(ps, make_matrix, n_layers=N_LAYERS, head=True, rank=0, world=1, gather="peer", replicate_small=True):
    """Records the pass on `ps` (qwengine_b200.Pass).

    make_matrix(spec, rows) -> matrix id for this rank's shard of `rows` rows (rows = spec.M // world);
    make_matrix(spec, spec.M, replicated=True) -> matrix id for a matrix this rank holds whole (only asked for when
    world > 1 and replicate_small).
    world > 1: gather = "peer" pushes every output slice into the peers' buffers from the matvec kernel and
    synchronises with one cross-GPU barrier per group of matvecs (the context must be peer-connected before the pass
    is created); gather = "nccl" records an NCCL all-gather after every matvec; gather = "none" records no exchange at
    all (this rank's share of the work alone, for timing: the results are incomplete).
    replicate_small: the attention-side projections (in_proj / q, k, v / out: 65 MB per layer) are held whole by every
    rank and computed by every rank: streaming 65 MB costs a GPU about 11 us, sharding them over N GPUs saves at most
    (1 - 1/N) of that and costs two cross-GPU exchanges of 4-5 us each per layer.  The FFN (115 MB per layer) and the
    head (1 GB) are row-sharded.  Bit-identical either way: a row's result does not depend on who computes it.
    Returns dict(in_buf, out_buf, out_len, topk_buf, topk_k).
    """
    x_in = ps.buffer_f32(HIDDEN)           # the token's hidden state: read by layer 0 only, never written, so that
                                           # every replay computes the same thing from the same input
    x = ps.buffer_f32(HIDDEN)              # residual-stream stand-in: output of every layer, input of the next
    xq = ps.buffer_q8k(HIDDEN)
    big = ps.buffer_f32(16384)             # projection outputs (in_proj / q+gate)
    kv = ps.buffer_f32(2048)
    iq = ps.buffer_q8k(INNER)
    gu = ps.buffer_f32(2 * FF)             # gate | up
    hq = ps.buffer_q8k(FF)
    ffn = ps.buffer_f32(HIDDEN)            # FFN block outputs (see below)
    logits = ps.buffer_f32(VOCAB) if head else None
    peer = world > 1 and gather == "peer"   # needs Context.peer_connect before the pass is created
    if hasattr(ps, "set_peer_store"):
        ps.set_peer_store(peer)

    whole = world > 1 and replicate_small   # the attention-side projections are not sharded

    def matvec(spec, src_q, dst, off, shard=True):
        if world > 1 and not shard:
            ps.gemv(make_matrix(spec, spec.M, replicated=True), src_q, dst, off, local=True)
            return
        rows = spec.M // world
        mid = make_matrix(spec, rows)
        ps.gemv(mid, src_q, dst, off + rank * rows)
        if world > 1 and gather == "nccl":
            ps.allgather(dst, off, rows)

    def sync(after_sharded=True):
        if peer and after_sharded:
            ps.barrier()

    for il in range(n_layers):
        attn, mats = layer_specs(il)
        ps.quantize(x_in if il == 0 else x, 0, HIDDEN, xq)
        if attn:
            matvec(mats[0], xq, big, 0, shard=not whole)
            matvec(mats[1], xq, kv, 0, shard=not whole)
            matvec(mats[2], xq, kv, 1024, shard=not whole)
            proj_out = mats[3]
        else:
            matvec(mats[0], xq, big, 0, shard=not whole)
            proj_out = mats[1]
        sync(not whole)
        ps.quantize(big, 0, INNER, iq)
        matvec(proj_out, iq, x, 0, shard=not whole)
        sync(not whole)
        ps.quantize(x, 0, HIDDEN, xq)
        gate, up, down = mats[-3:]
        matvec(gate, xq, gu, 0)
        matvec(up, xq, gu, FF)
        sync()
        ps.swiglu(gu, 0, gu, FF, FF, hq)
        # The FFN block's output goes to a buffer of its own, not back into x (except in the last layer, so that the
        # pass's result depends on it): without the model's RMSNorm in front of it, silu(g) * u squares the scale of
        # the stream at every layer and 64 chained layers leave the fp32 range whatever the weight scales are.  The
        # chain x -> projections -> x stays linear (gain near 1 per layer).
        matvec(down, hq, x if il == n_layers - 1 else ffn, 0)
        sync()
    best = None
    if head:
        ps.quantize(x, 0, HIDDEN, xq)
        matvec(MatSpec("lm_head", "Q6_K", VOCAB, HIDDEN), xq, logits, 0)
        sync()
        if hasattr(ps, "topk"):
            # what the sampler needs from the head (Engine::decode_batch's top-k, src/runtime/engine.cpp:1680 of the
            # reference project): TOPK values and positions per column instead of 248320 logits
            best = ps.buffer_f32(2 * TOPK)
            ps.topk(logits, 0, VOCAB, TOPK, best)
    return dict(in_buf=x_in, out_buf=logits if head else x, out_len=VOCAB if head else HIDDEN, topk_buf=best, topk_k=TOPK)


def oracle_forward(port, weights, x, n_layers, head=True):
    """CPU restatement of the same chain with the oracle (tests only).  weights: dict name -> uint8 [M, row_bytes]."""
    x = np.ascontiguousarray(x, np.float32)
    nb = x.shape[0]
    for il in range(n_layers):
        attn, mats = layer_specs(il)
        xq = port.quantize_q8k(x)
        big = port.gemv(F.get(mats[0].fmt).type_id, weights[mats[0].name], xq, HIDDEN)
        proj_out = mats[3] if attn else mats[1]
        iq = port.quantize_q8k(np.ascontiguousarray(big[:, :INNER]))
        x = port.gemv(F.get(proj_out.fmt).type_id, weights[proj_out.name], iq, INNER)
        xq = port.quantize_q8k(x)
        gate, up, down = mats[-3:]
        g = port.gemv(F.get(gate.fmt).type_id, weights[gate.name], xq, HIDDEN)
        u = port.gemv(F.get(up.fmt).type_id, weights[up.name], xq, HIDDEN)
        h = port.swiglu(g, u).reshape(nb, FF)
        y = port.gemv(F.get(down.fmt).type_id, weights[down.name], port.quantize_q8k(h), FF)
        if il == n_layers - 1:
            x = y
    if head:
        return port.gemv(F.Q6_K.type_id, weights["lm_head"], port.quantize_q8k(x), HIDDEN)
    return x
