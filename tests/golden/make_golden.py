#!/usr/bin/env python3
"""Generates tests/golden/ref_vectors.npz from the REFERENCE's own code.

Run in a checkout where oracle/_ref/libq38ref.so exists (built by `make -C oracle` from the reference
sources).  For seeded synthetic blocks it records what the reference computes:
  * dequantize_row_ref for the six formats it implements (Q5_K: gguf-py's dequantizer, the only
    independent implementation available; the reference has none);
  * quantize_row_q8_K_ref on N(0,1) activations and on the edge cases of the reference's tests
    (tests/unit/test_quant_ref.cpp:118-123, tests/kernels/test_cpu_gemv.cpp:77-92);
  * the AVX2 dot products get_vec_dot_n for nb = 1..3 for the five formats that have one.
The GPU box has no reference checkout; tests there compare against these committed vectors.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle                                  # noqa: E402
from qwengine_b200 import formats as F, synth  # noqa: E402

M, K, NB = 12, 768, 3


def edge_activations():
    rng = np.random.Generator(np.random.PCG64(1234))
    rows = []
    for t in range(9):
        rows.append(rng.standard_normal(K, dtype=np.float32) * np.float32(10.0 ** (t - 4)))
    z = np.zeros(K, np.float32)
    rows.append(z.copy())
    one = z.copy(); one[3::256] = -5.0
    rows.append(one)
    rows.append(rng.standard_normal(K, dtype=np.float32) * np.float32(1e-30))
    tie = z.copy(); tie[10] = 2.0; tie[20] = -2.0; tie[300] = -1.5; tie[301] = 1.5   # first maximum wins
    rows.append(tie)
    half = np.arange(K, dtype=np.float32) / np.float32(2.0) - np.float32(100.0)   # exact .5 products
    rows.append(half)
    return np.stack(rows)


def main():
    assert oracle.ref is not None, "build oracle/_ref first (make -C oracle)"
    out = {}
    x = synth.make_activations(NB, K, seed=77) * (np.arange(NB, dtype=np.float32)[:, None] + 1)
    out["x"] = x
    out["xq"] = oracle.ref.quantize_q8k(x)
    xe = edge_activations()
    out["x_edge"] = xe
    out["xq_edge"] = oracle.ref.quantize_q8k(xe)
    assert np.array_equal(out["xq_edge"], oracle.ref.quantize_q8k(xe, avx2=True))
    for name, f in F.FORMATS.items():
        scale = 2e-4 if name == "IQ3_XXS" else 1e-3   # 2e-4 puts many fp16 scales into the subnormal range
        w = synth.make_weights(f, M, K, seed=1000 + f.type_id, scale=scale)
        out[f"w_{name}"] = w
        if name == "Q5_K":
            import gguf
            from gguf import quants
            out[f"dq_{name}"] = quants.dequantize(w, gguf.GGMLQuantizationType.Q5_K).astype(np.float32)
        else:
            out[f"dq_{name}"] = oracle.ref.dequantize(f.type_id, w, K)
        if oracle.ref.has_vec_dot(f.type_id):
            for nb in (1, 2, 3):
                y, _ = oracle.ref.gemv(f.type_id, w, out["xq"][:nb], K)
                out[f"y{nb}_{name}"] = y
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
