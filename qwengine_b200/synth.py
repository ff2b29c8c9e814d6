"""Seeded synthetic GGUF blocks and activations.

The reference measures on tensors of a real model file, which is not available here; these
generators stand in for it.  Quant bytes are uniform over 0..255, which is a valid block for every
format of the path and exercises every codebook entry, sign pattern and sub-block scale; the fp16
super-block scales are |N(0,1)| * scale so that outputs stay O(1).
"""
import numpy as np

from . import formats as F

# byte offsets of the fp16 fields inside one block
_FP16_FIELDS = {
    "Q8_0": (0,), "Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,),
    "IQ3_XXS": (0,), "IQ3_S": (0,), "IQ4_XS": (0,),
    "Q2_K": (80, 82), "IQ2_XXS": (0,), "IQ2_XS": (0,), "IQ2_S": (0,), "IQ1_S": (0,), "IQ1_M": (),
}


# Q4_K / Q5_K weights are d*sc*q - dmin*m with unsigned q, sc, m: with dmin = ZERO_MEAN_DMIN * d their mean over
# uniformly random quants is zero, which keeps a chain of matvecs from amplifying the mean of its input.
ZERO_MEAN_DMIN = {"Q4_K": 7.5, "Q5_K": 15.5}


def make_weights(fmt, M: int, K: int, seed: int, scale: float = 1e-3, zero_mean: bool = False) -> np.ndarray:
    """Returns a uint8 array [M, row_bytes] of random valid blocks."""
    f = F.get(fmt)
    rng = np.random.Generator(np.random.PCG64(seed))
    nblk = K // f.block_elems
    w = rng.integers(0, 256, size=(M, nblk, f.block_bytes), dtype=np.uint8)
    for off in _FP16_FIELDS[f.name]:
        d = (np.abs(rng.standard_normal((M, nblk), dtype=np.float32)) * np.float32(scale)).astype(np.float16)
        if zero_mean and off == 2 and f.name in ZERO_MEAN_DMIN:
            d0 = w[:, :, 0:2].copy().view(np.float16).reshape(M, nblk).astype(np.float32)
            d = (d0 * np.float32(ZERO_MEAN_DMIN[f.name])).astype(np.float16)
        w[:, :, off:off + 2] = d.view(np.uint8).reshape(M, nblk, 2)
    if f.name == "IQ1_M":
        # the fp16 super-scale is scattered over the top nibbles of the four 16-bit scale words (bytes 48..55)
        bits = (np.abs(rng.standard_normal((M, nblk), dtype=np.float32)) * np.float32(scale)).astype(np.float16).view(np.uint16)
        for k in range(4):
            hi = w[:, :, 49 + 2 * k]
            w[:, :, 49 + 2 * k] = (hi & 0x0F) | ((((bits >> (4 * k)) & 0xF) << 4).astype(np.uint8))
    return w.reshape(M, nblk * f.block_bytes)


def make_activations(nb: int, K: int, seed: int) -> np.ndarray:
    """fp32 [nb, K], elements N(0,1)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((nb, K), dtype=np.float32)
