"""CPU checkers for the quantized matvec path -- TEST INFRASTRUCTURE, not product code.

``port``: this repository's plain-C restatement (oracle_port.c -> liboracle_port.so).
``ref`` : the reference's own sources compiled in place (oracle/_ref/libq38ref.so), or None when
          that library has not been built.
Only tests, the smoke check and the CPU-baseline leg of the benchmark import this package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
Q8K = 292

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def build():
    subprocess.run(["make", "-C", _HERE, "all"], check=True, stdout=subprocess.DEVNULL)


def _load(path):
    return C.CDLL(path) if os.path.exists(path) else None


class _Port:
    def __init__(self, lib):
        self.lib = lib
        lib.q38o_row_bytes.restype = C.c_size_t
        lib.q38o_row_bytes.argtypes = [C.c_uint32, C.c_int]
        lib.q38o_dequantize_row.argtypes = [C.c_uint32, _u8p, _f32p, C.c_int64]
        lib.q38o_quantize_row_q8_K.argtypes = [_f32p, _u8p, C.c_int64]
        lib.q38o_vec_dot_n.argtypes = [C.c_uint32, C.c_int, _u8p, _u8p, C.c_size_t, C.c_int, _f32p]
        lib.q38o_gemv.argtypes = [C.c_uint32, _u8p, C.c_size_t, C.c_int, C.c_int, _u8p, C.c_size_t, C.c_int, _f32p, C.c_int]
        lib.q38o_row_ref_mag.argtypes = [C.c_uint32, _u8p, C.c_size_t, C.c_int, C.c_int, _u8p, _f64p, _f64p]
        lib.q38o_swiglu.argtypes = [_f32p, _f32p, C.c_int, _f32p]
        lib.q38o_matmul_ref.argtypes = [C.c_uint32, _u8p, C.c_size_t, C.c_int, C.c_int, _f32p, C.c_int, C.c_int, _f64p, _f64p]
        lib.q38o_fp16_to_fp32.restype = C.c_float
        lib.q38o_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.q38o_fp32_to_fp16.restype = C.c_uint16
        lib.q38o_fp32_to_fp16.argtypes = [C.c_float]
        lib.q38o_fp32_to_bf16.restype = C.c_uint16
        lib.q38o_fp32_to_bf16.argtypes = [C.c_float]

    def dequantize(self, type_id, w):
        """w: uint8 [M, row_bytes] -> float32 [M, K]."""
        M, rb = w.shape
        K = rb * 256 // self.lib.q38o_row_bytes(type_id, 256)
        out = np.empty((M, K), np.float32)
        flat = np.ascontiguousarray(w).reshape(-1)
        if self.lib.q38o_dequantize_row(type_id, flat, out.reshape(-1), M * K):
            raise ValueError("unsupported format")
        return out

    def quantize_q8k(self, x):
        """x: float32 [nb, K] -> uint8 [nb, K/256*292]."""
        x = np.ascontiguousarray(x, np.float32)
        nb, K = x.shape
        out = np.zeros((nb, K // 256 * Q8K), np.uint8)
        self.lib.q38o_quantize_row_q8_K(x.reshape(-1), out.reshape(-1), nb * K)
        return out

    def gemv(self, type_id, w, xq, K):
        """w uint8 [M,row_bytes], xq uint8 [nb, K/256*292] -> y float32 [nb, M]."""
        M, rb = w.shape
        nb = xq.shape[0]
        y = np.zeros((nb, M), np.float32)
        rc = self.lib.q38o_gemv(type_id, np.ascontiguousarray(w).reshape(-1), rb, K, M,
                                np.ascontiguousarray(xq).reshape(-1), K // 256, nb, y.reshape(-1), M)
        if rc:
            raise ValueError("unsupported format")
        return y

    def row_ref_mag(self, type_id, w, xq_col, K):
        M, rb = w.shape
        ref = np.zeros(M, np.float64)
        mag = np.zeros(M, np.float64)
        self.lib.q38o_row_ref_mag(type_id, np.ascontiguousarray(w).reshape(-1), rb, K, M,
                                  np.ascontiguousarray(xq_col).reshape(-1), ref, mag)
        return ref, mag

    def swiglu(self, g, u):
        g = np.ascontiguousarray(g, np.float32).reshape(-1)
        u = np.ascontiguousarray(u, np.float32).reshape(-1)
        h = np.empty_like(g)
        self.lib.q38o_swiglu(g, u, g.size, h)
        return h

    def matmul_ref(self, type_id, w, X, K):
        """Y[B, M] (float64) and mag[B, M] for X float32 [B, K]."""
        M, rb = w.shape
        X = np.ascontiguousarray(X, np.float32)
        B = X.shape[0]
        Y = np.zeros((B, M), np.float64)
        mag = np.zeros((B, M), np.float64)
        self.lib.q38o_matmul_ref(type_id, np.ascontiguousarray(w).reshape(-1), rb, K, M, X.reshape(-1), X.shape[1], B,
                                 Y.reshape(-1), mag.reshape(-1))
        return Y, mag


class _Ref:
    def __init__(self, lib):
        self.lib = lib
        lib.q38ref_dequantize_row.argtypes = [C.c_uint32, _u8p, _f32p, C.c_int64]
        lib.q38ref_quantize_q8_K_scalar.argtypes = [_f32p, _u8p, C.c_int64]
        lib.q38ref_quantize_q8_K_avx2.argtypes = [_f32p, _u8p, C.c_int]
        lib.q38ref_has_vec_dot.argtypes = [C.c_uint32]
        lib.q38ref_vec_dot_n.argtypes = [C.c_uint32, C.c_int, _u8p, _u8p, C.c_size_t, C.c_int, _f32p]
        lib.q38ref_gemv.restype = C.c_double
        lib.q38ref_gemv.argtypes = [C.c_uint32, _u8p, C.c_size_t, C.c_int, C.c_int64, _u8p, C.c_size_t, C.c_int, _f32p,
                                    C.c_int64, C.c_int, C.c_int]
        lib.q38ref_fp16_to_fp32.restype = C.c_float
        lib.q38ref_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.q38ref_fp32_to_fp16.restype = C.c_uint16
        lib.q38ref_fp32_to_fp16.argtypes = [C.c_float]

    def has_vec_dot(self, type_id):
        return bool(self.lib.q38ref_has_vec_dot(type_id))

    def dequantize(self, type_id, w, K):
        M = w.shape[0]
        out = np.empty((M, K), np.float32)
        if self.lib.q38ref_dequantize_row(type_id, np.ascontiguousarray(w).reshape(-1), out.reshape(-1), M * K):
            raise ValueError("unsupported by the reference")
        return out

    def quantize_q8k(self, x, avx2=False):
        x = np.ascontiguousarray(x, np.float32)
        nb, K = x.shape
        out = np.zeros((nb, K // 256 * Q8K), np.uint8)
        for c in range(nb):
            if avx2:
                self.lib.q38ref_quantize_q8_K_avx2(x[c], out[c], K)
            else:
                self.lib.q38ref_quantize_q8_K_scalar(x[c], out[c], K)
        return out

    def gemv(self, type_id, w, xq, K, threads=1, reps=1):
        """Returns (y float32 [nb, M], seconds)."""
        M, rb = w.shape
        nb = xq.shape[0]
        y = np.zeros((nb, M), np.float32)
        sec = self.lib.q38ref_gemv(type_id, np.ascontiguousarray(w).reshape(-1), rb, K, M,
                                   np.ascontiguousarray(xq).reshape(-1), K // 256, nb, y.reshape(-1), M, threads, reps)
        if sec < 0:
            raise ValueError("no reference kernel for this format")
        return y, sec


def _get_port():
    p = os.path.join(_HERE, "liboracle_port.so")
    if not os.path.exists(p):
        build()
    return _Port(C.CDLL(p))


port = _get_port()
_ref_lib = _load(os.path.join(_HERE, "_ref", "libq38ref.so"))
ref = _Ref(_ref_lib) if _ref_lib is not None else None


# ---------------------------------------------------------------------------------------------------------------
# Per-32 activation format of the reference's GPU path (ActQ8: int8 q[K], float d[K/32], float s[K/32] = d * sum q),
# restated with numpy float32 arithmetic: src/cuda/gemv.cu:31-47 of the reference project (one warp per 32 values:
# d = amax / 127, q = round-half-even(v / d), zero block stays zero, s = d * (float) sum q).
# ---------------------------------------------------------------------------------------------------------------
def quantize_act_q8(x):
    """x float32 [n_rows, K] -> (q int8 [n_rows, K], d float32 [n_rows, K/32], s float32 [n_rows, K/32])."""
    x = np.ascontiguousarray(x, np.float32)
    n, K = x.shape
    v = x.reshape(n, K // 32, 32)
    amax = np.abs(v).max(axis=2)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        qf = np.rint((v / d[:, :, None]).astype(np.float32))
    qf = np.where(d[:, :, None] > 0, qf, np.float32(0))
    q = qf.astype(np.int8)
    s = (d * qf.sum(axis=2, dtype=np.float32)).astype(np.float32)
    return q.reshape(n, K), d, s


def act_q8_dequant(q, d):
    """The activations an ActQ8 row stands for: d[k / 32] * q[k], float32 [n_rows, K]."""
    n, K = q.shape
    return (q.reshape(n, K // 32, 32).astype(np.float32) * d[:, :, None]).reshape(n, K)


# ---------------------------------------------------------------------------------------------------------------
# top-k of the output head's logits (src/cuda/ops.cuh:142-144 of the reference project; its test orders by value
# descending, tests/kernels/test_ops.cu:425-447): values descending, equal values by ascending position, NaN last.
# ---------------------------------------------------------------------------------------------------------------
def topk(logits, k, index_offset=0):
    """logits float32 [rows, n] -> (values float32 [rows, k], positions int32 [rows, k]); slots past n: (NaN, -1)."""
    x = np.ascontiguousarray(logits, np.float32)
    rows, n = x.shape
    vals = np.full((rows, k), np.nan, np.float32)
    idx = np.full((rows, k), -1, np.int32)
    for r in range(rows):
        key = np.where(np.isnan(x[r]), -np.inf, x[r].astype(np.float64))
        nan_last = np.isnan(x[r]).astype(np.int8)
        order = np.lexsort((np.arange(n), -key, nan_last))[:k]   # last key is the primary one
        vals[r, :len(order)] = x[r, order]
        idx[r, :len(order)] = order + index_offset
    return vals, idx
