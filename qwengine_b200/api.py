"""ctypes binding of the C ABI (include/q38b200.h) for torch CUDA tensors.

Mirrors the reference's CUDA-side interface for this path (src/cuda/gemv.cuh:14-37,
src/cuda/prefill.cuh:17-28): weights are uint8 tensors holding GGUF blocks row by row, outputs are
``y[c, r]`` (column-major in the reference's sense: column c at ``y + c * y_ld``).
"""
import ctypes as C
import os

import torch

from . import formats as F

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OUT_F32, OUT_F16, OUT_BF16 = 0, 1, 2
_OUT_DTYPES = {OUT_F32: torch.float32, OUT_F16: torch.float16, OUT_BF16: torch.bfloat16}


class Q38BError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} ({status})")


def library_path():
    return os.path.join(_HERE, "libq38b200.so")


def load_library():
    """Loads libq38b200.so; raises if it has not been built (there is no fallback path)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m qwengine_b200.build` (needs nvcc)")
    lib = C.CDLL(path)
    vp, ll, i32, u32, sz = C.c_void_p, C.c_longlong, C.c_int, C.c_uint32, C.c_size_t
    lib.q38b_ctx_create.argtypes = [i32, C.POINTER(vp)]
    lib.q38b_ctx_destroy.argtypes = [vp]
    lib.q38b_ctx_destroy.restype = None
    lib.q38b_ctx_check.argtypes = [vp, vp]
    lib.q38b_last_cuda_error.argtypes = [vp]
    lib.q38b_ctx_set_pdl.argtypes = [vp, i32]
    lib.q38b_ctx_set_uniform_columns.argtypes = [vp, i32]
    lib.q38b_ctx_set_static_weights.argtypes = [vp, i32]
    lib.q38b_status_string.argtypes = [i32]
    lib.q38b_status_string.restype = C.c_char_p
    lib.q38b_format_supported.argtypes = [u32]
    lib.q38b_row_bytes.argtypes = [u32, i32]
    lib.q38b_row_bytes.restype = sz
    lib.q38b_q8k_bytes.argtypes = [i32]
    lib.q38b_q8k_bytes.restype = sz
    lib.q38b_quantize_q8k.argtypes = [vp, vp, ll, i32, i32, vp, ll, vp]
    lib.q38b_gemv_q8k.argtypes = [vp, u32, vp, sz, i32, i32, vp, ll, i32, vp, ll, i32, vp]
    lib.q38b_swiglu_q8k.argtypes = [vp, vp, vp, ll, i32, i32, vp, vp, ll, vp]
    lib.q38b_dequant_rows.argtypes = [vp, u32, vp, sz, i32, i32, vp, i32, vp]
    lib.q38b_gemv_f32.argtypes = [vp, u32, vp, sz, i32, i32, vp, ll, i32, vp, ll, i32, vp, sz, vp]
    lib.q38b_gemv_f32_static.argtypes = [vp, u32, vp, sz, i32, i32, vp, ll, i32, vp, ll, i32, vp]
    lib.q38b_gemv_f32_static_capacity.restype = sz
    lib.q38b_gemm_prefill.argtypes = [vp, u32, vp, sz, i32, i32, vp, ll, i32, vp, ll, i32, vp]
    lib.q38b_gemm_prefill_f16.argtypes = [vp, u32, vp, sz, i32, i32, vp, ll, i32, vp, ll, i32, vp]
    lib.q38b_comm_unique_id.argtypes = [vp]
    lib.q38b_comm_init.argtypes = [vp, i32, i32, vp]
    lib.q38b_peer_arena_create.argtypes = [vp, sz, vp]
    lib.q38b_peer_connect.argtypes = [vp, i32, i32, vp]
    lib.q38b_peer_barrier.argtypes = [vp, vp]
    lib.q38b_pass_op_barrier.argtypes = [vp]
    lib.q38b_pass_set_peer_store.argtypes = [vp, i32]
    lib.q38b_pass_create.argtypes = [vp, i32, C.POINTER(vp)]
    lib.q38b_pass_destroy.argtypes = [vp]
    lib.q38b_pass_destroy.restype = None
    lib.q38b_pass_buffer_f32.argtypes = [vp, i32]
    lib.q38b_pass_buffer_q8k.argtypes = [vp, i32]
    lib.q38b_pass_buffer_ptr.argtypes = [vp, i32]
    lib.q38b_pass_buffer_ptr.restype = vp
    lib.q38b_pass_matrix_upload.argtypes = [vp, u32, vp, sz, i32, i32, i32, i32]
    lib.q38b_pass_matrix_device.argtypes = [vp, u32, vp, sz, i32, i32]
    lib.q38b_pass_op_quantize.argtypes = [vp, i32, i32, i32, i32]
    lib.q38b_pass_op_gemv.argtypes = [vp, i32, i32, i32, i32]
    lib.q38b_pass_op_gemv_local.argtypes = [vp, i32, i32, i32, i32]
    lib.q38b_pass_op_swiglu.argtypes = [vp, i32, i32, i32, i32, i32, i32]
    lib.q38b_pass_op_allgather.argtypes = [vp, i32, i32, i32]
    lib.q38b_pass_run.argtypes = [vp, i32, vp]
    lib.q38b_pass_run_host.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, i32, vp]
    lib.q38b_pass_weight_bytes.argtypes = [vp]
    lib.q38b_pass_weight_bytes.restype = ll
    lib.q38b_pass_kernel_count.argtypes = [vp]
    lib.q38b_pass_set_merge.argtypes = [vp, i32]
    lib.q38b_add_rmsnorm_q8k.argtypes = [vp, vp, vp, vp, vp, i32, ll, i32, C.c_float, vp, vp, ll, vp]
    lib.q38b_gemv_bf16.argtypes = [vp, vp, i32, i32, vp, vp, vp]
    lib.q38b_swiglu_rows_inplace.argtypes = [vp, vp, vp, i32, i32, ll, i32, vp]
    lib.q38b_topk.argtypes = [vp, vp, ll, i32, i32, i32, i32, vp, vp, i32, vp]
    lib.q38b_pass_op_topk.argtypes = [vp, i32, i32, i32, i32, i32]
    lib.q38b_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.q38b_gguf_close.argtypes = [vp]
    lib.q38b_gguf_find.argtypes = [vp, C.c_char_p]
    lib.q38b_pass_matrix_from_gguf.argtypes = [vp, vp, i32, i32, i32]
    lib.q38b_ctx_set_wait_budget_cycles.argtypes = [vp, ll]
    lib.q38b_debug_fake_silent_peer.argtypes = [vp, i32]
    lib.q38b_quantize_act_q8.argtypes = [vp, vp, i32, i32, vp, vp, vp, vp]
    lib.q38b_gemv_act_q8.argtypes = [vp, u32, vp, sz, i32, i32, vp, vp, i32, i32, vp, i32, i32, vp]
    lib.q38b_debug_set_rowgroup.argtypes = [vp, i32]
    lib.q38b_debug_occupancy_shortfalls.argtypes = [vp, i32]
    lib.q38b_debug_set_one_cta.argtypes = [vp, i32]
    lib.q38b_debug_set_gemv_part_items.argtypes = [vp, ll]
    lib.q38b_gemv_group.argtypes = [vp, u32, i32, vp, sz, i32, vp, vp, vp, vp, vp]
    _LIB = lib
    return lib


def status_string(status):
    return load_library().q38b_status_string(int(status)).decode()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Context:
    """One per process and GPU (q38b_ctx)."""

    def __init__(self, device=0):
        self.lib = load_library()
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library has no CPU path")
        self.device = torch.device("cuda", device)
        h = C.c_void_p()
        rc = self.lib.q38b_ctx_create(device, C.byref(h))
        if rc:
            raise Q38BError(rc, "q38b_ctx_create")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.q38b_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _rc(self, rc, what):
        if rc:
            if rc == -4:
                what += f" [cudaError {self.lib.q38b_last_cuda_error(self.h)}]"
            raise Q38BError(rc, what)

    def check(self):
        """Synchronises the current stream and raises if a kernel reported a bounded wait that ran out."""
        self._rc(self.lib.q38b_ctx_check(self.h, _stream()), "q38b_ctx_check")

    def peer_arena_create(self, nbytes=256 << 20):
        """Allocates this rank's peer-visible arena; returns its 64-byte CUDA IPC handle."""
        raw = (C.c_ubyte * 64)()
        self._rc(self.lib.q38b_peer_arena_create(self.h, nbytes, raw), "q38b_peer_arena_create")
        return bytes(raw)

    def peer_connect(self, n_ranks, rank, handles):
        self._rc(self.lib.q38b_peer_connect(self.h, n_ranks, rank, b"".join(handles)), "q38b_peer_connect")

    def set_static_weights(self, enabled):
        self._rc(self.lib.q38b_ctx_set_static_weights(self.h, int(bool(enabled))), "q38b_ctx_set_static_weights")

    def set_uniform_columns(self, enabled):
        self._rc(self.lib.q38b_ctx_set_uniform_columns(self.h, int(bool(enabled))), "q38b_ctx_set_uniform_columns")

    def debug_set_rowgroup(self, enabled):
        """Test hook: enabled=False keeps the one-column kernel on its lane-per-granule mapping for every format."""
        self._rc(self.lib.q38b_debug_set_rowgroup(self.h, int(bool(enabled))), "q38b_debug_set_rowgroup")

    def debug_set_one_cta(self, mode):
        """Test hook: one CTA per SM for the one-column kernel: 0 never, otherwise wherever such a plan fits (default)."""
        self._rc(self.lib.q38b_debug_set_one_cta(self.h, int(mode)), "q38b_debug_set_one_cta")

    def debug_set_gemv_part_items(self, items):
        """Test hook: the multi-column kernel's K-part scratch area counts as `items` (tile, part) sums (0: its real size)."""
        self._rc(self.lib.q38b_debug_set_gemv_part_items(self.h, int(items)), "q38b_debug_set_gemv_part_items")

    def set_wait_budget_cycles(self, cycles):
        self._rc(self.lib.q38b_ctx_set_wait_budget_cycles(self.h, int(cycles)), "q38b_ctx_set_wait_budget_cycles")

    def set_pdl(self, enabled):
        self._rc(self.lib.q38b_ctx_set_pdl(self.h, int(bool(enabled))), "q38b_ctx_set_pdl")

    # ---- activations -------------------------------------------------------------------------
    def quantize_q8k(self, x, out=None):
        """x float32 [nb, K] (row stride = x.stride(0)) -> uint8 [nb, K/256*292] of Q8_K blocks."""
        assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
        nb, K = x.shape
        if out is None:
            out = torch.empty((nb, K // 256 * F.Q8K_BLOCK_BYTES), dtype=torch.uint8, device=x.device)
        self._rc(self.lib.q38b_quantize_q8k(self.h, x.data_ptr(), x.stride(0), K, nb, out.data_ptr(),
                                            out.stride(0) // F.Q8K_BLOCK_BYTES, _stream()), "q38b_quantize_q8k")
        return out

    def swiglu_q8k(self, g, u, want_h=True, want_q=True):
        """h = silu(g) * u for float32 [nb, n]; returns (h or None, q8k blocks or None)."""
        assert g.shape == u.shape and g.stride() == u.stride() and g.stride(1) == 1
        nb, n = g.shape
        h = torch.empty_like(g) if want_h else None
        q = torch.empty((nb, n // 256 * F.Q8K_BLOCK_BYTES), dtype=torch.uint8, device=g.device) if want_q else None
        if h is not None:
            assert h.stride() == g.stride()
        self._rc(self.lib.q38b_swiglu_q8k(self.h, g.data_ptr(), u.data_ptr(), g.stride(0), n, nb,
                                          h.data_ptr() if h is not None else None,
                                          q.data_ptr() if q is not None else None,
                                          (q.stride(0) // F.Q8K_BLOCK_BYTES) if q is not None else 0, _stream()),
                 "q38b_swiglu_q8k")
        return h, q

    # ---- matvec ------------------------------------------------------------------------------
    def gemv(self, fmt, W, xq, K, out=None, accumulate=False, M=None):
        """W uint8 [M, row_bytes]; xq uint8 [nb, K/256*292]; returns y float32 [nb, M] (y[c, r])."""
        f = F.get(fmt)
        assert W.is_cuda and W.dtype == torch.uint8 and W.dim() == 2 and W.stride(1) == 1
        M = W.shape[0] if M is None else M
        nb = xq.shape[0]
        if out is None:
            out = torch.empty((nb, M), dtype=torch.float32, device=W.device)
        self._rc(self.lib.q38b_gemv_q8k(self.h, f.type_id, W.data_ptr(), W.stride(0), K, M, xq.data_ptr(),
                                        xq.stride(0) // F.Q8K_BLOCK_BYTES, nb, out.data_ptr(), out.stride(0),
                                        int(bool(accumulate)), _stream()), "q38b_gemv_q8k")
        return out

    def quantize_act_q8(self, x):
        """x float32 [n_rows, K] -> (q int8 [n_rows, K], d float32 [n_rows, K/32], s float32 [n_rows, K/32]): the per-32
        activation format of the reference GPU path."""
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        n, K = x.shape
        q = torch.empty((n, K), dtype=torch.int8, device=x.device)
        d = torch.empty((n, K // 32), dtype=torch.float32, device=x.device)
        s = torch.empty_like(d)
        self._rc(self.lib.q38b_quantize_act_q8(self.h, x.data_ptr(), K, n, q.data_ptr(), d.data_ptr(), s.data_ptr(), _stream()),
                 "q38b_quantize_act_q8")
        return q, d, s

    def gemv_act_q8(self, fmt, W, q, d, K, out=None, accumulate=False):
        """W uint8 [M, row_bytes]; q int8 [nb, K], d float32 [nb, K/32] (contiguous); returns y float32 [nb, M]."""
        f = F.get(fmt)
        M, nb = W.shape[0], q.shape[0]
        if out is None:
            out = torch.empty((nb, M), dtype=torch.float32, device=W.device)
        self._rc(self.lib.q38b_gemv_act_q8(self.h, f.type_id, W.data_ptr(), W.stride(0), K, M, q.data_ptr(), d.data_ptr(), nb,
                                           q.stride(0), out.data_ptr(), out.stride(0), int(bool(accumulate)), _stream()),
                 "q38b_gemv_act_q8")
        return out

    def add_rmsnorm_q8k(self, x, w, a=None, b=None, eps=1e-6, want_xn=True):
        """x float32 [rows, n] (updated in place when a or b is given); returns (xn float32 or None, q8k uint8 [rows, n/256*292])."""
        rows, n = x.shape
        xn = torch.empty_like(x) if want_xn else None
        q8 = torch.empty((rows, n // 256 * F.Q8K_BLOCK_BYTES), dtype=torch.uint8, device=x.device)
        ptr = lambda t: t.data_ptr() if t is not None else None
        self._rc(self.lib.q38b_add_rmsnorm_q8k(self.h, x.data_ptr(), ptr(a), ptr(b), w.data_ptr(), n, x.stride(0), rows, eps, ptr(xn),
                                               q8.data_ptr(), n // 256, _stream()), "q38b_add_rmsnorm_q8k")
        return xn, q8

    def gemv_bf16(self, W, x):
        """W bfloat16 [N, K], x float32 [K] -> y float32 [N]."""
        N, K = W.shape
        y = torch.empty(N, dtype=torch.float32, device=W.device)
        self._rc(self.lib.q38b_gemv_bf16(self.h, W.data_ptr(), K, N, x.data_ptr(), y.data_ptr(), _stream()), "q38b_gemv_bf16")
        return y

    def topk(self, logits, k, index_offset=0):
        """The k largest of each row of `logits` [rows, n] (fp32, device): (values [rows, k], positions [rows, k] int32)."""
        rows, n = logits.shape
        vals = torch.empty((rows, k), dtype=torch.float32, device=logits.device)
        idx = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
        self._rc(self.lib.q38b_topk(self.h, logits.data_ptr(), logits.stride(0), n, rows, k, index_offset, vals.data_ptr(),
                                    idx.data_ptr(), k, _stream()), "q38b_topk")
        return vals, idx

    def swiglu_rows_inplace(self, G, U, n, kind):
        """G, U float32 [B, ld]; writes silu(G[:, :n]) * U[:, :n] over the start of every row of G as 16-bit floats."""
        self._rc(self.lib.q38b_swiglu_rows_inplace(self.h, G.data_ptr(), U.data_ptr(), G.shape[0], n, G.stride(0), kind, _stream()),
                 "q38b_swiglu_rows_inplace")

    def gemv_group(self, fmt, Ws, K, xq=None, x_f32=None):
        """q38b_gemv_group: up to three matrices [M_i, row_bytes] of one format on one column, given as Q8_K blocks
        (xq uint8 [1, K/256*292]) or as floats (x_f32 [K] or [1, K]); returns the list of y_i float32 [M_i]."""
        import ctypes
        f = F.get(fmt)
        n = len(Ws)
        outs = [torch.empty(w.shape[0], dtype=torch.float32, device=w.device) for w in Ws]
        Wp = (ctypes.c_void_p * n)(*[w.data_ptr() for w in Ws])
        yp = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
        Ms = (ctypes.c_int * n)(*[w.shape[0] for w in Ws])
        self._rc(self.lib.q38b_gemv_group(self.h, f.type_id, n, Wp, Ws[0].stride(0), K, Ms, xq.data_ptr() if xq is not None else None,
                                          x_f32.data_ptr() if x_f32 is not None else None, yp, _stream()), "q38b_gemv_group")
        return outs

    def gemv_f32(self, fmt, W, x, K, scratch=None, out=None, accumulate=False):
        """Matvec from fp32 activations x [nb, K]; `scratch` is a uint8 device tensor for the Q8_K blocks."""
        f = F.get(fmt)
        nb, M = x.shape[0], W.shape[0]
        if scratch is None:
            scratch = torch.empty(nb * (K // 256) * F.Q8K_BLOCK_BYTES, dtype=torch.uint8, device=W.device)
        if out is None:
            out = torch.empty((nb, M), dtype=torch.float32, device=W.device)
        self._rc(self.lib.q38b_gemv_f32(self.h, f.type_id, W.data_ptr(), W.stride(0), K, M, x.data_ptr(), x.stride(0), nb,
                                        out.data_ptr(), out.stride(0), int(bool(accumulate)), scratch.data_ptr(), scratch.numel(),
                                        _stream()), "q38b_gemv_f32")
        return out

    def gemv_f32_static(self, fmt, W, x, K, out=None, accumulate=False):
        """q38b_gemv_f32_static: like gemv_f32 but the Q8_K scratch is the library's built-in array (no allocation)."""
        f = F.get(fmt)
        nb, M = x.shape[0], W.shape[0]
        assert out is not None, "the caller brings the output buffer: this path allocates nothing"
        self._rc(self.lib.q38b_gemv_f32_static(self.h, f.type_id, W.data_ptr(), W.stride(0), K, M, x.data_ptr(), x.stride(0), nb,
                                               out.data_ptr(), out.stride(0), int(bool(accumulate)), _stream()),
                 "q38b_gemv_f32_static")
        return out

    def gemv_raw(self, type_id, W_ptr, row_bytes, K, M, xq_ptr, x_stride, nb, y_ptr, y_ld, accumulate=0):
        """Unchecked pass-through to q38b_gemv_q8k; returns the status code."""
        return self.lib.q38b_gemv_q8k(self.h, type_id, W_ptr, row_bytes, K, M, xq_ptr, x_stride, nb, y_ptr, y_ld,
                                      accumulate, _stream())

    def gemm_prefill(self, fmt, W, X, K, out=None, accumulate=False):
        """W uint8 [M, row_bytes]; X bfloat16 or float16 [B, K] (the operand type of the tensor-core product follows X);
        returns Y float32 [B, M] = X @ dequant(W)^T."""
        f = F.get(fmt)
        assert X.dtype in (torch.bfloat16, torch.float16) and X.stride(1) == 1
        M, B = W.shape[0], X.shape[0]
        if out is None:
            out = torch.empty((B, M), dtype=torch.float32, device=W.device)
        fn = self.lib.q38b_gemm_prefill if X.dtype == torch.bfloat16 else self.lib.q38b_gemm_prefill_f16
        self._rc(fn(self.h, f.type_id, W.data_ptr(), W.stride(0), K, M, X.data_ptr(), X.stride(0), B,
                    out.data_ptr(), out.stride(0), int(bool(accumulate)), _stream()), "q38b_gemm_prefill")
        return out

    def dequant_rows(self, fmt, W, K, kind=OUT_F32):
        f = F.get(fmt)
        rows = W.shape[0]
        out = torch.empty((rows, K), dtype=_OUT_DTYPES[kind], device=W.device)
        self._rc(self.lib.q38b_dequant_rows(self.h, f.type_id, W.data_ptr(), W.stride(0), K, rows, out.data_ptr(), kind,
                                            _stream()), "q38b_dequant_rows")
        return out


class Pass:
    """Recorded decode pass over resident matrices (q38b_pass): the all-HBM planner's run-time object."""

    def __init__(self, ctx, max_nb=1):
        self.ctx, self.lib, self.max_nb = ctx, ctx.lib, max_nb
        h = C.c_void_p()
        ctx._rc(self.lib.q38b_pass_create(ctx.h, max_nb, C.byref(h)), "q38b_pass_create")
        self.h = h
        self._keep = []          # device tensors adopted with matrix_device stay alive with the pass
        self._sizes = {}

    def close(self):
        if getattr(self, "h", None):
            self.lib.q38b_pass_destroy(self.h)
            self.h = None

    def _id(self, rc, what):
        if rc < 0:
            raise Q38BError(rc, what)
        return rc

    def buffer_f32(self, n):
        i = self._id(self.lib.q38b_pass_buffer_f32(self.h, n), "q38b_pass_buffer_f32")
        self._sizes[i] = n
        return i

    def buffer_q8k(self, K):
        return self._id(self.lib.q38b_pass_buffer_q8k(self.h, K), "q38b_pass_buffer_q8k")

    def buffer_tensor(self, buf):
        """A torch view [max_nb, n] of an fp32 buffer of the pass (no copy)."""
        n = self._sizes[buf]
        ptr = self.lib.q38b_pass_buffer_ptr(self.h, buf)
        return _tensor_from_ptr(ptr, (self.max_nb, n), self.ctx.device)

    def matrix_upload(self, fmt, w_host, K, shard=0, n_shards=1):
        """w_host: numpy uint8 [M, row_bytes] in host memory; uploads rows of this shard."""
        f = F.get(fmt)
        M, rb = w_host.shape
        return self._id(self.lib.q38b_pass_matrix_upload(self.h, f.type_id, w_host.ctypes.data, rb, K, M, shard, n_shards),
                        "q38b_pass_matrix_upload")

    def matrix_from_gguf(self, gguf_file, name, shard=0, n_shards=1):
        """Uploads this rank's rows of the named 2-D tensor of an open GGUF file (GgufFile); returns the matrix id."""
        idx = self.lib.q38b_gguf_find(gguf_file.h, name.encode())
        if idx < 0:
            raise KeyError(name)
        return self._id(self.lib.q38b_pass_matrix_from_gguf(self.h, gguf_file.h, idx, shard, n_shards), "q38b_pass_matrix_from_gguf")

    def matrix_device(self, fmt, W, K):
        f = F.get(fmt)
        self._keep.append(W)
        return self._id(self.lib.q38b_pass_matrix_device(self.h, f.type_id, W.data_ptr(), W.stride(0), K, W.shape[0]),
                        "q38b_pass_matrix_device")

    def quantize(self, src, off, K, dst):
        self.ctx._rc(self.lib.q38b_pass_op_quantize(self.h, src, off, K, dst), "q38b_pass_op_quantize")

    def gemv(self, mat, src_q, dst, off=0, local=False):
        """local=True: the output is not pushed to the peers (a matrix every rank holds whole)."""
        fn = self.lib.q38b_pass_op_gemv_local if local else self.lib.q38b_pass_op_gemv
        self.ctx._rc(fn(self.h, mat, src_q, dst, off), "q38b_pass_op_gemv")

    def swiglu(self, g, g_off, u, u_off, n, dst_q):
        self.ctx._rc(self.lib.q38b_pass_op_swiglu(self.h, g, g_off, u, u_off, n, dst_q), "q38b_pass_op_swiglu")

    def set_peer_store(self, enabled):
        self.ctx._rc(self.lib.q38b_pass_set_peer_store(self.h, int(bool(enabled))), "q38b_pass_set_peer_store")

    def set_merge(self, enabled):
        """enabled=False: single-column runs launch one kernel per recorded step (no shared launches, no folded quantize)."""
        self.ctx._rc(self.lib.q38b_pass_set_merge(self.h, int(bool(enabled))), "q38b_pass_set_merge")

    def topk(self, src, off, n, k, dst):
        self.ctx._rc(self.lib.q38b_pass_op_topk(self.h, src, off, n, k, dst), "q38b_pass_op_topk")

    def barrier(self):
        self.ctx._rc(self.lib.q38b_pass_op_barrier(self.h), "q38b_pass_op_barrier")

    def allgather(self, buf, off, count):
        self.ctx._rc(self.lib.q38b_pass_op_allgather(self.h, buf, off, count), "q38b_pass_op_allgather")

    def run(self, nb=1):
        self.ctx._rc(self.lib.q38b_pass_run(self.h, nb, _stream()), "q38b_pass_run")

    def run_host(self, nb, in_buf, x_host, out_buf, out_off, y_host):
        """x_host, y_host: C-contiguous numpy float32 [nb, len]; host to device and back inside the call."""
        self.ctx._rc(self.lib.q38b_pass_run_host(self.h, nb, in_buf, x_host.ctypes.data, x_host.shape[1], out_buf, out_off,
                                                 y_host.ctypes.data, y_host.shape[1], _stream()), "q38b_pass_run_host")

    @property
    def weight_bytes(self):
        return int(self.lib.q38b_pass_weight_bytes(self.h))

    @property
    def kernel_count(self):
        return int(self.lib.q38b_pass_kernel_count(self.h))


class GgufFile:
    """A memory-mapped GGUF model file (q38b_gguf_open)."""

    def __init__(self, path):
        import ctypes
        self.lib = load_library()
        self.h = ctypes.c_void_p()
        rc = self.lib.q38b_gguf_open(str(path).encode(), ctypes.byref(self.h))
        if rc != 0:
            raise Q38BError(rc, "q38b_gguf_open")

    def close(self):
        if self.h:
            self.lib.q38b_gguf_close(self.h)
            self.h = None


def _tensor_from_ptr(ptr, shape, device):
    """Wraps device memory owned by the library as a float32 torch tensor (via __cuda_array_interface__)."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 2}
    return torch.as_tensor(h, device=device)
