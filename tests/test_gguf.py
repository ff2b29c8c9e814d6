"""GGUF reader of the planner (qwengine_b200/csrc/q38b_gguf.cpp) against files written by gguf-py: tensor table, data
pointers, alignment key, and refusal of truncated or foreign files.  No GPU needed."""
import ctypes as C
import os

import numpy as np
import pytest

from qwengine_b200 import formats as F, synth

gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def lib():
    from qwengine_b200 import build, load_library
    build.build()
    l = load_library()
    l.q38b_gguf_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    l.q38b_gguf_close.argtypes = [C.c_void_p]
    l.q38b_gguf_tensor_count.argtypes = [C.c_void_p]
    l.q38b_gguf_find.argtypes = [C.c_void_p, C.c_char_p]
    l.q38b_gguf_tensor.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), C.POINTER(C.c_int),
                                   C.POINTER(C.c_longlong * 4), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
    return l


def write_model(path, alignment=None):
    w = gguf.GGUFWriter(path, "qwen35")
    w.add_string("general.name", "synthetic")
    w.add_uint32("qwen35.block_count", 2)
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_array("some.ints", [1, 2, 3, 4])
    if alignment:
        w.add_custom_alignment(alignment)
    tensors = {}
    for i, (name, fmt, M, K) in enumerate([("blk.0.ffn_gate.weight", "IQ3_XXS", 24, 1024), ("blk.0.ffn_down.weight", "IQ4_XS", 16, 512),
                                           ("blk.0.attn_q.weight", "Q4_K", 8, 256), ("output.weight", "Q6_K", 40, 256)]):
        f = F.get(fmt)
        data = synth.make_weights(f, M, K, seed=50 + i)
        tensors[name] = (f, M, K, data)
        w.add_tensor(name, data, raw_shape=data.shape, raw_dtype=gguf.GGMLQuantizationType(f.type_id))
    norm = np.arange(256, dtype=np.float32)
    w.add_tensor("output_norm.weight", norm)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors, norm


def read_all(lib, path):
    h = C.c_void_p()
    rc = lib.q38b_gguf_open(path.encode(), C.byref(h))
    if rc != 0:
        return rc, None
    out = {}
    for i in range(lib.q38b_gguf_tensor_count(h)):
        name, typ, nd, dims, data, nbytes = C.c_char_p(), C.c_uint32(), C.c_int(), (C.c_longlong * 4)(), C.c_void_p(), C.c_size_t()
        assert lib.q38b_gguf_tensor(h, i, C.byref(name), C.byref(typ), C.byref(nd), C.byref(dims), C.byref(data), C.byref(nbytes)) == 0
        raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nbytes.value,)).copy()
        out[name.value.decode()] = (typ.value, nd.value, list(dims), raw, data.value)
        assert lib.q38b_gguf_find(h, name.value) == i
    assert lib.q38b_gguf_find(h, b"no.such.tensor") == -1
    lib.q38b_gguf_close(h)
    return 0, out


@pytest.mark.parametrize("alignment", [None, 64])
def test_tensor_table_and_data(lib, tmp_path, alignment):
    path = str(tmp_path / "m.gguf")
    tensors, norm = write_model(path, alignment)
    rc, got = read_all(lib, path)
    assert rc == 0 and len(got) == len(tensors) + 1
    for name, (f, M, K, data) in tensors.items():
        typ, nd, dims, raw, _ = got[name]
        assert typ == f.type_id and nd == 2 and dims[:2] == [K, M]       # GGUF stores the row length first
        assert np.array_equal(raw, data.reshape(-1))
    typ, nd, dims, raw, _ = got["output_norm.weight"]
    assert typ == 0 and nd == 1 and dims[0] == 256 and np.array_equal(raw.view(np.float32), norm)


def test_rejects_foreign_and_truncated_files(lib, tmp_path):
    path = str(tmp_path / "m.gguf")
    write_model(path)
    blob = open(path, "rb").read()
    bad = str(tmp_path / "bad.gguf")
    h = C.c_void_p()
    open(bad, "wb").write(b"NOPE" + blob[4:])
    assert lib.q38b_gguf_open(bad.encode(), C.byref(h)) == -2            # Q38B_ERR_UNSUPPORTED: not a GGUF file
    for cut in (30, 200, len(blob) // 2, len(blob) - 1):                  # inside the header, the tables, the data
        open(bad, "wb").write(blob[:cut])
        assert lib.q38b_gguf_open(bad.encode(), C.byref(h)) != 0, cut
    open(bad, "wb").write(blob[:8] + (2 ** 60).to_bytes(8, "little") + blob[16:])   # absurd tensor count
    assert lib.q38b_gguf_open(bad.encode(), C.byref(h)) != 0
    assert lib.q38b_gguf_open(str(tmp_path / "missing.gguf").encode(), C.byref(h)) != 0
