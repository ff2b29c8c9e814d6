"""The C-ABI library loads without a GPU and exports every symbol include/q38b200.h declares."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from qwengine_b200 import build, load_library
    build.build()
    return load_library()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "q38b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q38b_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/q38b200.h but not exported"


def test_format_table(lib):
    from qwengine_b200 import formats as F
    for f in F.FORMATS.values():
        assert lib.q38b_format_supported(f.type_id) == 1
        for K in (256, 5120, 6144, 17408):
            assert lib.q38b_row_bytes(f.type_id, K) == f.row_bytes(K)
    for f in F.ONE_COLUMN.values():
        assert lib.q38b_format_supported(f.type_id) == 1
        assert lib.q38b_row_bytes(f.type_id, 5120) == f.row_bytes(5120)
    for unsupported in (0, 1, 2, 3, 11, 20, 30):   # F32, F16, Q4_0, Q4_1, Q3_K, IQ4_NL, BF16
        assert lib.q38b_format_supported(unsupported) == 0
        assert lib.q38b_row_bytes(unsupported, 5120) == 0
    assert lib.q38b_row_bytes(18, 5000) == 0
    assert lib.q38b_q8k_bytes(5120) == 20 * 292


def test_status_strings(lib):
    for s in range(0, -8, -1):
        assert lib.q38b_status_string(s)


def test_no_gpu_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.q38b_ctx_create(0, C.byref(h)) == -7   # Q38B_ERR_NO_DEVICE
    assert not h.value
    import qwengine_b200 as q
    with pytest.raises(RuntimeError):
        q.Context(0)


def test_null_arguments_rejected(lib):
    assert lib.q38b_ctx_create(0, None) == -1
    assert lib.q38b_gemv_q8k(None, 18, None, 0, 0, 0, None, 0, 0, None, 0, 0, None) == -1
    assert lib.q38b_ctx_check(None, None) == -1
