"""Launch planner of the recorded pass (q38b_plan.cu: merge_plan) on step lists, without a device: which steps share a
launch, and that the recorded order against cross-GPU barriers and all-gathers is kept on several ranks."""
import ctypes as C

import numpy as np
import pytest

Q, MV, SW, GA, BA = 0, 1, 2, 3, 4   # step kinds of the test hook


@pytest.fixture(scope="module")
def plan():
    from qwengine_b200 import build, load_library
    build.build()
    lib = load_library()
    i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
    lib.q38b_debug_merge_plan.argtypes = [C.c_int, C.c_int, C.c_int, i32p, i32p]

    def run(n_ranks, nb, steps):
        s = np.array(steps, np.int32).reshape(-1, 3)
        out = np.zeros(len(s), np.int32)
        n = lib.q38b_debug_merge_plan(n_ranks, nb, len(s), s, out)
        assert n >= 0
        return n, out.tolist()
    return run


def test_quantize_folds_and_column_mates_share_a_launch(plan):
    steps = [(Q, 4, 0), (MV, 4, 0), (MV, 4, 512), (MV, 4, 1024), (SW, 5, 0), (MV, 5, 2048)]
    n, where = plan(1, 1, steps)
    assert n == 1 and where == [-1, 1, 1, 1, 4, 5]


def test_single_rank_steps_over_barriers(plan):
    """On one GPU a barrier does nothing, so matvecs on one column merge across it."""
    n, where = plan(1, 1, [(MV, 4, 0), (BA, 0, 0), (MV, 4, 512)])
    assert n == 1 and where == [0, 1, 0]


def test_barrier_is_a_hard_cut_on_several_ranks(plan):
    """A matvec recorded after a cross-GPU barrier must not be launched (and push to the peers) before it."""
    n, where = plan(2, 1, [(MV, 4, 0), (BA, 0, 0), (MV, 4, 512)])
    assert n == 0 and where == [0, 1, 2]
    n, where = plan(2, 1, [(Q, 4, 0), (BA, 0, 0), (MV, 4, 0), (MV, 4, 512)])
    assert where[0] == 0, "a quantize step is not folded across a barrier"
    assert where[2] == where[3] == 2


def test_gather_keeps_its_order_against_overlapping_outputs(plan):
    # the second matvec writes inside the range the gather (512 floats per rank from offset 0) collects: stays behind it
    n, where = plan(2, 1, [(MV, 4, 0), (GA, 0, 0), (MV, 4, 512)])
    assert where == [0, 1, 2]
    # a matvec writing elsewhere may join the launch in front of the gather
    n, where = plan(2, 1, [(MV, 4, 0), (GA, 0, 0), (MV, 4, 4096)])
    assert n == 1 and where == [0, 1, 0]


def test_decode_pass_shape_on_two_ranks(plan):
    """quantize, q / k / v, barrier, quantize, o, barrier: the shape qwengine_b200.decode_pass records."""
    steps = [(Q, 4, 0), (MV, 4, 0), (MV, 4, 512), (MV, 4, 1024), (BA, 0, 0), (Q, 5, 0), (MV, 5, 2048), (BA, 0, 0)]
    n, where = plan(2, 1, steps)
    assert n == 2 and where == [-1, 1, 1, 1, 4, -1, 6, 7]
