"""B200-native quantized matvec / prefill GEMM for the q38rt (QWENgine) runtime.

The product is ``libq38b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/q38b200.h``); this package loads it and gives the tests and the benchmark a thin torch-tensor
wrapper.  There is no CPU fallback: without the built library or without a GPU the calls raise.
"""
from . import formats, synth            # noqa: F401
from .api import Context, GgufFile, Pass, Q38BError, load_library, library_path   # noqa: F401
