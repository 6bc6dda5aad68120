"""B200 executor for GEHTP WTOP runlists: Python face of libgehtp_cuda.so.

The compute lives in the shared library (hand-written sm_100a kernels behind the
reference's `wt_parse` / `wt_exec_*` C API). This package only loads it through
ctypes, builds runlist blobs, and mirrors the reference interface for tests and
benches. There is no CPU path: if the library is missing, loading raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgehtp_cuda.so")
_lib = None


def lib():
    """The loaded libgehtp_cuda.so. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libgehtp_cuda.so is not built (run `python -m gehtp_b200.build`); "
                "this package has no CPU fallback")
        from .wtop import bind
        _lib = bind(ctypes.CDLL(LIB_PATH))
    return _lib


from .wtop import (BlobBuilder, Engine, WtBlob, pack_w4a16, parse_blob, S, ST, OP)  # noqa: E402,F401
