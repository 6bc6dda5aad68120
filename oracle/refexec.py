"""Loads the CPU checkers: the reference executor built for the host
(oracle/_ref/libgehtp_ref.so) and this repo's C restatement (oracle/liboracle.so).
TEST INFRASTRUCTURE — never imported by the product package."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_PATH = os.path.join(_HERE, "_ref", "libgehtp_ref.so")
ORC_PATH = os.path.join(_HERE, "liboracle.so")


def ref_lib(private_dir=None):
    """The reference's own executor (scalar CPU paths), or None when not built.
    With private_dir the library is copied there first, which gives the caller
    an instance with its own global engine state."""
    if not os.path.exists(REF_PATH):
        return None
    from gehtp_b200.wtop import bind
    path = REF_PATH
    if private_dir:
        import shutil
        import uuid
        path = os.path.join(private_dir, "libgehtp_ref_%s.so" % uuid.uuid4().hex)
        shutil.copy(REF_PATH, path)
    lib = bind(ctypes.CDLL(path))
    lib.wt_exec_set_trace(0)
    return lib


def orc_lib():
    if not os.path.exists(ORC_PATH):
        raise RuntimeError("oracle/liboracle.so not built: run `make -C oracle`")
    c = ctypes
    lib = c.CDLL(ORC_PATH)
    vp, u32 = c.c_void_p, c.c_uint32
    lib.orc_f16_to_f32.argtypes = [c.c_uint16]
    lib.orc_f16_to_f32.restype = c.c_float
    lib.orc_f32_to_f16.argtypes = [c.c_float]
    lib.orc_f32_to_f16.restype = c.c_uint16
    lib.orc_w4_unpack_i8.argtypes = [vp, vp, u32, u32]
    lib.orc_w4_dequant.argtypes = [vp, vp, u32, u32]
    lib.orc_w4a16_matmul.argtypes = [vp, vp, vp, u32, u32, u32]
    lib.orc_matmul_f16.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, c.c_int, c.c_int, c.c_int, u32]
    lib.orc_rmsnorm2.argtypes = [vp, vp, vp, vp, u32, u32]
    lib.orc_softmax.argtypes = [vp, vp, u32, u32]
    lib.orc_binary.argtypes = [vp, vp, vp, u32, u32]
    lib.orc_unary.argtypes = [vp, vp, u32, u32]
    lib.orc_kv_append.argtypes = [vp, vp, u32, u32, vp, vp, u32]
    lib.orc_kv_gather.argtypes = [vp, vp, u32, u32, u32, u32, u32, u32, vp, vp]
    lib.orc_attn_decode_chain.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, c.c_float, c.c_int, vp, vp]
    lib.orc_attn_decode_f64.argtypes = [vp, vp, u32, u32, u32, u32, u32, c.c_double, vp, vp]
    lib.orc_conv1d_ssm.argtypes = [vp, vp, vp, u32, u32, u32]
    lib.orc_conv1d_step.argtypes = [vp, vp, vp, vp, u32, u32]
    lib.orc_delta_chunk.argtypes = [vp] * 7 + [c.c_int] * 5
    lib.orc_delta_token.argtypes = [vp, c.c_int, vp, vp, vp, c.c_float, c.c_float, vp]
    return lib


def ptr(a):
    return None if a is None else a.ctypes.data
