"""The C-ABI library loads without a GPU, exports every function the headers
declare, and refuses to compute when no CUDA device is present."""
import ctypes
import os
import re

import numpy as np

import gehtp_b200
from gehtp_b200.runlists import DecoderConfig, build_decode_runlist
from gehtp_b200.wtop import Engine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for h in ("gehtp_cuda.h", "wtop_format.h"):
        src = open(os.path.join(ROOT, "include", h)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        for m in re.finditer(r"^[ \t]*(?!static|typedef|struct|enum|#)[A-Za-z_][\w \t\*]*?\b(\w+)\s*\(", src, flags=re.M):
            names.append(m.group(1))
    return sorted(set(n for n in names if n.startswith(("wt_", "gehtp_")) and n not in ("wt_rd_u32", "wt_rd_u16")))


def test_every_declared_symbol_is_exported(cuda):
    names = declared_functions()
    assert len(names) >= 30, names
    missing = [n for n in names if not hasattr(cuda, n)]
    assert not missing, missing


def test_struct_layout_matches_header(cuda):
    from gehtp_b200.wtop import WtBlob, WtOp, WtSlot
    assert ctypes.sizeof(WtSlot) == 24 and ctypes.sizeof(WtOp) == 68
    assert WtBlob.slots.offset == 16 and WtBlob.ops.offset == 16 + 24 * 4096
    assert cuda.gehtp_w4a16_slot_bytes(1024, 3072) == 1024 * 3072 // 2 + 2 * 16 * 3072


def test_no_cpu_fallback(cuda):
    """Without a CUDA device a run fails loudly instead of computing on the host."""
    import torch
    if torch.cuda.is_available():
        return
    cfg = DecoderConfig(128, 1, 4, 2, 64, 256, 512, 1e6, "tiny")
    buf, man = build_decode_runlist(cfg, 1, 32, quant="w4")
    eng = Engine(cuda, buf)
    try:
        eng.run_io(np.zeros(man["face_u16"], np.uint16), man["token_temp"], None)
        raise AssertionError("run succeeded without a GPU")
    except Exception as e:
        assert "no CUDA device" in str(e)
    a = np.zeros((1, 64), np.float16)
    assert cuda.gehtp_rmsnorm(a.ctypes.data, a.ctypes.data, None, a.ctypes.data, 1, 64) == -1
