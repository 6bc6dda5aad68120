"""WTOP blob writer and a thin ctypes mirror of the executor C API.

The wire format is the reference's (kernels/include/oplist_parse.h:1-31); the
writer plays the role of the reference's `wtop_emit` / `pack_oplist` for
hand-built runlists. `Engine` wraps any library that exports the reference
engine API — this repo's CUDA library or, in tests, the reference executor
compiled for the host — so one blob can be run through both and compared.
"""
import ctypes
import struct

import numpy as np

WT_MAX_SLOTS, WT_MAX_OPS, WT_MAX_ARGS = 4096, 65536, 16
SLOT_EXT_IN, SLOT_EXT_OUT, SLOT_TEMPOFF = 0xFFFFFFFF, 0xFFFFFFFE, 0xFFFFFFFD
SLOT_EXT_WGT, SLOT_STATE, KV_POS_AUTO = 0xFFFFFFFC, 0xFFFFFFFB, 0xFFFFFFFA


class OP:
    NOP, MATMUL_W4A16, RMSNORM, PIN, SILU, IM2COL, CONV2D, ADD, SPILL, FILL = range(10)
    TRANSPOSE, UNARY, BINARY, SOFTMAX, CONCAT, SLICE, SPLIT, REDUCE, CUMSUM = range(10, 19)
    CONV1D_SSM, GATHER, ARGMAX, KV_APPEND, KV_GATHER, MATMUL_F16, RMSNORM2 = range(19, 26)
    BROADCAST, TRANSPOSE_GEN, SCATTER_ND, CONV1D_SSM_STEP, DELTA_CHUNK = range(26, 31)
    DMA, PAD, MATMUL_F16_SPLIT = 33, 34, 35


ARITY = {0: 0, 1: 6, 2: 4, 3: 1, 4: 3, 5: 15, 6: 13, 7: 4, 8: 4, 9: 4, 10: 6, 11: 4, 12: 5, 13: 4,
         14: 16, 15: 16, 16: 16, 17: 9, 18: 7, 19: 6, 20: 15, 21: 3, 22: 4, 23: 7, 24: 7, 25: 5,
         26: 12, 27: 8, 28: 14, 29: 6, 30: 12, 33: 8, 34: 7, 35: 9}


# argument positions that name the temp(s) an op writes
_OUT_ARGS = {1: (2,), 4: (1,), 7: (2,), 10: (1,), 11: (1,), 12: (2,), 13: (1,), 14: (8,), 15: (1,), 16: (1,),
             17: (1,), 18: (1,), 19: (2,), 20: (2,), 21: (1,), 23: (1, 2), 24: (2,), 25: (3,), 26: (1,),
             27: (1,), 28: (3,), 29: (2,), 30: (5,), 34: (1,), 35: (2,)}


def op_out_temps(op):
    """Temp ids an op record writes (a parsed `WtOp` or an (opcode, args) pair)."""
    opcode, args = (op.opcode, list(op.args)) if hasattr(op, "opcode") else op
    pos = _OUT_ARGS.get(opcode, ())
    if opcode == OP.BINARY and args[4] == 8:      # SELECT form [cond, a, b, out, 8]
        pos = (3,)
    return [args[i] & 0x3FFF for i in pos if not (opcode == OP.KV_GATHER and args[i] == 0)]


def S(slot):
    """Reference to a slot in an op argument."""
    return 0x8000 | slot


def ST(state):
    """Reference to a persistent state in an op argument."""
    return 0x6000 | state


def _align(x, a=128):
    return (x + a - 1) // a * a


def pack_w4a16(q, scales):
    """Weight slot bytes for opcode 1, group-64 form.

    q: uint8 [K, N] with values 0..15; scales: float16 [K/64, N].
    Layout: nibbles [K][N/2] (low nibble = even column), then the scales.
    """
    q = np.ascontiguousarray(q, dtype=np.uint8)
    K, N = q.shape
    assert K % 64 == 0 and N % 16 == 0 and q.max(initial=0) < 16
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    assert scales.shape == (K // 64, N)
    nib = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return nib.tobytes() + scales.tobytes()


class BlobBuilder:
    """Collects slots and ops and serialises a WTOP v1 (or v2 past 4 GB) blob."""

    def __init__(self):
        self.slots = []   # (bytes-like or None, len, count, addr)
        self.ops = []
        self.force_v2 = False

    def add_slot(self, data, count=None, addr=0):
        if isinstance(data, np.ndarray):
            if count is None:
                count = data.size
            data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        else:
            data = np.frombuffer(bytes(data), dtype=np.uint8)
        assert data.size > 0
        if count is None:
            count = data.size // 2
        self.slots.append((data, int(data.size), int(count), addr))
        return len(self.slots) - 1

    def add_ext_in(self, nbytes, baked=None):
        data = np.zeros(nbytes, np.uint8) if baked is None else np.frombuffer(bytes(baked), np.uint8)
        assert data.size == nbytes
        return self.add_slot(data, count=nbytes // 2, addr=SLOT_EXT_IN)

    def add_states(self, sizes):
        return self.add_slot(struct.pack("<I%dI" % len(sizes), len(sizes), *sizes), addr=SLOT_STATE)

    def add_tempoff(self, cap, entries, bump_kb=0, vtcm_kb=0):
        """entries: (temp_id, offset, size); temp_id may carry 0x4000 for the on-chip region."""
        body = struct.pack("<III", cap, (vtcm_kb << 16) | bump_kb, len(entries))
        for tid, off, size in entries:
            body += struct.pack("<III", tid, off, size)
        return self.add_slot(body, addr=SLOT_TEMPOFF)

    def add_op(self, opcode, args, check=True):
        args = [int(a) & 0xFFFFFFFF for a in args]
        if check:
            assert ARITY.get(opcode) == len(args), (opcode, len(args))
        self.ops.append((opcode, args))
        return len(self.ops) - 1

    def build(self):
        offs, pos = [], 0
        for _, ln, _, _ in self.slots:
            offs.append(pos)
            pos = _align(pos + ln)
        v2 = self.force_v2 or pos > 0xFFFFFFF0
        head = b"WTOP" + struct.pack("<HHII", 2 if v2 else 1, 0x1234, len(self.slots), len(self.ops))
        tab = bytearray()
        for (_, ln, cnt, addr), off in zip(self.slots, offs):
            if v2:
                tab += struct.pack("<IIIIII", ln, cnt, off & 0xFFFFFFFF, off >> 32, addr, 0)
            else:
                tab += struct.pack("<IIII", ln, cnt, off, addr)
        ops = bytearray()
        for opcode, args in self.ops:
            ops += struct.pack("<HH%dI" % len(args), opcode, len(args), *args)
        pre = head + bytes(tab) + bytes(ops)
        woff = _align(len(pre))
        out = np.zeros(woff + max(pos, 1), dtype=np.uint8)
        out[:len(pre)] = np.frombuffer(pre, np.uint8)
        for (data, ln, _, _), off in zip(self.slots, offs):
            out[woff + off: woff + off + ln] = data
        return out


class WtSlot(ctypes.Structure):
    _fields_ = [("len", ctypes.c_uint32), ("count", ctypes.c_uint32), ("offset", ctypes.c_uint64),
                ("addr", ctypes.c_uint32)]


class WtOp(ctypes.Structure):
    _fields_ = [("opcode", ctypes.c_uint16), ("n_args", ctypes.c_uint16), ("args", ctypes.c_uint32 * WT_MAX_ARGS)]


class WtBlob(ctypes.Structure):
    _fields_ = [("ver", ctypes.c_uint16), ("n_slots", ctypes.c_uint32), ("n_ops", ctypes.c_uint32),
                ("weight_off", ctypes.c_uint32), ("slots", WtSlot * WT_MAX_SLOTS), ("ops", WtOp * WT_MAX_OPS),
                ("weight_base", ctypes.c_void_p), ("weight_bytes", ctypes.c_size_t)]


class WtStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint32) for n in ("ops", "nop", "matmul", "rmsnorm", "silu", "pin", "pin_skipped",
                                                "im2col", "conv2d", "add", "spill", "fill", "transpose")]


class WtOpTs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint32) for n in ("start_us", "dur_us", "dma_us", "dma_bytes", "engine")]


def bind(lib):
    """Declares the argument types of the engine API on a loaded library."""
    c = ctypes
    P = c.POINTER
    lib.wt_parse.argtypes = [c.c_void_p, c.c_size_t, P(WtBlob)]
    lib.wt_parse.restype = c.c_int
    lib.wt_err_str.argtypes = [c.c_int]
    lib.wt_err_str.restype = c.c_char_p
    lib.wt_exec_run.argtypes = [P(WtBlob), P(c.c_uint32), P(c.c_int64), c.c_char_p, c.c_size_t]
    lib.wt_exec_run_range.argtypes = [P(WtBlob), c.c_uint32, c.c_uint32, P(c.c_uint32), P(c.c_int64), c.c_char_p, c.c_size_t]
    lib.wt_exec_run_io.argtypes = [P(WtBlob), c.c_void_p, c.c_void_p, c.c_uint32, P(c.c_uint32), P(c.c_int64), c.c_char_p, c.c_size_t]
    for f in (lib.wt_exec_run, lib.wt_exec_run_range, lib.wt_exec_run_io):
        f.restype = c.c_int
    lib.wt_exec_temp.argtypes = [c.c_uint32]
    lib.wt_exec_temp.restype = c.c_void_p
    lib.wt_exec_temp_bytes.argtypes = [c.c_uint32]
    lib.wt_exec_temp_bytes.restype = c.c_uint32
    lib.wt_exec_temp_last_bytes.argtypes = [c.c_uint32]
    lib.wt_exec_temp_last_bytes.restype = c.c_uint32
    lib.wt_exec_shutdown.restype = None
    lib.wt_exec_state_reset.restype = None
    lib.wt_exec_pool_init.argtypes = [c.c_void_p, c.c_uint32, c.c_uint32, P(c.c_uint32)]
    lib.wt_exec_pool_init.restype = None
    lib.wt_exec_get_stats.argtypes = [P(WtStats)]
    lib.wt_exec_set_ext_weights.argtypes = [c.c_void_p]
    lib.wt_exec_set_ts.argtypes = [P(WtOpTs), c.c_uint32]
    lib.wt_exec_set_trace.argtypes = [c.c_int]
    lib.wt_exec_set_hook.argtypes = [c.c_char_p]
    if hasattr(lib, "gehtp_cuda_launch_count"):
        lib.gehtp_cuda_launch_count.restype = c.c_uint64
        lib.gehtp_cuda_fused_ops.restype = c.c_uint32
        lib.gehtp_cuda_const_ops.restype = c.c_uint32
        lib.gehtp_cuda_demoted_temps.restype = c.c_uint32
        lib.gehtp_cuda_stream.restype = c.c_void_p
        lib.gehtp_cuda_temp_dev.argtypes = [c.c_uint32]
        lib.gehtp_cuda_temp_dev.restype = c.c_void_p
        lib.gehtp_cuda_last_error.restype = c.c_char_p
        lib.gehtp_cuda_set_device.argtypes = [c.c_int]
        lib.gehtp_cuda_set_fusion.argtypes = [c.c_int]
        lib.gehtp_cuda_set_graph.argtypes = [c.c_int]
        lib.gehtp_cuda_run_dev.argtypes = [P(WtBlob), c.c_void_p, c.c_void_p, c.c_uint32, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_run_profiled.argtypes = [P(WtBlob), c.c_void_p, c.c_uint32, P(c.c_float), c.c_uint32, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_profiled_attn.argtypes = [P(c.c_float), P(c.c_uint32)]
        lib.gehtp_cuda_profiled_attn.restype = None
        lib.gehtp_cuda_state_load.argtypes = [P(WtBlob), c.c_uint32, c.c_void_p, c.c_size_t, c.c_int, c.c_uint32, c.c_uint32, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_state_set_count.argtypes = [c.c_uint32, c.c_uint32]
        lib.gehtp_cuda_state_read.argtypes = [c.c_uint32, c.c_void_p, c.c_size_t]
        lib.gehtp_cuda_state_save_hds1.argtypes = [P(WtBlob), c.c_char_p, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_state_load_hds1.argtypes = [P(WtBlob), c.c_char_p, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_tp_init.argtypes = [c.c_int, c.c_int, c.c_void_p, c.c_size_t]
        lib.gehtp_cuda_tp_unique_id.argtypes = [c.c_void_p, c.c_size_t]
        lib.gehtp_cuda_tp_allreduce_after.argtypes = [P(c.c_uint32), c.c_uint32]
        lib.gehtp_cuda_tp_p2p_export.argtypes = [c.c_void_p, c.c_size_t]
        lib.gehtp_cuda_tp_p2p_import.argtypes = [c.c_void_p, c.c_size_t, c.c_int]
        lib.gehtp_cuda_tp_p2p_disable.restype = None
        lib.gehtp_cuda_status_message.argtypes = [c.c_uint32, c.c_char_p, c.c_size_t]
        lib.gehtp_cuda_set_wait_limit.argtypes = [c.c_uint32]
        lib.gehtp_cuda_set_wait_limit.restype = None
        lib.gehtp_cuda_tp_p2p_loopback.argtypes = [c.c_int]
        lib.gehtp_attn_decode_noalloc_status.restype = c.c_int
        lib.gehtp_w4a16_slot_bytes.argtypes = [c.c_uint32, c.c_uint32]
        lib.gehtp_w4a16_slot_bytes.restype = c.c_size_t
        lib.gehtp_w4a16_matmul.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32, c.c_uint32, c.c_int]
        lib.gehtp_w4a16_unpack.argtypes = [c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32]
        lib.gehtp_rmsnorm.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32]
        lib.gehtp_attn_decode.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32,
                                          c.c_uint32, c.c_uint32, c.c_uint32, c.c_float]
        vp, u32 = c.c_void_p, c.c_uint32
        lib.gehtp_dev_w4_repack.argtypes = [vp, vp, u32, u32]
        lib.gehtp_dev_w4a16_matmul.argtypes = [vp, vp, vp, vp, u32, u32, u32, c.c_int]
        lib.gehtp_dev_matmul_f16_nk.argtypes = [vp, vp, vp, u32, u32, u32]
        lib.gehtp_dev_w4a16_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, u32]
        lib.gehtp_dev_rmsnorm.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32]
        lib.gehtp_cuda_capture_end_replay.argtypes = [c.c_int, P(c.c_float)]
        lib.gehtp_attn_decode_noalloc.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32,
                                                  c.c_uint32, c.c_uint32, c.c_uint32, c.c_float, c.c_void_p]
    return lib


def parse_blob(lib, buf):
    """wt_parse on a numpy uint8 buffer. Returns (rc, WtBlob); the blob keeps pointers into buf."""
    blob = WtBlob()
    rc = lib.wt_parse(buf.ctypes.data, buf.size, ctypes.byref(blob))
    return rc, blob


class EngineError(RuntimeError):
    def __init__(self, rc, msg):
        super().__init__("op %d failed: %s" % (rc, msg) if rc > 0 else "run failed (%d): %s" % (rc, msg))
        self.rc, self.msg = rc, msg


class Engine:
    """One parsed blob on one engine library (the reference API allows one engine per process)."""

    def __init__(self, lib, buf):
        self.lib = lib
        self.buf = np.ascontiguousarray(buf, dtype=np.uint8)
        rc, self.blob = parse_blob(lib, self.buf)
        if rc != 0:
            raise ValueError("wt_parse: %s (%d)" % (lib.wt_err_str(rc).decode(), rc))
        self._err = ctypes.create_string_buffer(256)

    def _check(self, rc):
        if rc != 0:
            raise EngineError(rc, self._err.value.decode(errors="replace"))

    def run(self, op_us=None):
        self._check(self.lib.wt_exec_run(ctypes.byref(self.blob), None, op_us, self._err, 256))

    def run_range(self, first, count):
        self._check(self.lib.wt_exec_run_range(ctypes.byref(self.blob), first, count, None, None, self._err, 256))

    def run_io(self, inp, out_temp, out=None):
        """inp: numpy array or None; out: preallocated numpy array or None. Returns out."""
        ip = None
        if inp is not None:
            self._in_keep = np.ascontiguousarray(inp)
            ip = self._in_keep.ctypes.data
        op = out.ctypes.data if out is not None else None
        # wt_exec_run_io copies the temp's last byte count into `out` and takes no size (the reference's contract):
        # a buffer that was too small is reported right after the call instead of corrupting the heap in silence
        self._check(self.lib.wt_exec_run_io(ctypes.byref(self.blob), ip, op, out_temp, None, None, self._err, 256))
        if out is not None and self.lib.wt_exec_temp_last_bytes(out_temp) > out.nbytes:
            raise ValueError("out held %d bytes, temp %d wrote %d: memory behind `out` was overwritten"
                             % (out.nbytes, out_temp, self.lib.wt_exec_temp_last_bytes(out_temp)))
        return out

    def temp(self, tid, dtype=np.float16):
        n = self.lib.wt_exec_temp_last_bytes(tid)
        p = self.lib.wt_exec_temp(tid)
        if not p or not n:
            return None
        raw = (ctypes.c_uint8 * n).from_address(p)
        return np.frombuffer(bytes(raw), dtype=dtype).copy()

    def shutdown(self):
        self.lib.wt_exec_shutdown()

    def state_reset(self):
        self.lib.wt_exec_state_reset()

    def state_save_hds1(self, path):
        """Writes the 42-state decode table as an "HDS1" file (compiler/src/ops/host_decode_state.cpp:41-62)."""
        if self.lib.gehtp_cuda_state_save_hds1(ctypes.byref(self.blob), str(path).encode(), self._err, 256) != 0:
            raise EngineError(-1, self._err.value.decode(errors="replace"))

    def state_load_hds1(self, path):
        """Returns 0 (loaded) or 1 (no such file); raises on a bad file or a state table of another shape."""
        rc = self.lib.gehtp_cuda_state_load_hds1(ctypes.byref(self.blob), str(path).encode(), self._err, 256)
        if rc < 0:
            raise EngineError(-1, self._err.value.decode(errors="replace"))
        return rc
