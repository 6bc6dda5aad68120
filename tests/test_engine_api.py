"""The parts of the engine API beside the run calls (kernels/include/oplist_exec.h:56-114):
statistics, per-op trace lines, the caller-provided pool with static offsets, and the
bookkeeping opcodes (NOP, PIN, SPILL, FILL, DMA) — each on the CUDA engine and on the
reference executor with the same blob — plus how device-side bounded waits are reported."""
import ctypes
import os

import numpy as np
import pytest

from gehtp_b200.wtop import OP, S, BlobBuilder, Engine, WtStats


def bookkeeping_blob(rng):
    """NOP, PIN, ADD x2, SPILL, FILL, DMA slot->temp and temp->temp, 4-D TRANSPOSE (opcode 10)."""
    x = rng.standard_normal(256).astype(np.float16)
    y = rng.standard_normal(256).astype(np.float16)
    b = BlobBuilder()
    sx, sy = b.add_slot(x), b.add_slot(y)
    pool = b.add_slot(np.zeros(512, np.float16))
    b.add_op(OP.NOP, [])
    b.add_op(OP.PIN, [sx])
    b.add_op(OP.ADD, [S(sx), S(sy), 1, 256])                       # t1 = x + y
    b.add_op(OP.SPILL, [1, pool, 64, 256])                           # pool[64 B ...] = t1
    b.add_op(OP.FILL, [pool, 64, 2, 256])                            # t2 = pool[64 B ...]
    b.add_op(OP.ADD, [2, S(sx), 3, 256])                             # t3 = t2 + x
    b.add_op(OP.DMA, [S(sy), 4, 256, 128, 0, 0, 0xFF, 0xFF])         # t4[0:256 B] = y bytes 128..383
    b.add_op(OP.DMA, [3, 5, 128, 64, 32, 0, 0xFF, 0xFF])             # t5[32:160 B] = t3 bytes 64..191
    b.add_op(OP.TRANSPOSE, [3, 6, 4, 8, 8, 0 | 3 << 8 | 1 << 16 | 2 << 24])   # t3 viewed [1,4,8,8] NHWC -> NCHW
    want = {3: ((x + y).astype(np.float16) + x).astype(np.float16), 4: y[64:192]}
    return b, want


def run_both(cuda, ref, fn):
    out = []
    for lib in (cuda, ref):
        out.append(fn(lib))
    return out


@pytest.mark.gpu
def test_bookkeeping_ops_and_stats_match_the_reference(cuda, ref):
    def go(lib):
        b, want = bookkeeping_blob(np.random.default_rng(5))
        eng = Engine(lib, b.build())
        eng.run()
        st = WtStats()
        lib.wt_exec_get_stats(ctypes.byref(st))
        temps = {t: eng.temp(t).view(np.uint16) for t in (1, 2, 3, 4, 6)}
        t5 = eng.temp(5).view(np.uint16)[16:80]       # only bytes 32..159 of temp 5 are defined
        eng.shutdown()
        for t, w in want.items():
            assert np.array_equal(temps[t], w.view(np.uint16)), t
        return {n: getattr(st, n) for n, _ in WtStats._fields_}, temps, t5
    (st_c, tc, t5c), (st_r, tr, t5r) = run_both(cuda, ref, go)
    assert st_c == st_r, (st_c, st_r)
    assert st_c["ops"] == 9 and st_c["nop"] == 1 and st_c["add"] == 2 and st_c["pin"] == 1 and st_c["transpose"] == 1
    for t in tc:
        assert np.array_equal(tc[t], tr[t]), t
    assert np.array_equal(t5c, t5r)


@pytest.mark.gpu
def test_trace_lines(cuda, tmp_path, monkeypatch):
    """wt_exec_set_trace(1): one `pre` and one `op` line per op, in the reference's format
    (oplist_exec.c:2521-2561); nothing is written with the trace off."""
    path = tmp_path / "optrace.txt"
    monkeypatch.setenv("GEHTP_TRACE_FILE", str(path))
    b, _ = bookkeeping_blob(np.random.default_rng(5))
    eng = Engine(cuda, b.build())
    cuda.wt_exec_set_trace(0)
    eng.run()
    assert not path.exists() or path.read_text() == ""
    cuda.wt_exec_set_trace(1)
    try:
        eng.run()
    finally:
        cuda.wt_exec_set_trace(0)
    eng.shutdown()
    lines = path.read_text().splitlines()
    codes = [0, 3, 7, 8, 9, 7, 33, 33, 10]
    assert len(lines) == 2 * len(codes)
    for i, c in enumerate(codes):
        assert lines[2 * i].startswith("pre%d code=%d a=" % (i, c)) and " pool=" in lines[2 * i]
        assert lines[2 * i + 1].startswith("op%d code=%d rc=0 us=" % (i, c))
    args = eng.blob.ops[2].args
    assert lines[4].split(" a=")[1].split(" ")[0] == "%d,%d,%d,%d" % (args[0], args[1], args[2], args[3])


@pytest.mark.gpu
def test_pool_init_static_offsets(cuda, ref):
    """wt_exec_pool_init (oplist_exec.c:359-368): temps with an entry in the caller's offset
    table live at pool + offset, temps whose entry is 0xFFFFFFFF go to the bump region behind
    the static part; results are those of the plain run."""
    rng = np.random.default_rng(8)
    x = rng.standard_normal(512).astype(np.float16)
    b = BlobBuilder()
    sx = b.add_slot(x)
    b.add_op(OP.UNARY, [S(sx), 1, 512, 0])          # t1 = -x
    b.add_op(OP.ADD, [1, S(sx), 2, 512])            # t2 = 0
    b.add_op(OP.BINARY, [1, S(sx), 3, 512, 2])      # t3 = -x*x
    buf = b.build()
    offs = np.full(4096, 0xFFFFFFFF, np.uint32)
    offs[1], offs[2] = 2048, 0
    want3 = ((-x).astype(np.float16) * x).astype(np.float16)

    # The reference frees the pool in wt_exec_shutdown and only a shutdown initialises its
    # on-chip offset array when no TEMPOFF slot did: shutdown first, pool from the C allocator.
    libc = ctypes.CDLL(None)
    libc.memalign.restype = ctypes.c_void_p
    libc.memalign.argtypes = [ctypes.c_size_t, ctypes.c_size_t]
    pool = libc.memalign(128, 1 << 16)
    ref.wt_exec_shutdown()
    ref.wt_exec_pool_init(pool, 1 << 16, 4096, offs.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)))
    eng = Engine(ref, buf)
    eng.run()
    assert ref.wt_exec_temp(1) == pool + 2048 and ref.wt_exec_temp(2) == pool
    assert ref.wt_exec_temp(3) >= pool + 4096
    assert np.array_equal(eng.temp(3), want3)
    eng.shutdown()

    host_base = np.zeros(16, np.uint8)   # only says "a pool is given": device memory is the engine's own
    cuda.wt_exec_pool_init(host_base.ctypes.data, 1 << 16, 4096, offs.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)))
    try:
        eng = Engine(cuda, buf)
        eng.run()
        d1, d2, d3 = (cuda.gehtp_cuda_temp_dev(t) for t in (1, 2, 3))
        assert d1 - d2 == 2048, "static offsets are not honoured"
        assert d3 < d2 or d3 >= d2 + 4096, "a temp without an entry landed in the static region"
        assert np.array_equal(eng.temp(3), want3)
        assert np.array_equal(eng.temp(1), (-x).astype(np.float16))
        eng.shutdown()
    finally:
        cuda.wt_exec_pool_init(None, 0, 0, None)
    # and back to the engine's own placement
    eng = Engine(cuda, buf)
    eng.run()
    assert np.array_equal(eng.temp(3), want3)
    eng.shutdown()


def test_status_word_messages(cuda):
    """Each device-side bounded wait has its own code and message; a KV miss keeps the
    reference's 1-based op index as the return value."""
    msg = ctypes.create_string_buffer(160)
    seen = set()
    for code, frag in ((0x80000001, b"all-reduce timed out"), (0x80000002, b"attention timed out"),
                       (0x80000003, b"GEMM timed out")):
        assert cuda.gehtp_cuda_status_message(code, msg, 160) == -1
        assert frag in msg.value, msg.value
        seen.add(msg.value)
    assert len(seen) == 3
    assert cuda.gehtp_cuda_status_message(7, msg, 160) == 7 and b"kv gather miss" in msg.value and b"op 6" in msg.value
    assert cuda.gehtp_cuda_status_message(0x80000077, msg, 160) == -1 and b"0x80000077" in msg.value


@pytest.mark.gpu
def test_lost_peer_is_reported_not_waited_for(cuda):
    """A rank whose peers never write: the exchange kernel's wait runs into its (here
    shortened) limit, the run returns -1 "all-reduce timed out", nothing hangs, and the
    engine keeps working. The peers are stand-in mailboxes on the same GPU
    (gehtp_cuda_tp_p2p_loopback), so no second process and no fault is involved."""
    rng = np.random.default_rng(11)
    rows, width = 4, 256
    x = rng.standard_normal((rows, width)).astype(np.float16)
    w = (rng.standard_normal((width, width)) * 0.1).astype(np.float16)
    res = rng.standard_normal((rows, width)).astype(np.float16)
    gam = rng.normal(1, 0.1, width).astype(np.float16)

    def blob():
        b = BlobBuilder()
        sx, sw, sr, sg = b.add_slot(x), b.add_slot(w), b.add_slot(res), b.add_slot(gam)
        sz = b.add_slot(np.zeros(width, np.float16))
        b.add_op(OP.MATMUL_F16, [S(sx), S(sw), 1, rows, width, width, 0])     # row-parallel projection (partial sums)
        b.add_op(OP.ADD, [1, S(sr), 2, rows * width])
        b.add_op(OP.RMSNORM2, [2, S(sg), S(sz), 3, rows * width])
        return b.build()

    eng = Engine(cuda, blob())
    eng.run()
    want = eng.temp(3).copy()
    eng.shutdown()

    after = (ctypes.c_uint32 * 1)(0)
    for fusion in (1, 0):           # fused exchange+add+norm kernel, then the stand-alone all-reduce kernel
        cuda.gehtp_cuda_set_fusion(fusion)
        cuda.gehtp_cuda_set_wait_limit(2000)
        assert cuda.gehtp_cuda_tp_p2p_loopback(2) == 0, cuda.gehtp_cuda_last_error()
        try:
            assert cuda.gehtp_cuda_tp_allreduce_after(after, 1) == 0
            eng = Engine(cuda, blob())
            with pytest.raises(Exception) as ei:
                eng.run()
            assert ei.value.rc == -1 and "all-reduce timed out" in ei.value.msg
            eng.shutdown()
        finally:
            cuda.gehtp_cuda_tp_shutdown()
            cuda.gehtp_cuda_set_wait_limit(0)
            cuda.gehtp_cuda_set_fusion(1)
        eng = Engine(cuda, blob())
        eng.run()
        assert np.array_equal(eng.temp(3), want)
        eng.shutdown()
