"""WTOP parser: accepts what the writer produces, refuses each malformed class
with the reference's error code (kernels/include/oplist_parse.h:277-292), and
agrees with the reference's own parser byte for byte on the parsed struct."""
import ctypes
import struct

import numpy as np
import pytest

from gehtp_b200.wtop import OP, S, BlobBuilder, WtBlob, parse_blob


def sample_blob(v2=False):
    b = BlobBuilder()
    b.force_v2 = v2
    s0 = b.add_slot(np.arange(40, dtype=np.float16))
    s1 = b.add_ext_in(64)
    b.add_states([4096, 512])
    b.add_op(OP.UNARY, [S(s0), 1, 40, 14])
    b.add_op(OP.ADD, [1, S(s0), 2, 40])
    b.add_op(OP.MATMUL_F16, [S(s1), S(s0), 3, 1, 4, 8, 0])
    b.add_op(OP.NOP, [])
    return b.build()


def test_round_trip(cuda):
    for v2 in (False, True):
        buf = sample_blob(v2)
        rc, w = parse_blob(cuda, buf)
        assert rc == 0
        assert (w.ver, w.n_slots, w.n_ops) == (2 if v2 else 1, 3, 4)
        assert w.slots[0].len == 80 and w.slots[0].count == 40 and w.slots[0].offset == 0
        assert w.slots[1].addr == 0xFFFFFFFF and w.slots[2].addr == 0xFFFFFFFB
        assert w.slots[1].offset % 128 == 0 and w.weight_off % 128 == 0
        assert w.ops[0].opcode == OP.UNARY and list(w.ops[0].args[:4]) == [0x8000, 1, 40, 14]
        assert w.ops[2].n_args == 7 and w.weight_bytes == buf.size - w.weight_off
        base = ctypes.cast(w.weight_base, ctypes.POINTER(ctypes.c_uint16))
        assert [base[i] for i in range(3)] == list(np.arange(3, dtype=np.float16).view(np.uint16))


def corruptions():
    good = sample_blob()
    def mod(fn):
        b = good.copy()
        return fn(b)
    def put(b, off, fmt, *v):
        b[off:off + struct.calcsize(fmt)] = np.frombuffer(struct.pack(fmt, *v), np.uint8)
        return b
    slot0, ops0 = 16, 16 + 3 * 16
    return [
        ("short", good[:12].copy(), -1),
        ("magic", mod(lambda b: put(b, 0, "<4s", b"WTOQ")), -2),
        ("version", mod(lambda b: put(b, 4, "<H", 3)), -3),
        ("endian", mod(lambda b: put(b, 6, "<H", 0x3412)), -4),
        ("nslots0", mod(lambda b: put(b, 8, "<I", 0)), -5),
        ("nslots_big", mod(lambda b: put(b, 8, "<I", 4097)), -5),
        ("nops0", mod(lambda b: put(b, 12, "<I", 0)), -6),
        ("slots_overrun", good[:40].copy(), -7),
        ("slot_len0", mod(lambda b: put(b, slot0, "<I", 0)), -8),
        ("slot_past_end", mod(lambda b: put(b, slot0, "<I", 1 << 20)), -8),
        ("op_trunc", good[:ops0 + 6].copy(), -9),
        ("opcode", mod(lambda b: put(b, ops0, "<H", 31)), -10),
        ("arity", mod(lambda b: put(b, ops0 + 2, "<H", 3)), -11),
        ("bad_ref", mod(lambda b: put(b, ops0 + 4, "<I", 0x8000 | 99)), -12),
        ("align", mod(lambda b: put(b, slot0 + 8, "<I", 64)), -13),
    ]


@pytest.mark.parametrize("name,buf,code", corruptions(), ids=[c[0] for c in corruptions()])
def test_malformed_blobs_are_refused(cuda, name, buf, code):
    rc, _ = parse_blob(cuda, buf)
    assert rc == code
    assert cuda.wt_err_str(rc) not in (b"OK", b"unknown")


def test_agrees_with_reference_parser(cuda, ref):
    blobs = [sample_blob(), sample_blob(True)] + [c[1] for c in corruptions()]
    rng = np.random.default_rng(0)
    good = sample_blob()
    for _ in range(300):   # random single-byte damage in the header / tables
        b = good.copy()
        i = int(rng.integers(0, 200))
        b[i] = rng.integers(0, 256)
        blobs.append(b)
    for buf in blobs:
        rc1, w1 = parse_blob(cuda, buf)
        rc2, w2 = parse_blob(ref, buf)
        assert rc1 == rc2
        if rc1 == 0:
            assert (w1.ver, w1.n_slots, w1.n_ops, w1.weight_off, w1.weight_bytes) == \
                   (w2.ver, w2.n_slots, w2.n_ops, w2.weight_off, w2.weight_bytes)
            n = ctypes.sizeof(WtBlob.slots.size and WtBlob)  # compare slot and op tables that were filled
            s1 = bytes(ctypes.string_at(ctypes.addressof(w1.slots), 24 * w1.n_slots))
            s2 = bytes(ctypes.string_at(ctypes.addressof(w2.slots), 24 * w2.n_slots))
            assert [x for i, x in enumerate(s1) if i % 24 < 20] == [x for i, x in enumerate(s2) if i % 24 < 20]
            for i in range(w1.n_ops):
                a, b2 = w1.ops[i], w2.ops[i]
                assert (a.opcode, a.n_args, list(a.args[:a.n_args])) == (b2.opcode, b2.n_args, list(b2.args[:b2.n_args]))
