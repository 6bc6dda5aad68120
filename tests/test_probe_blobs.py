"""Blobs compiled by the reference's own chain run unchanged.

tests/golden/probe/ holds the reference's `qnn_probe` model as its own
`hnnx_compile` + `wtop_emit` wrote it (compiler/tools/wtop_emit.cpp:74 `emit`;
TAG_MEM_PLAN copied at :129-145, TEMPOFF slot at :569-602), once without and
once with `--ddr-budget`, the f32 logits of the reference's `host_run`, and every
op's output from the reference's device executor compiled for the host
(tests/golden/make_probe_blobs.py wrote them). The CPU tests pin those files to
each other and to a fresh run of the reference executor; the GPU tests push both
blobs through wt_parse + wt_exec_run_io of the CUDA library as they are.
"""
import glob
import json
import os
import struct

import numpy as np
import pytest

from conftest import cos_sim, ulp_diff_f16
from gehtp_b200.wtop import OP, Engine, op_out_temps, parse_blob

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "probe")
# ops that are bit-exact against the reference given the same input bytes: rearrangements,
# add/sub/mul/div, and MATMUL_F16 in the one-kernel-per-op plan (k ascending, as the scalar loop)
BITWISE = {OP.GATHER, OP.SPLIT, OP.SLICE, OP.CONCAT, OP.BROADCAST, OP.TRANSPOSE_GEN, OP.ADD, OP.BINARY, OP.MATMUL_F16}
# number of leading arguments that are input references
IN_ARGS = {OP.ADD: 2, OP.UNARY: 1, OP.BINARY: 2, OP.SOFTMAX: 1, OP.SLICE: 1, OP.SPLIT: 1, OP.GATHER: 2,
           OP.MATMUL_F16: 2, OP.RMSNORM2: 1, OP.BROADCAST: 1, OP.TRANSPOSE_GEN: 1}


def load(name):
    buf = np.fromfile(os.path.join(HERE, name + ".wtop"), np.uint8)
    man = json.load(open(os.path.join(HERE, name + ".manifest.json")))
    return buf, man


def ids():
    return np.fromfile(os.path.join(HERE, "ids.i32.raw"), np.int32)


def host_logits():
    return np.fromfile(os.path.join(HERE, "host_run.f32.raw"), np.float32).reshape(32, 256)


def check_logits(got_f16, what):
    """The reference's own whole-model gate (scripts/judge_logits.py): cosine and per-row top-1."""
    got = np.asarray(got_f16, np.float16).astype(np.float64).reshape(32, 256)
    want = host_logits().astype(np.float64)
    assert cos_sim(got, want) >= 0.9999, what
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), what
    assert (got.argmax(1) == want.argmax(1)).all(), what + ": top-1 differs"


def tempoff_entries(buf, blob):
    for i in range(blob.n_slots):
        sl = blob.slots[i]
        if sl.addr == 0xFFFFFFFD:
            raw = buf[blob.weight_off + sl.offset: blob.weight_off + sl.offset + sl.len].tobytes()
            cap, _reserve, n = struct.unpack_from("<III", raw, 0)
            return cap, [struct.unpack_from("<III", raw, 12 + 12 * k) for k in range(n)]
    return None, []


def hooked_run(lib, eng, pairs, inp):
    for f in glob.glob("/tmp/hook_*_*.f16.raw"):
        os.remove(f)
    spec = ",".join("%d:%d" % p for p in pairs).encode()
    lib.wt_exec_set_hook(spec)
    try:
        eng.run_io(inp, 0)
    finally:
        lib.wt_exec_set_hook(None)
    out = {}
    for i, t in pairs:
        fn = "/tmp/hook_%d_%d.f16.raw" % (i, t)
        assert os.path.exists(fn), "no dump for op %d temp %d" % (i, t)
        out[(i, t)] = np.fromfile(fn, np.uint16)
        os.remove(fn)
    return out


def test_fixture_is_what_the_reference_emits(cuda):
    """Both blobs parse with this library's wt_parse; op list and manifest agree;
    the planned blob carries the 14-entry offset table whose entries alias."""
    for name in ("probe_noplan", "probe_plan"):
        buf, man = load(name)
        rc, blob = parse_blob(cuda, buf)
        assert rc == 0
        assert blob.n_ops == man["n_ops"] == 99 and blob.n_slots == man["n_slots"]
        assert [blob.ops[i].opcode for i in range(99)] == man["opcodes"]
        assert man["output_temp"] == 8 and man["input_elems"] == 32
        cap, ents = tempoff_entries(buf, blob)
        if name == "probe_noplan":
            assert cap is None
        else:
            assert cap == 67108864 and len(ents) == 14
            off = {tid: o for tid, o, _ in ents}
            assert off[1] == off[3] and off[5] == off[8] == off[12]   # recycled temp ids share plan offsets


def test_reference_executor_on_its_own_blob(ref):
    """The no-plan blob on the reference's device executor (host build) meets the
    host_run golden and reproduces the committed per-op dumps bit for bit; the
    planned blob corrupts itself there (aliased live temps) — the hazard the CUDA
    planner has to avoid, not reproduce."""
    buf, man = load("probe_noplan")
    eng = Engine(ref, buf)
    gold = np.load(os.path.join(HERE, "ref_ops.npz"))
    pairs = [(i, t) for i in range(eng.blob.n_ops) for t in op_out_temps(eng.blob.ops[i])]
    assert sorted("op%d_t%d" % p for p in pairs) == sorted(gold.files)
    dumps = hooked_run(ref, eng, pairs, ids())
    for (i, t), got in dumps.items():
        assert np.array_equal(got, gold["op%d_t%d" % (i, t)]), (i, t)
    check_logits(eng.temp(man["output_temp"]), "reference executor, no-plan blob")
    eng.shutdown()

    buf, man = load("probe_plan")
    eng = Engine(ref, buf)
    eng.run_io(ids(), 0)
    bad = eng.temp(man["output_temp"]).astype(np.float64)
    assert cos_sim(bad, host_logits()) < 0.5
    eng.shutdown()


@pytest.mark.gpu
def test_compiled_blobs_run_unchanged(cuda):
    """Both compiled blobs through the CUDA engine: logits meet the host_run gate, the
    planned blob gives the same logits as the unplanned one, and its aliasing table
    entries are moved out of the static pool."""
    logits = {}
    for name in ("probe_noplan", "probe_plan"):
        buf, man = load(name)
        for fusion in (1, 0):
            cuda.gehtp_cuda_set_fusion(fusion)
            eng = Engine(cuda, buf)
            out = np.zeros(32 * 256, np.float16)
            for _ in range(4):   # eager, eager, captured graph, replay
                out[:] = 0
                eng.run_io(ids(), man["output_temp"], out)
                check_logits(out, "%s fusion=%d" % (name, fusion))
            logits[(name, fusion)] = out.copy()
            if name == "probe_plan":
                assert cuda.gehtp_cuda_demoted_temps() > 0
            else:
                assert cuda.gehtp_cuda_demoted_temps() == 0
            eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    assert np.array_equal(logits[("probe_noplan", 0)], logits[("probe_plan", 0)])
    assert np.array_equal(logits[("probe_noplan", 1)], logits[("probe_plan", 1)])


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["probe_noplan", "probe_plan"])
def test_every_op_against_the_reference_dumps(cuda, name):
    """wt_exec_set_hook dumps of all 99 ops against the reference executor's: byte
    moves bit-exact, arithmetic within 2 fp16 steps (the reference's own per-op gate,
    kernels/examples/38)."""
    buf, man = load(name)
    gold = np.load(os.path.join(HERE, "ref_ops.npz"))
    eng = Engine(cuda, buf)
    pairs = [(i, t) for i in range(eng.blob.n_ops) for t in op_out_temps(eng.blob.ops[i])]
    dumps = hooked_run(cuda, eng, pairs, ids())
    exact = {}          # temp id -> its current bytes equal the reference's
    stats = {"exact": 0, "steps": 0, "drift": 0}
    for (i, t), got in dumps.items():
        want = gold["op%d_t%d" % (i, t)]
        op = eng.blob.ops[i]
        opcode, args = op.opcode, list(op.args)
        assert got.shape == want.shape, (i, t, got.shape, want.shape)
        n_in = args[10] if opcode == OP.CONCAT else IN_ARGS[opcode]
        clean_in = all((a & 0x8000) or exact.get(a & 0x3FFF, False) for a in args[:n_in])
        same = bool(np.array_equal(got, want))
        exact[t] = same
        bitwise = opcode in BITWISE or (opcode == OP.UNARY and args[3] in (0, 5, 14))
        if clean_in and bitwise:
            assert same, "op %d (opcode %d): same input bytes, different output bytes" % (i, opcode)
            stats["exact"] += 1
            continue
        d = ulp_diff_f16(got, want)
        a = got.view(np.float16).astype(np.float64)
        b = want.view(np.float16).astype(np.float64)
        if clean_in:
            # the reference's own per-op gate (kernels/examples/38): transcendental unary and
            # rmsnorm within 1 fp16 step, softmax within 2
            assert d.max() <= 2, "op %d (opcode %d): %d fp16 steps from the reference" % (i, opcode, d.max())
            stats["steps"] += 1
            continue
        # inputs already differ by earlier roundings: the project's fp16 gate, per op
        assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() and cos_sim(a, b) >= 0.9999, \
            "op %d (opcode %d): max err %g of %g" % (i, opcode, np.abs(a - b).max(), np.abs(b).max())
        stats["drift"] += 1
    print(name, stats)
    assert stats["exact"] >= 10
    eng.shutdown()


def test_external_weights_v2_blob_on_the_reference_executor(cuda, ref):
    """probe_ext_v2.wtop (wtop_emit --ext-weights --force-v2): a v2 header with 24-byte slot
    records; weight slots are EXT_WGT descriptors into probe_ext_v2.weights.bin
    (compiler/tools/wtop_emit.cpp:608-620, 700-711). Parsed by this library's wt_parse, it names
    the same bytes as the inline blob; on the reference executor with wt_exec_set_ext_weights
    (oplist_exec.c:2583) it reproduces the inline blob's logits bit for bit, and without the
    external area it fails instead of reading something else."""
    buf, man = load("probe_ext_v2")
    ibuf, _ = load("probe_noplan")
    wts = np.fromfile(os.path.join(HERE, "probe_ext_v2.weights.bin"), np.uint8)
    rc, blob = parse_blob(cuda, buf)
    assert rc == 0 and blob.ver == 2 and blob.n_ops == 99
    rc, inline = parse_blob(cuda, ibuf)
    n_ext = 0
    for i in range(blob.n_slots):
        sl, il = blob.slots[i], inline.slots[i]
        if sl.addr != 0xFFFFFFFC:
            continue
        n_ext += 1
        assert sl.len == il.len and sl.offset + sl.len <= wts.size
        assert np.array_equal(wts[sl.offset: sl.offset + sl.len],
                              ibuf[inline.weight_off + il.offset: inline.weight_off + il.offset + il.len])
    assert n_ext >= 10
    gold = np.load(os.path.join(HERE, "ref_ops.npz"))["op98_t8"]
    eng = Engine(ref, buf)
    with pytest.raises(Exception):
        eng.run_io(ids(), 0)
    ref.wt_exec_set_ext_weights(wts.ctypes.data)
    eng.run_io(ids(), 0)
    assert np.array_equal(eng.temp(man["output_temp"]).view(np.uint16), gold)
    eng.shutdown()


@pytest.mark.gpu
def test_external_weights_v2_blob(cuda, tmp_path):
    """The EXT_WGT / v2 blob through the CUDA engine: refused without the external area, equal
    to the inline blob's logits with it; and through the host runner, which finds
    <blob>.weights.bin beside the blob as the reference's runner does
    (kernels/examples/42_gehtp_runner/main.c:261)."""
    import shutil
    import subprocess
    buf, man = load("probe_ext_v2")
    ibuf, _ = load("probe_noplan")
    wts = np.fromfile(os.path.join(HERE, "probe_ext_v2.weights.bin"), np.uint8)
    want = np.zeros(32 * 256, np.float16)
    eng = Engine(cuda, ibuf)
    eng.run_io(ids(), man["output_temp"], want)
    eng.shutdown()
    cuda.wt_exec_set_ext_weights(None)
    eng = Engine(cuda, buf)
    with pytest.raises(Exception):
        eng.run_io(ids(), man["output_temp"], None)
    eng.shutdown()
    cuda.wt_exec_set_ext_weights(wts.ctypes.data)
    try:
        eng = Engine(cuda, buf)
        got = np.zeros(32 * 256, np.float16)
        eng.run_io(ids(), man["output_temp"], got)
        eng.shutdown()
    finally:
        cuda.wt_exec_set_ext_weights(None)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    check_logits(got, "external weights, v2 blob")

    runner = os.path.join(os.path.dirname(HERE), "..", "..", "gehtp_b200", "gehtp_run")
    for f in ("probe_ext_v2.wtop", "probe_ext_v2.weights.bin", "ids.i32.raw"):
        shutil.copy(os.path.join(HERE, f), tmp_path / f)
    job = tmp_path / "job.txt"
    job.write_text("blob %s\ninput %s\noutput %s\nout_temp %d\nweights_size %d\n" % (
        tmp_path / "probe_ext_v2.wtop", tmp_path / "ids.i32.raw", tmp_path / "out.raw", man["output_temp"], wts.size))
    r = subprocess.run([runner, "job", str(job)], capture_output=True, text=True)
    assert r.returncode == 0 and "[ext-weights]" in r.stdout, r.stdout + r.stderr
    out = np.frombuffer((tmp_path / "out.raw").read_bytes(), np.float16)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16))
