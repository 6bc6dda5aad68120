"""Decode-state files in the layout of the reference's host golden ("HDS1",
compiler/src/ops/host_decode_state.cpp:14-62): save after some steps, check the
file against the states read back one by one, then reset, load and continue —
the continued run must equal the uninterrupted one bit for bit."""
import struct

import numpy as np
import pytest

from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine, EngineError

pytestmark = pytest.mark.gpu

N_KV, N_CONV, N_DELTA = 6, 18, 18                    # host_decode_state.hpp:18-20
KV_ELEMS, KV_MAX, CONV_C, DC, H, D = 512, 64, 6144, 4, 16, 128
CONV_BYTES, DELTA_BYTES = (DC - 1) * CONV_C * 4, H * D * D * 4
KV_SLOTS = 64
FILE_BYTES = 8 + 4 * N_KV + 2 * N_KV * KV_MAX * KV_ELEMS * 4 + N_CONV * CONV_BYTES + N_DELTA * DELTA_BYTES
KV_STATE, CONV_STATE, DELTA_STATE = 2, N_KV + 3, N_KV + N_CONV + 5
T_KT, T_V, T_CONV, T_DELTA = 1, 2, 3, 4
FACE = [("k", KV_ELEMS), ("v", KV_ELEMS), ("x", CONV_C), ("dk", H * D), ("dv", H * D), ("dq", H * D), ("beta", H), ("g", H)]
FACE_ELEMS = sum(n for _, n in FACE)


def decode_table_runlist(n_states=N_KV + N_CONV + N_DELTA):
    """One step that appends to KV ring 2, steps conv window 3 and delta state 5 (global ids 2, 9, 29)."""
    rng = np.random.default_rng(77)
    b = BlobBuilder()
    face = b.add_ext_in(FACE_ELEMS * 2)
    sizes = [KV_SLOTS * KV_ELEMS * 4] * N_KV + [CONV_BYTES] * N_CONV + [DELTA_BYTES] * N_DELTA
    b.add_states(sizes[:n_states])
    w = b.add_slot((rng.standard_normal((DC, CONV_C)) * 0.5).astype(np.float16))
    part, off, t = {}, 0, 10
    for name, n in FACE:
        b.add_op(OP.SLICE, [S(face), t, n, 1, off, 0, 0, off + n, 0, 0, 1, 1, 1, FACE_ELEMS, 1, 1])
        part[name], off, t = t, off + n, t + 1
    b.add_op(OP.KV_APPEND, [part["k"], part["v"], ST(KV_STATE), KV_POS_AUTO])
    b.add_op(OP.KV_GATHER, [ST(KV_STATE), T_KT, T_V, KV_POS_AUTO, 4, 2, 256])
    b.add_op(OP.CONV1D_SSM_STEP, [part["x"], S(w), T_CONV, ST(CONV_STATE), CONV_C, DC])
    b.add_op(OP.DELTA_CHUNK, [part["dk"], part["dv"], part["dq"], part["beta"], part["g"], T_DELTA, ST(DELTA_STATE), 1, 1, H, D, 0])
    return b.build()


def step_input(rng):
    f = {n: rng.standard_normal(c).astype(np.float32) for n, c in FACE}
    dk = f["dk"].reshape(H, D)
    f["dk"] = (dk / np.linalg.norm(dk, axis=-1, keepdims=True)).reshape(-1)
    f["beta"] = 1.0 / (1.0 + np.exp(-f["beta"]))
    f["g"] = np.log(1.0 / (1.0 + np.exp(-f["g"])))
    return np.concatenate([f[n] for n, _ in FACE]).astype(np.float16)


def run_steps(eng, inputs):
    outs = []
    for x in inputs:
        eng.run_io(x, T_KT)
        outs.append([eng.temp(t, np.uint16) for t in (T_KT, T_V, T_CONV, T_DELTA)])
    return outs


def read_state(lib, idx, nbytes):
    buf = np.zeros(nbytes, np.uint8)
    assert lib.gehtp_cuda_state_read(idx, buf.ctypes.data, nbytes) == 0
    return buf


def test_state_file_round_trip(cuda, tmp_path):
    rng = np.random.default_rng(5)
    inputs = [step_input(rng) for _ in range(8)]
    path = tmp_path / "decode.hds1"
    cuda.wt_exec_state_reset()
    eng = Engine(cuda, decode_table_runlist())
    assert eng.state_load_hds1(path) == 1                     # no file yet: states stay zero
    run_steps(eng, inputs[:5])
    eng.state_save_hds1(path)
    raw = path.read_bytes()
    assert len(raw) == FILE_BYTES and raw[:4] == b"HDS1"
    assert struct.unpack_from("<I", raw, 4)[0] == N_KV + N_CONV + N_DELTA
    counts = struct.unpack_from("<%dI" % N_KV, raw, 8)
    assert counts == tuple(5 if i == KV_STATE else 0 for i in range(N_KV))
    off = 8 + 4 * N_KV
    kf = np.frombuffer(raw, np.float32, N_KV * KV_MAX * KV_ELEMS, off).reshape(N_KV, KV_MAX, KV_ELEMS)
    off += kf.nbytes
    vf = np.frombuffer(raw, np.float32, N_KV * KV_MAX * KV_ELEMS, off).reshape(N_KV, KV_MAX, KV_ELEMS)
    off += vf.nbytes
    for p in range(5):                                        # position p holds the k and v faces of step p
        assert np.array_equal(kf[KV_STATE, p], inputs[p][:KV_ELEMS].astype(np.float32))
        assert np.array_equal(vf[KV_STATE, p], inputs[p][KV_ELEMS:2 * KV_ELEMS].astype(np.float32))
    assert not kf[KV_STATE, 5:].any() and not kf[:KV_STATE].any() and not vf[KV_STATE + 1:].any()
    conv = np.frombuffer(raw, np.uint8, N_CONV * CONV_BYTES, off).reshape(N_CONV, CONV_BYTES)
    off += conv.nbytes
    delta = np.frombuffer(raw, np.uint8, N_DELTA * DELTA_BYTES, off).reshape(N_DELTA, DELTA_BYTES)
    assert np.array_equal(conv[CONV_STATE - N_KV], read_state(cuda, CONV_STATE, CONV_BYTES))
    assert np.array_equal(delta[DELTA_STATE - N_KV - N_CONV], read_state(cuda, DELTA_STATE, DELTA_BYTES))
    win = conv[CONV_STATE - N_KV].view(np.float32).reshape(DC - 1, CONV_C)   # window rows, oldest first
    x0 = 2 * KV_ELEMS
    for i in range(DC - 1):
        assert np.array_equal(win[i], inputs[2 + i][x0:x0 + CONV_C].astype(np.float32))
    assert not conv[0].any() and not delta[0].any()
    # delta state rows are the value dimension, columns the key dimension (host_decode_delta_step,
    # host_decode_state.cpp:130-154): S *= e^g; S += beta (v - S k) k^T
    Sref = np.zeros((H, D, D))
    o = 2 * KV_ELEMS + CONV_C
    for x in inputs[:5]:
        f = x.astype(np.float64)
        dk, dv = f[o:o + H * D].reshape(H, D), f[o + H * D:o + 2 * H * D].reshape(H, D)
        beta, g = f[o + 3 * H * D:o + 3 * H * D + H], f[o + 3 * H * D + H:o + 3 * H * D + 2 * H]
        for h in range(H):
            Sref[h] *= np.exp(g[h])
            Sref[h] += np.outer(beta[h] * (dv[h] - Sref[h] @ dk[h]), dk[h])
    Sdev = delta[DELTA_STATE - N_KV - N_CONV].view(np.float32).reshape(H, D, D)
    assert np.abs(Sdev - Sref).max() <= 1e-4 * np.abs(Sref).max()

    straight = run_steps(eng, inputs[5:])
    eng.state_reset()
    assert eng.state_load_hds1(path) == 0
    resumed = run_steps(eng, inputs[5:])
    for a, b2 in zip(straight, resumed):
        for x, y in zip(a, b2):
            assert x is not None and np.array_equal(x, y)
    eng.shutdown()
    cuda.wt_exec_state_reset()


def test_state_file_refusals(cuda, tmp_path):
    cuda.wt_exec_state_reset()
    eng = Engine(cuda, decode_table_runlist())
    rng = np.random.default_rng(6)
    run_steps(eng, [step_input(rng)])
    before = read_state(cuda, DELTA_STATE, DELTA_BYTES)
    bad = tmp_path / "bad.hds1"
    bad.write_bytes(b"HDS0" + bytes(64))
    with pytest.raises(EngineError, match="state file"):
        eng.state_load_hds1(bad)
    short = tmp_path / "short.hds1"
    short.write_bytes(b"HDS1" + struct.pack("<I", 42) + bytes(100))
    with pytest.raises(EngineError, match="state file"):
        eng.state_load_hds1(short)
    assert np.array_equal(before, read_state(cuda, DELTA_STATE, DELTA_BYTES))     # a refused file changes nothing
    eng.shutdown()
    cuda.wt_exec_state_reset()
    small = Engine(cuda, decode_table_runlist(n_states=30))   # not the 42-state decode table
    with pytest.raises(EngineError, match="42 states"):
        small.state_save_hds1(tmp_path / "x.hds1")
    small.shutdown()
    cuda.wt_exec_state_reset()


def test_runner_carries_a_sequence_across_processes(tmp_path):
    """`state_file` in the runner's job file: 5 steps in one process and 3 in the next equal 8 in one."""
    import os
    import subprocess
    runner = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gehtp_b200", "gehtp_run")
    rng = np.random.default_rng(9)
    inputs = [step_input(rng) for _ in range(8)]
    blob = tmp_path / "decode.wtop"
    blob.write_bytes(decode_table_runlist().tobytes())

    def job(tag, xs, state):
        for i, x in enumerate(xs):
            (tmp_path / ("%s.in.%d" % (tag, i))).write_bytes(x.tobytes())
        text = "blob %s\ninput %s\noutput %s\nout_temp %d\nsteps %d\n" % (
            blob, tmp_path / (tag + ".in"), tmp_path / (tag + ".out"), T_DELTA, len(xs))
        if state:
            text += "state_file %s\n" % state
        (tmp_path / (tag + ".job")).write_text(text)
        r = subprocess.run([runner, "job", str(tmp_path / (tag + ".job"))], capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        return [(tmp_path / ("%s.out.%d" % (tag, i))).read_bytes() for i in range(len(xs))], r.stdout

    whole, _ = job("whole", inputs, None)
    state = tmp_path / "seq.hds1"
    first, log1 = job("first", inputs[:5], state)
    assert "absent, states start at zero" in log1 and "[state] saved" in log1 and state.stat().st_size == FILE_BYTES
    second, log2 = job("second", inputs[5:], state)
    assert "[state] loaded" in log2
    assert first + second == whole
