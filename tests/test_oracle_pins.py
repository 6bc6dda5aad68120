"""Pins the C restatement (oracle/liboracle.so) to the reference: bit for bit
against the committed golden vectors (outputs of the reference executor, made by
tests/golden/make_golden.py) and, where the reference library is at hand,
against fresh runs of it on other seeds."""
import os

import numpy as np
import pytest

from gehtp_b200.wtop import OP, S, BlobBuilder, Engine
from oracle.refexec import ptr

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_ops.npz"))


def u16(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.mark.parametrize("name", ["matmul_plain", "matmul_t0", "matmul_t1", "matmul_t0t1", "matmul_batched", "matmul_batched_t1"])
def test_matmul_golden(orc, name):
    a, w = G[name + "/in_a"], G[name + "/in_w"]
    M, K, N, t0, t1, Bn = [int(v) for v in G[name + "/in_dims"]]
    y = np.zeros(max(Bn, 1) * M * N, np.uint16)
    orc.orc_matmul_f16(ptr(a), ptr(w), ptr(y), M, K, N, 0, N, t0, t1, 1 if Bn else 0, max(Bn, 1))
    assert np.array_equal(y, G[name + "/out1"])


def test_rmsnorm_softmax_golden(orc):
    x, g, b = G["rmsnorm2/in_x"], G["rmsnorm2/in_g"], G["rmsnorm2/in_b"]
    y = np.zeros(x.size, np.uint16)
    orc.orc_rmsnorm2(ptr(x), ptr(g), ptr(b), ptr(y), x.shape[0], x.shape[1])
    assert np.array_equal(y, G["rmsnorm2/out1"])
    for name in ("softmax_wide", "softmax_narrow"):
        x = G[name + "/in_x"]
        y = np.zeros(x.size, np.uint16)
        orc.orc_softmax(ptr(x), ptr(y), x.shape[0], x.shape[1])
        assert np.array_equal(y, G[name + "/out1"])


def test_unary_binary_golden(orc):
    x = G["unary/in_x"]
    for sub in range(17):
        y = np.zeros(x.size, np.uint16)
        assert orc.orc_unary(ptr(x), ptr(y), x.size, sub) == 0
        assert np.array_equal(y, G["unary/out%d" % (sub + 1)]), sub
    a, b = G["binary/in_a"], G["binary/in_b"]
    for sub in range(6):
        y = np.zeros(a.size, np.uint16)
        orc.orc_binary(ptr(a), ptr(b), ptr(y), a.size, sub)
        assert np.array_equal(y, G["binary/out%d" % (sub + 1)]), sub


def test_kv_ring_golden(orc):
    k, v = G["kv/in_k"], G["kv/in_v"]
    nh, kvh, hd, nslots = [int(x) for x in G["kv/in_dims"]]
    ring = np.zeros(nslots * kvh * hd * 2, np.uint16)
    posmap = np.full(nslots, 0xFFFFFFFF, np.uint32)
    for i in range(k.shape[0]):
        orc.orc_kv_append(ptr(ring), ptr(posmap), nslots, kvh * hd, ptr(k[i]), ptr(v[i]), i)
    kT = np.zeros(nh * hd * nslots, np.uint16)
    vo = np.zeros(nh * nslots * hd, np.uint16)
    assert orc.orc_kv_gather(ptr(ring), ptr(posmap), nslots, 6, nslots, nh, kvh, hd, ptr(kT), ptr(vo)) == 0
    assert np.array_equal(kT, G["kv/out1"]) and np.array_equal(vo, G["kv/out2"])
    kT5 = np.zeros(nh * hd * 5, np.uint16)
    vo5 = np.zeros(nh * 5 * hd, np.uint16)
    assert orc.orc_kv_gather(ptr(ring), ptr(posmap), nslots, 5, 5, nh, kvh, hd, ptr(kT5), ptr(vo5)) == 0
    assert np.array_equal(kT5, G["kv/out3"]) and np.array_equal(vo5, G["kv/out4"])
    assert orc.orc_kv_gather(ptr(ring), ptr(posmap), nslots, 7, 7, nh, kvh, hd, ptr(kT), ptr(vo)) == -1   # position 6 missing


def test_gdn_golden(orc):
    x, w = G["conv/in_x"], G["conv/in_w"]
    seq, C = x.shape
    y = np.zeros(x.size, np.uint16)
    orc.orc_conv1d_ssm(ptr(x), ptr(w), ptr(y), seq, C, w.shape[0])
    assert np.array_equal(y, G["conv/out1"])
    win = np.zeros((w.shape[0] - 1) * C, np.float32)
    for i in range(4):
        ys = np.zeros(C, np.uint16)
        orc.orc_conv1d_step(ptr(np.ascontiguousarray(x[i])), ptr(w), ptr(ys), ptr(win), C, w.shape[0])
        assert np.array_equal(ys, G["conv/out%d" % (2 + i)])
    H, D, c, ntok = [int(v) for v in G["delta/in_dims"]]
    S_ = np.zeros(H * D * D, np.float32)
    keep = [np.ascontiguousarray(G["delta/in_" + n]) for n in ("k", "v", "q", "beta", "g")]   # keep the arrays alive
    args = [ptr(a) for a in keep]
    for t, q_raw in ((1, 0), (2, 1)):
        y = np.zeros(H * ntok * D, np.uint16)
        assert orc.orc_delta_chunk(*args, ptr(y), ptr(S_), c, ntok, H, D, q_raw) == 0
        got = y.reshape(H, ntok, D)[:, :c]
        want = G["delta/out%d" % t].reshape(H, ntok, D)[:, :c]
        assert np.array_equal(got, want)


def test_delta_chunk_split_consistency(orc):
    """Two chunks of 16 = one chunk of 32 = 32 single-token steps, to fp32
    rounding (the three-way gate of the reference's test_kv_ssm_ops.c)."""
    H, D, c, ntok = [int(v) for v in G["delta/in_dims"]]
    names = ("k", "v", "q", "beta", "g")
    full = {n: G["delta/in_" + n] for n in names}

    def run(chunks):
        S_ = np.zeros(H * D * D, np.float32)
        ys = np.zeros((H, ntok, D), np.float16)
        t0 = 0
        for cl in chunks:
            sub = [np.ascontiguousarray(full[n][:, t0:t0 + cl]) for n in names]
            y = np.zeros(H * cl * D, np.uint16)
            assert orc.orc_delta_chunk(*[ptr(a) for a in sub], ptr(y), ptr(S_), cl, cl, H, D, 0) == 0
            ys[:, t0:t0 + cl] = y.view(np.float16).reshape(H, cl, D)
            t0 += cl
        return ys.astype(np.float64), S_
    y2, S2 = run([16, 16])
    y1, S1 = run([32])
    yt, St = run([1] * 32)
    for ya, Sa in ((y1, S1), (yt, St)):
        assert np.abs(ya - y2).max() <= 2e-2 * np.abs(y2).max()
        assert np.abs(Sa - S2).max() <= 2e-3


def test_fp16_converters_exhaustive(orc):
    bits = np.arange(65536, dtype=np.uint16)
    f = bits.view(np.float16).astype(np.float32)
    for i in range(0, 65536, 257):
        v = orc.orc_f16_to_f32(int(bits[i]))
        assert (np.isnan(v) and np.isnan(f[i])) or v == f[i]
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 2000),
                         np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5], np.float32)])
    for x in xs:
        want = np.float32(x).astype(np.float16).view(np.uint16)
        assert orc.orc_f32_to_f16(float(x)) == int(want), x


def test_w4_dequant_matches_numpy(orc):
    from gehtp_b200.runlists import dequant_f16, rand_w4
    rng = np.random.default_rng(4)
    nib, scales = rand_w4(rng, 128, 48)
    slot = np.concatenate([nib.reshape(-1), scales.view(np.uint8).reshape(-1)])
    w = np.zeros((128, 48), np.float16)
    orc.orc_w4_dequant(ptr(slot), ptr(w), 128, 48)
    assert np.array_equal(u16(w), u16(dequant_f16(nib, scales)))


@pytest.mark.parametrize("seed", [1, 2])
def test_fresh_reference_runs(orc, ref, seed):
    """Other seeds and shapes than the golden file, straight against the reference library."""
    rng = np.random.default_rng(seed)
    M, K, N = 7, 200, 65
    a = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.standard_normal((N, K)).astype(np.float16)
    x = rng.standard_normal((9, 96)).astype(np.float16)
    b = BlobBuilder()
    sa, sw, sx = b.add_slot(a), b.add_slot(w), b.add_slot(x)
    b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, 2])
    b.add_op(OP.SOFTMAX, [S(sx), 2, 9, 96])
    b.add_op(OP.SOFTMAX, [S(sx), 3, 8, 108])
    eng = Engine(ref, b.build())
    eng.run()
    y = np.zeros(M * N, np.uint16)
    orc.orc_matmul_f16(ptr(a), ptr(w), ptr(y), M, K, N, 0, N, 0, 1, 0, 1)
    assert np.array_equal(y, eng.temp(1, np.uint16))
    for t, (rows, n) in ((2, (9, 96)), (3, (8, 108))):
        s = np.zeros(rows * n, np.uint16)
        orc.orc_softmax(ptr(x), ptr(s), rows, n)
        assert np.array_equal(s, eng.temp(t, np.uint16))
    eng.shutdown()
