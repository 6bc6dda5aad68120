"""GPU parity of single ops: each case builds a one-op (or few-op) runlist,
runs it through the CUDA library's wt_exec_run_io and through the reference
executor compiled for the host, and compares temps. Byte moves and exact
arithmetic must agree bit for bit; ops with transcendental functions within
one fp16 step (the reference's own per-opcode gates allow 1-2)."""
import numpy as np
import pytest

from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine
from conftest import assert_fp16_close, ulp_diff_f16

pytestmark = pytest.mark.gpu


def run_both(cuda, ref, builder, out_temps, inp=None, dtype=np.uint16):
    buf = builder.build()
    res = []
    for lib in (cuda, ref):
        eng = Engine(lib, buf)
        eng.run_io(inp, out_temps[0], None)
        res.append([eng.temp(t, dtype) for t in out_temps])
        eng.shutdown()
    return res


def rnd16(rng, shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float16)


@pytest.mark.parametrize("sub", list(range(17)))
@pytest.mark.parametrize("n", [7, 1000])
def test_unary(cuda, ref, sub, n):
    rng = np.random.default_rng(100 + sub)
    x = rnd16(rng, n, 2.0)
    x[:3] = [0.0, -0.0, 5.5][:min(3, n)]
    b = BlobBuilder()
    s = b.add_slot(x)
    b.add_op(OP.UNARY, [S(s), 1, n, sub])
    (g,), (r,) = run_both(cuda, ref, b, [1])
    exact = sub in (0, 2, 5, 11, 14, 15, 16)
    tol = 0 if exact else 1
    assert ulp_diff_f16(g, r).max() <= tol


@pytest.mark.parametrize("sub", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("n", [5, 31, 32, 4099])
def test_binary_bit_exact(cuda, ref, sub, n):
    rng = np.random.default_rng(200 + sub)
    a, c = rnd16(rng, n, 3.0), rnd16(rng, n, 3.0)
    c[0] = 0.0
    a[1] = c[1]
    if sub == 5:
        a, c = np.abs(a), np.abs(c)
    b = BlobBuilder()
    sa, sc = b.add_slot(a), b.add_slot(c)
    b.add_op(OP.BINARY, [S(sa), S(sc), 1, n, sub])
    b.add_op(OP.ADD, [S(sa), S(sc), 2, n])
    (g1, g2), (r1, r2) = run_both(cuda, ref, b, [1, 2])
    assert np.array_equal(g1, r1)
    assert np.array_equal(g2, r2)


def test_select(cuda, ref):
    rng = np.random.default_rng(5)
    n = 300
    cond = (rng.random(n) > 0.5).astype(np.float16)
    t, f = rnd16(rng, n), np.array([2.5], np.float16)
    b = BlobBuilder()
    sc, st, sf = b.add_slot(cond), b.add_slot(t), b.add_slot(f)
    b.add_op(OP.BINARY, [S(sc), S(st), S(sf), 1, 8])
    (g,), (r,) = run_both(cuda, ref, b, [1])
    assert np.array_equal(g, r)


@pytest.mark.parametrize("rows,n", [(3, 17), (4, 64), (16, 4096), (1, 32), (2, 8191)])
def test_softmax(cuda, ref, rows, n):
    rng = np.random.default_rng(rows * 1000 + n)
    x = rnd16(rng, (rows, n), 4.0)
    b = BlobBuilder()
    s = b.add_slot(x)
    b.add_op(OP.SOFTMAX, [S(s), 1, rows, n])
    (g,), (r,) = run_both(cuda, ref, b, [1])
    assert ulp_diff_f16(g, r).max() <= 2


@pytest.mark.parametrize("rows,width", [(1, 1024), (512, 1024), (8, 2560), (5, 96), (3, 128)])
def test_rmsnorm2(cuda, ref, rows, width):
    rng = np.random.default_rng(rows + width)
    x = rnd16(rng, (rows, width))
    x[0] *= np.float16(1e-4)   # a tiny row: the case the reference keeps its scalar double path for
    gam = rng.normal(1, 0.1, width).astype(np.float16)
    beta = rng.normal(0, 0.1, width).astype(np.float16)
    b = BlobBuilder()
    sx, sg, sb = b.add_slot(x), b.add_slot(gam), b.add_slot(beta)
    sz = b.add_slot(np.zeros(width, np.float16))
    b.add_op(OP.RMSNORM2, [S(sx), S(sg), S(sz), 1, rows * width])
    b.add_op(OP.RMSNORM2, [S(sx), S(sg), S(sb), 2, rows * width])
    (g1, g2), (r1, r2) = run_both(cuda, ref, b, [1, 2])
    # double sums are reduced in a different order: allow one fp16 step, expect almost none
    for g, r in ((g1, r1), (g2, r2)):
        d = ulp_diff_f16(g, r)
        assert d.max() <= 1 and (d > 0).mean() < 1e-3


MM_CASES = [  # M, K, N, t0, t1, Bn   (shapes of the reference's host GEMV test plus tiles)
    (1, 64, 64, 0, 0, 0), (1, 128, 200, 0, 1, 0), (16, 96, 130, 0, 0, 0), (16, 96, 130, 1, 0, 0),
    (32, 64, 64, 1, 1, 0), (1, 128, 40, 0, 0, 6), (1, 40, 128, 0, 0, 6), (3, 64, 96, 0, 1, 4),
    (130, 70, 90, 0, 0, 0), (64, 128, 64, 0, 0, 2), (2, 1024, 3072, 0, 0, 0),
]


@pytest.mark.parametrize("M,K,N,t0,t1,Bn", MM_CASES)
def test_matmul_f16_bit_exact(cuda, ref, M, K, N, t0, t1, Bn):
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    nb = max(Bn, 1)
    a, w = rnd16(rng, (nb, M, K)), rnd16(rng, (nb, K, N), 0.1)
    if t0:
        a = np.ascontiguousarray(a.transpose(0, 2, 1))
    if t1:
        w = np.ascontiguousarray(w.transpose(0, 2, 1))
    flags = t0 | (t1 << 1) | ((4 | (Bn << 16)) if Bn else 0)
    b = BlobBuilder()
    sa, sw = b.add_slot(a), b.add_slot(w)
    b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, flags])
    cuda.gehtp_cuda_set_fusion(0)          # the one-kernel-per-op plan keeps the reference's ascending-k sums
    try:
        (g,), (r,) = run_both(cuda, ref, b, [1])
    finally:
        cuda.gehtp_cuda_set_fusion(1)
    assert np.array_equal(g, r)


NK_CASES = [  # M, K, N: weights stored [N, K]; M < 32 -> streaming GEMV, M >= 128 -> tcgen05 GEMM, between -> exact kernel
    (1, 128, 200), (3, 1024, 520), (8, 2560, 512), (20, 64, 136), (31, 256, 96), (64, 128, 128),
    (128, 64, 128), (130, 128, 256), (256, 512, 384), (300, 1024, 1280),
    (256, 3072, 512),     # 8 tiles, 48 k blocks: K is split into runs
]


@pytest.mark.parametrize("M,K,N", NK_CASES)
def test_matmul_f16_nk_tensor_paths(cuda, ref, M, K, N):
    """FullyConnected weights as the emitter stores them ([N, K], flags bit 1) under the default plan:
    the fp16 gate against the reference, and bit-equality on small integers, where every summation
    order gives the same fp32 sums (the trick of kernels/host/test_gemv_f16.c)."""
    rng = np.random.default_rng(M + 3 * K + 7 * N)
    for ints in (False, True):
        if ints:
            a = rng.integers(-4, 5, (M, K)).astype(np.float16)
            w = rng.integers(-3, 4, (N, K)).astype(np.float16)
        else:
            a, w = rnd16(rng, (M, K)), rnd16(rng, (N, K), 0.1)
        b = BlobBuilder()
        sa, sw = b.add_slot(a), b.add_slot(w)
        b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, 2])
        (g,), (r,) = run_both(cuda, ref, b, [1])
        if ints:
            assert np.array_equal(g, r)
        else:
            assert_fp16_close(g.view(np.float16), r.view(np.float16), "matmul_f16 [N,K] %dx%dx%d" % (M, K, N))


def test_matmul_f16_nk_split_chunks(cuda, ref):
    """MATMUL_F16_SPLIT over a tensor-core shape: chunks of 128 columns written into rows of N_full."""
    rng = np.random.default_rng(45)
    M, K, N = 256, 256, 384
    a, w = rnd16(rng, (M, K)), rnd16(rng, (N, K), 0.2)
    b = BlobBuilder()
    sa, sw = b.add_slot(a), b.add_slot(w)
    b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, 2])
    for n0 in range(0, N, 128):
        b.add_op(OP.MATMUL_F16_SPLIT, [S(sa), S(sw), 2, M, K, N, n0, 128, 2])
    (g1, g2), (r1, r2) = run_both(cuda, ref, b, [1, 2])
    assert np.array_equal(g1, g2), "chunked and whole tensor-core runs differ"
    assert_fp16_close(g1.view(np.float16), r1.view(np.float16), "split matmul")


def test_matmul_split_equals_whole(cuda, ref):
    """The byte-exact chunked-vs-whole gate of the reference's emitter test."""
    rng = np.random.default_rng(44)
    M, K, N = 32, 64, 160
    a, w = rnd16(rng, (M, K)), rnd16(rng, (N, K), 0.2)
    b = BlobBuilder()
    sa, sw = b.add_slot(a), b.add_slot(w)
    b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, 2])
    for n0 in range(0, N, 64):
        b.add_op(OP.MATMUL_F16_SPLIT, [S(sa), S(sw), 2, M, K, N, n0, min(64, N - n0), 2])
    (g1, g2), (r1, r2) = run_both(cuda, ref, b, [1, 2])
    assert np.array_equal(g1, g2) and np.array_equal(g1, r1) and np.array_equal(g2, r2)


def test_data_movement_ops(cuda, ref):
    rng = np.random.default_rng(9)
    x = rnd16(rng, (6, 8, 10))
    idx = np.array([3, 0, 5, 5], np.int32)
    b = BlobBuilder()
    sx = b.add_slot(x)
    si = b.add_slot(idx, count=4)
    t = iter(range(1, 40))
    outs = []

    def out():
        v = next(t)
        outs.append(v)
        return v
    n = x.size
    b.add_op(OP.TRANSPOSE_GEN, [S(sx), out(), 3, 6, 8, 10, 1, 2 | 0 << 8 | 1 << 16])
    b.add_op(OP.TRANSPOSE_GEN, [S(sx), out(), 2, 48, 10, 1, 1, 1 | 0 << 8])
    b.add_op(OP.SLICE, [S(sx), out(), 3 * 4 * 5, 3, 1, 2, 0, 4, 6, 10, 1, 1, 2, 6, 8, 10])
    b.add_op(OP.SPLIT, [outs[0], out()] + [0] * 7 + [0, 3, 2, 5, 1, 0, 1])
    b.add_op(OP.CONCAT, [S(sx), S(sx), outs[1]] + [0] * 5 + [out(), 0, 3, 3 * n, 10, 10, 10, 0])
    b.add_op(OP.BROADCAST, [S(si), out(), 8 * 8, 8, 1, 1, 1, 8, 1, 1, 8, 8])
    b.add_op(OP.REDUCE, [S(sx), out(), n, 1, 0, 6, 8, 10, 1])
    b.add_op(OP.REDUCE, [S(sx), out(), n, 2, 2, 6, 8, 10, 1])
    b.add_op(OP.REDUCE, [S(sx), out(), n, 0, 1, 6, 8, 10, 1])
    b.add_op(OP.PAD, [S(sx), out(), 48, 10, 16, 3, 0x3C00])
    b.add_op(OP.CUMSUM, [S(sx), out(), 48, 10, 0, 0, 0])
    b.add_op(OP.CUMSUM, [S(sx), out(), 48, 10, 0, 1, 1])
    b.add_op(OP.GATHER, [S(sx), S(si), out(), 4 * 80, 0 | 1 << 8 | 3 << 16, 6, 8, 10, 1, 1, 4, 1, 1, 1, 1])
    b.add_op(OP.ARGMAX, [S(sx), out(), n])
    b.add_op(OP.UNARY, [S(sx), out(), n, 14])
    b.add_op(OP.TRANSPOSE, [S(sx), out(), 6, 8, 10, 0 | 3 << 8 | 1 << 16 | 2 << 24])
    upd = rnd16(rng, (2, 80))
    su = b.add_slot(upd)
    sidx = b.add_slot(np.array([[4], [1]], np.int32), count=2)
    b.add_op(OP.SCATTER_ND, [S(sx), S(sidx), S(su), out(), n, 3, 6, 8, 10, 1, 1, 1, 2, 80])
    g, r = run_both(cuda, ref, b, outs)
    for i, (x1, x2) in enumerate(zip(g, r)):
        assert x1 is not None and np.array_equal(x1, x2), "output %d (temp %d) differs" % (i, outs[i])


def test_reduce_minmax_long_rows_bit_exact(cuda, ref):
    """Max / min over long rows take the CTA-per-row kernel; +0 / -0 ties must resolve as in a sequential scan."""
    rng = np.random.default_rng(12)
    L = 5000
    x = rnd16(rng, (4, L))
    x[1] = -np.abs(x[1]) - 1.0          # max is the least negative
    x[2] = -np.abs(x[2])
    x[2, 777] = np.float16(-0.0)        # -0 first, +0 later: max keeps -0
    x[2, 3000] = np.float16(0.0)
    x[3] = np.abs(x[3])
    x[3, 4000] = np.float16(0.0)        # +0 first, -0 later: min keeps +0
    x[3, 4500] = np.float16(-0.0)
    b = BlobBuilder()
    sx = b.add_slot(x)
    outs = [1, 2]
    b.add_op(OP.REDUCE, [S(sx), 1, x.size, 1, 2, 4, L, 1, 1])
    b.add_op(OP.REDUCE, [S(sx), 2, x.size, 1, 3, 4, L, 1, 1])
    g, r = run_both(cuda, ref, b, outs)
    for x1, x2 in zip(g, r):
        assert x1 is not None and np.array_equal(x1, x2)


def test_kv_ring_append_gather_bit_exact(cuda, ref):
    """KV append -> GQA gather byte round trip, ring wrap, zero tail (test_kv_ssm_ops.c of the reference)."""
    rng = np.random.default_rng(3)
    nh, kvh, hd, nslots = 8, 2, 64, 16
    b = BlobBuilder()
    b.add_states([kvh * hd * 4 * nslots, kvh * hd * 4 * nslots])
    steps = 5
    ks = [b.add_slot(rnd16(rng, kvh * hd)) for _ in range(steps)]
    vs = [b.add_slot(rnd16(rng, kvh * hd)) for _ in range(steps)]
    for i in range(steps):
        b.add_op(OP.KV_APPEND, [S(ks[i]), S(vs[i]), ST(0), KV_POS_AUTO])
        b.add_op(OP.KV_APPEND, [S(ks[i]), S(vs[i]), ST(1), i])
    b.add_op(OP.KV_GATHER, [ST(0), 1, 2, KV_POS_AUTO, nh, kvh, hd])   # AUTO: width nslots, zero tail
    b.add_op(OP.KV_GATHER, [ST(1), 3, 4, steps, nh, kvh, hd])          # explicit: width n_kv
    b.add_op(OP.KV_GATHER, [ST(1), 5, 0, 3, nh, kvh, hd])              # single face
    cuda.wt_exec_state_reset()
    ref.wt_exec_state_reset()
    g, r = run_both(cuda, ref, b, [1, 2, 3, 4, 5])
    for x1, x2 in zip(g, r):
        assert np.array_equal(x1, x2)
    assert g[0].size == nh * hd * nslots


def test_kv_gather_miss_is_an_error(cuda, ref):
    rng = np.random.default_rng(3)
    kvh, hd, nslots = 2, 64, 4
    b = BlobBuilder()
    b.add_states([kvh * hd * 4 * nslots])
    k = b.add_slot(rnd16(rng, kvh * hd))
    b.add_op(OP.KV_APPEND, [S(k), S(k), ST(0), 0])
    b.add_op(OP.KV_APPEND, [S(k), S(k), ST(0), 5])      # wraps onto slot 1, evicting nothing yet
    b.add_op(OP.KV_GATHER, [ST(0), 1, 2, 2, 4, kvh, hd])  # position 1 was never written -> miss
    buf = b.build()
    for lib in (cuda, ref):
        lib.wt_exec_state_reset()
        eng = Engine(lib, buf)
        with pytest.raises(Exception) as ei:
            eng.run()
        assert ei.value.rc == 3 and "kv gather miss" in ei.value.msg
        eng.shutdown()
        lib.wt_exec_state_reset()


def test_conv1d_and_delta(cuda, ref):
    rng = np.random.default_rng(12)
    seq, C, k = 40, 96, 4
    x, w = rnd16(rng, (seq, C)), rnd16(rng, (k, C), 0.5)
    H, D, c, ntok = 3, 128, 20, 40
    kk = rnd16(rng, (H, ntok, D))
    kk = (kk / np.linalg.norm(kk.astype(np.float32), axis=-1, keepdims=True)).astype(np.float16)
    vv, qq = rnd16(rng, (H, ntok, D)), rnd16(rng, (H, ntok, D))
    beta = (1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16)
    gg = np.log(1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16)
    b = BlobBuilder()
    b.add_states([(k - 1) * C * 4, H * D * D * 4])
    sx, sw = b.add_slot(x), b.add_slot(w)
    b.add_op(OP.CONV1D_SSM, [S(sx), sw, 1, seq, C, k])
    xs = [b.add_slot(x[i]) for i in range(3)]
    for i in range(3):
        b.add_op(OP.CONV1D_SSM_STEP, [S(xs[i]), S(sw), 2 + i, ST(0), C, k])
    sl = [b.add_slot(a) for a in (kk, vv, qq, beta, gg)]
    # two chunks of 20 tokens: the second one is addressed by slicing token rows out first
    b.add_op(OP.DELTA_CHUNK, [S(sl[0]), S(sl[1]), S(sl[2]), S(sl[3]), S(sl[4]), 6, ST(1), c, ntok, H, D, 0])
    b.add_op(OP.DELTA_CHUNK, [S(sl[0]), S(sl[1]), S(sl[2]), S(sl[3]), S(sl[4]), 7, ST(1), c, ntok, H, D, 1])
    cuda.wt_exec_state_reset()
    ref.wt_exec_state_reset()
    g, r = run_both(cuda, ref, b, [1, 2, 3, 4, 6, 7])
    assert np.array_equal(g[0], r[0])                       # pure conv: exact products, same order
    for i in (1, 2, 3):
        assert ulp_diff_f16(g[i], r[i]).max() <= 1          # SiLU inside
    for i in (4, 5):                                        # only the first c tokens of each head are written
        gv = g[i].view(np.float16).reshape(H, ntok, D)[:, :c]
        rv = r[i].view(np.float16).reshape(H, ntok, D)[:, :c]
        assert_fp16_close(gv, rv, "delta chunk y")
    cuda.wt_exec_state_reset()
    ref.wt_exec_state_reset()


@pytest.mark.parametrize("H,D,c,nchunks", [(4, 128, 64, 6), (2, 64, 64, 4), (3, 128, 40, 3)])
def test_delta_chunk_tensor_core_form(cuda, ref, H, D, c, nchunks):
    """The mma form of the chunked delta rule (fused plans) against the scalar form (one kernel per op) and the
    reference, over several chunks that carry the fp32 state: y of every chunk within the fp16 gate of the reference,
    within four fp16 steps of the largest output of the scalar form (hi + lo operands keep the products fp32-class; what
    differs is the order of the fp32 sums and where the entries of T below its diagonal blocks are rounded to fp16), and
    the final state equal to the scalar form's to 2e-3 of its largest entry."""
    rng = np.random.default_rng(500 + D + c)
    ntok = c
    b = BlobBuilder()
    b.add_states([H * D * D * 4])
    outs = []
    for ch in range(nchunks):
        kk = rnd16(rng, (H, ntok, D))
        kk = (kk / np.linalg.norm(kk.astype(np.float32), axis=-1, keepdims=True)).astype(np.float16)
        vv, qq = rnd16(rng, (H, ntok, D)), rnd16(rng, (H, ntok, D))
        beta = (1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16)
        gg = np.log(1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16) * np.float16(0.25)
        sl = [b.add_slot(a) for a in (kk, vv, qq, beta, gg)]
        b.add_op(OP.DELTA_CHUNK, [S(sl[0]), S(sl[1]), S(sl[2]), S(sl[3]), S(sl[4]), 1 + ch, ST(0), c, ntok, H, D, ch & 1])
        outs.append(1 + ch)
    buf = b.build()
    res, states = {}, {}
    for name, lib, fusion in (("mma", cuda, 1), ("scalar", cuda, 0), ("ref", ref, None)):
        if fusion is not None:
            cuda.gehtp_cuda_set_fusion(fusion)
        lib.wt_exec_state_reset()
        eng = Engine(lib, buf)
        eng.run_io(None, outs[0], None)
        res[name] = [eng.temp(t).view(np.float16).reshape(H, ntok, D).copy() for t in outs]
        if lib is cuda:
            st = np.zeros(H * D * D, np.float32)
            assert cuda.gehtp_cuda_state_read(0, st.ctypes.data, st.nbytes) == 0
            states[name] = st
        eng.shutdown()
        lib.wt_exec_state_reset()
    cuda.gehtp_cuda_set_fusion(1)
    for ch in range(nchunks):
        assert_fp16_close(res["mma"][ch], res["ref"][ch], "delta chunk %d vs reference" % ch)
        a, sc = res["mma"][ch].astype(np.float64), res["scalar"][ch].astype(np.float64)
        assert np.abs(a - sc).max() <= 2.0 ** -8 * np.abs(sc).max(), ch
    assert np.abs(states["mma"] - states["scalar"]).max() <= 2e-3 * np.abs(states["scalar"]).max()


def test_error_strings_match_reference(cuda, ref):
    """Bad operands are refused before any launch, with the reference's message and op index."""
    cases = []
    b = BlobBuilder(); s = b.add_slot(np.zeros(8, np.float16))
    b.add_op(OP.UNARY, [S(s), 1, 8, 14]); b.add_op(OP.UNARY, [7, 2, 8, 0])      # temp 7 never written
    cases.append((b, 2, "unary ref fail"))
    b = BlobBuilder(); s = b.add_slot(np.zeros(8, np.float16))
    b.add_op(OP.UNARY, [S(s), 1, 8, 99])
    cases.append((b, 1, "unary unknown subtype 99"))
    b = BlobBuilder(); s = b.add_slot(np.zeros(8, np.float16))
    b.add_op(OP.REDUCE, [S(s), 1, 8, 7, 0, 8, 1, 1, 1])
    cases.append((b, 1, "reduce axis/subtype bad (axis=7 sub=0)"))
    b = BlobBuilder(); s = b.add_slot(np.zeros(8, np.float16))
    b.add_op(OP.RMSNORM2, [S(s), S(s), S(s), 1, 12])
    cases.append((b, 1, "rmsnorm2 shape n12 rw8"))
    b = BlobBuilder(); s = b.add_slot(np.zeros(8, np.float16))
    b.add_op(OP.KV_APPEND, [S(s), S(s), 5, 0])
    cases.append((b, 1, "kv state_ref not 0x6000|idx (0x5)"))
    for bld, rc, msg in cases:
        buf = bld.build()
        for lib in (cuda, ref):
            eng = Engine(lib, buf)
            with pytest.raises(Exception) as ei:
                eng.run()
            assert ei.value.rc == rc and ei.value.msg == msg, (ei.value.rc, ei.value.msg)
            eng.shutdown()
