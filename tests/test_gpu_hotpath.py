"""GPU parity of the hot path: W4A16 matmul (group-64), decode attention over
the KV ring, and whole decode runlists, all through the C-ABI of
libgehtp_cuda.so, against the CPU oracle on the same seeded inputs.

Gate for fp16 results (stated by the project): max |err| <= 1e-2 * max|ref| and
cosine >= 0.9999; int4 unpacking and KV indexing are bit-exact."""
import ctypes

import numpy as np
import pytest

from gehtp_b200.runlists import (DecoderConfig, build_decode_runlist, build_prefill_runlist, decode_face,
                                 dequant_f16, nib_to_q, rand_w4)
from gehtp_b200.wtop import OP, S, BlobBuilder, Engine, pack_w4a16
from conftest import assert_fp16_close
from oracle.refexec import ptr

pytestmark = pytest.mark.gpu


def slot_bytes(nib, scales):
    return np.concatenate([nib.reshape(-1), scales.view(np.uint8).reshape(-1)])


@pytest.mark.parametrize("K,N", [(64, 16), (128, 48), (1024, 3072), (2560, 1024)])
def test_w4_unpack_bit_exact(cuda, orc, K, N):
    rng = np.random.default_rng(K + N)
    nib, scales = rand_w4(rng, K, N)
    got = np.zeros((K, N), np.int8)
    assert cuda.gehtp_w4a16_unpack(ptr(nib), ptr(got), K, N) == 0, cuda.gehtp_cuda_last_error()
    want = np.zeros((K, N), np.int8)
    orc.orc_w4_unpack_i8(ptr(nib), ptr(want), K, N)
    assert np.array_equal(got, want)
    assert np.array_equal(want, nib_to_q(nib).astype(np.int8) - 8)
    assert np.array_equal(np.frombuffer(pack_w4a16(nib_to_q(nib), scales), np.uint8), slot_bytes(nib, scales))


W4_SHAPES = [(1, 1024, 3072), (1, 64, 16), (3, 192, 80), (8, 2560, 2048), (16, 1024, 1024), (40, 512, 256),
             (128, 1024, 3072), (256, 512, 384), (130, 320, 272)]


@pytest.mark.parametrize("M,K,N", W4_SHAPES)
def test_w4a16_matmul_vs_oracle(cuda, orc, M, K, N):
    """Config 1 of the baseline (M128 K1024 N3072, seed 1001) and the GEMV / ragged shapes around it."""
    rng = np.random.default_rng(1001)
    a = rng.standard_normal((M, K)).astype(np.float16)
    nib, scales = rand_w4(rng, K, N)
    slot = slot_bytes(nib, scales)
    got = np.zeros((M, N), np.float16)
    assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(got), M, K, N, 0) == 0, cuda.gehtp_cuda_last_error()
    want = np.zeros((M, N), np.float16)
    orc.orc_w4a16_matmul(ptr(a), ptr(slot), ptr(want), M, K, N)
    assert_fp16_close(got, want, "w4a16 %dx%dx%d" % (M, K, N))


# the last two shapes give a CTA more than one tile (both TMEM accumulator buffers in use),
# with one and with two 128-row halves per tile; M = 1000 leaves a ragged last tile
@pytest.mark.parametrize("M,K,N", [(128, 1024, 3072), (128, 64, 128), (256, 512, 384), (200, 2560, 1280), (512, 1024, 4096),
                                   (640, 256, 6144), (1000, 512, 5120), (2304, 256, 5120), (512, 3072, 1024), (64, 2560, 1024)])
def test_w4a16_tcgen05_gemm_vs_oracle(cuda, orc, M, K, N):
    """The tensor-core (tcgen05 / TMEM) path on its own, config 1 of the baseline first."""
    rng = np.random.default_rng(1001)
    a = rng.standard_normal((M, K)).astype(np.float16)
    nib, scales = rand_w4(rng, K, N)
    slot = slot_bytes(nib, scales)
    got = np.zeros((M, N), np.float16)
    assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(got), M, K, N, 2) == 0, cuda.gehtp_cuda_last_error()
    want = np.zeros((M, N), np.float16)
    orc.orc_w4a16_matmul(ptr(a), ptr(slot), ptr(want), M, K, N)
    assert_fp16_close(got, want, "tcgen05 w4a16 %dx%dx%d" % (M, K, N))
    skinny = np.zeros((M, N), np.float16)
    assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(skinny), M, K, N, 1) == 0
    assert_fp16_close(got, skinny, "tcgen05 vs streaming kernel")
    # Every tile configuration walks K in the same order, so configurations that give every SM a tile agree bit for
    # bit; with fewer tiles than SMs K is cut into runs (split K, the cut depends on the tile count) and the fp32
    # partial sums meet in another order: the fp16 gate then.
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for path in (3, 4, 5):
        if path == 5 and N % 256:
            continue
        other = np.zeros((M, N), np.float16)
        assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(other), M, K, N, path) == 0, cuda.gehtp_cuda_last_error()
        rows = 128 if path == 3 else 256
        cols = 256 if path == 5 else 128
        fewest = -(-M // 256) * (N // 256) if N % 256 == 0 else -(-M // 256) * (N // 128)
        if fewest >= sms:
            assert np.array_equal(other.view(np.uint16), got.view(np.uint16)), "tile configuration %d differs" % path
        else:
            assert_fp16_close(other, want, "tile configuration %d (%d x %d)" % (path, rows, cols))
    # twice the same call: the same bits (the runs are added in run order)
    again = np.zeros((M, N), np.float16)
    assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(again), M, K, N, 2) == 0
    assert np.array_equal(again.view(np.uint16), got.view(np.uint16))


def test_w4a16_exact_on_small_integers(cuda, orc):
    """With integer activations and power-of-two scales every product and sum is
    exact in fp32, so the result must equal the oracle bit for bit whatever the
    summation order (the trick of the reference's host GEMV test)."""
    rng = np.random.default_rng(7)
    M, K, N = 5, 256, 64
    a = rng.integers(-3, 4, (M, K)).astype(np.float16)
    nib = rng.integers(0, 256, (K, N // 2), dtype=np.uint8)
    scales = np.full((K // 64, N), 0.5, np.float16)
    slot = slot_bytes(nib, scales)
    got = np.zeros((M, N), np.float16)
    want = np.zeros((M, N), np.float16)
    assert cuda.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(got), M, K, N, 1) == 0
    orc.orc_w4a16_matmul(ptr(a), ptr(slot), ptr(want), M, K, N)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def make_ring(rng, nslots, kvh, hd, n_kv):
    ring = np.zeros((nslots, 2, kvh * hd), np.float16)
    ring[:n_kv] = rng.standard_normal((n_kv, 2, kvh * hd)).astype(np.float16)
    return ring


@pytest.mark.parametrize("nh,kvh,hd,n_kv,nslots", [(16, 8, 128, 4096, 4096), (32, 8, 128, 1000, 1024),
                                                    (4, 4, 64, 70, 128), (8, 2, 128, 1, 64), (64, 16, 128, 333, 512)])
def test_attn_decode_vs_chain_and_f64(cuda, orc, nh, kvh, hd, n_kv, nslots):
    """Config 2 of the baseline (16 q / 8 kv heads, hd 128, ctx 4096, seed 1002) and ragged variants.
    The fused kernel must meet the gate against the op chain and be no less
    accurate than the chain when both are measured against float64."""
    rng = np.random.default_rng(1002)
    q = rng.standard_normal((nh, hd)).astype(np.float16)
    ring = make_ring(rng, nslots, kvh, hd, n_kv)
    mask = np.zeros(n_kv, np.float16)
    if n_kv > 8:
        mask[rng.integers(0, n_kv, 5)] = -np.inf
    scale = float(np.float16(1 / np.sqrt(hd)))
    got = np.zeros((nh, hd), np.float16)
    rc = cuda.gehtp_attn_decode(ptr(q), ptr(ring), ptr(mask), ptr(got), nh, kvh, hd, n_kv, nslots, scale)
    assert rc == 0, cuda.gehtp_cuda_last_error()
    chain = np.zeros((nh, hd), np.float16)
    posmap = np.arange(nslots, dtype=np.uint32)
    assert orc.orc_attn_decode_chain(ptr(q), ptr(ring), ptr(posmap), nslots, n_kv, nh, kvh, hd, scale, 0, ptr(mask), ptr(chain)) == 0
    exact = np.zeros((nh, hd), np.float64)
    orc.orc_attn_decode_f64(ptr(q), ptr(ring), nslots, n_kv, nh, kvh, hd, scale, ptr(mask), ptr(exact))
    assert_fp16_close(got, chain, "fused vs chain")
    e_fused = np.abs(got.astype(np.float64) - exact).max()
    e_chain = np.abs(chain.astype(np.float64) - exact).max()
    assert e_fused <= 1.5 * e_chain + 1e-3, (e_fused, e_chain)


TINY = DecoderConfig(256, 2, 4, 2, 128, 512, 1024, 1e6, "tiny")


def run_decode(lib, buf, man, cfg, steps, fuse=None, graph=None, tokens=None):
    if fuse is not None:
        lib.gehtp_cuda_set_fusion(fuse)
    if graph is not None:
        lib.gehtp_cuda_set_graph(graph)
    lib.wt_exec_state_reset()
    eng = Engine(lib, buf)
    B = man["B"]
    logits, toks = [], []
    for pos in range(steps):
        ids = tokens[pos] if tokens is not None else [(7 * pos + 3 * b + 1) % 1000 for b in range(B)]
        face = decode_face(man, ids, pos, cfg.head_dim, cfg.rope_theta)
        out = np.zeros(2 * B, np.uint16)
        eng.run_io(face, man["token_temp"], out)
        toks.append(out.view(np.int32).copy())
        logits.append(eng.temp(man["logits_temp"]).reshape(B, -1).copy())
    eng.shutdown()
    lib.wt_exec_state_reset()
    return logits, toks


@pytest.mark.parametrize("B", [1, 3, 20])      # 20 rows: the two-row-tile forms of the GEMV and of the dual SwiGLU GEMV
def test_decode_runlist_matches_reference(cuda, ref, B):
    """A decoder decode runlist (W4A16 weights) on the GPU, fused and op-by-op,
    against the same graph with dequantised weights on the reference executor."""
    steps, nslots = 5, 64
    buf_w4, man = build_decode_runlist(TINY, B, nslots, seed=11, quant="w4")
    buf_f16, man2 = build_decode_runlist(TINY, B, nslots, seed=11, quant="f16")
    assert man["token_temp"] == man2["token_temp"]
    r_logits, r_toks = run_decode(ref, buf_f16, man2, TINY, steps)
    for fuse, graph in ((0, 0), (1, 0), (1, 1)):
        g_logits, g_toks = run_decode(cuda, buf_w4, man, TINY, steps, fuse=fuse, graph=graph)
        for s in range(steps):
            assert_fp16_close(g_logits[s], r_logits[s], "logits step %d fuse=%d graph=%d" % (s, fuse, graph))
    cuda.gehtp_cuda_set_fusion(1)
    cuda.gehtp_cuda_set_graph(1)


def test_decode_wide_qkv_projection_takes_rotary_epilogue(cuda, ref):
    """With 48 heads of 128 (6144 columns) the q|k|v projection is wide enough for the variant whose
    epilogue applies the rotary embedding and appends to the KV ring; one more op is then fused."""
    cfg = DecoderConfig(512, 1, 32, 8, 128, 512, 512, 1e6, "wide-heads")
    B, steps, nslots = 2, 3, 32
    buf_w4, man = build_decode_runlist(cfg, B, nslots, seed=13, quant="w4")
    buf_f16, man2 = build_decode_runlist(cfg, B, nslots, seed=13, quant="f16")
    r_logits, _ = run_decode(ref, buf_f16, man2, cfg, steps)
    g_logits, _ = run_decode(cuda, buf_w4, man, cfg, steps, fuse=1, graph=1)
    fused_with = cuda.gehtp_cuda_fused_ops()
    u_logits, _ = run_decode(cuda, buf_w4, man, cfg, steps, fuse=0, graph=0)
    for s in range(steps):
        assert_fp16_close(g_logits[s], r_logits[s], "logits step %d" % s)
        # the epilogue keeps every rounding point of the op chain: fused and op-by-op agree bit for bit
        assert np.array_equal(g_logits[s].view(np.uint16), u_logits[s].view(np.uint16)) or \
            np.abs(g_logits[s].astype(np.float32) - u_logits[s].astype(np.float32)).max() <= 1e-2 * np.abs(u_logits[s]).max()
    assert fused_with >= 25 + 1 + 5 + 2 + 2      # attention chain + its projection, SwiGLU, two add+norm pairs
    cuda.gehtp_cuda_set_fusion(1)
    cuda.gehtp_cuda_set_graph(1)


def test_run_range_pieces_equal_whole_run(cuda):
    """Whole-step run vs one run_range call per op: every temp byte-identical
    (the reference's on-device gate 30)."""
    buf, man = build_decode_runlist(TINY, 2, 32, seed=5, quant="w4")
    cuda.gehtp_cuda_set_fusion(0)
    cuda.gehtp_cuda_set_graph(0)
    face = decode_face(man, [3, 4], 0, TINY.head_dim, TINY.rope_theta)
    temps = {}
    for mode in ("whole", "pieces"):
        cuda.wt_exec_state_reset()
        eng = Engine(cuda, buf)
        if mode == "whole":
            eng.run_io(face, man["token_temp"], None)
        else:
            # EXT_IN data must be resident for piecewise runs: bake the face through one run_io first
            eng.run_io(face, man["token_temp"], None)
            cuda.wt_exec_state_reset()
            for i in range(man["n_ops"]):
                eng.run_range(i, 1)
        temps[mode] = [eng.temp(t, np.uint16) for t in range(1, man["token_temp"] + 1)]
        eng.shutdown()
    for a, b in zip(temps["whole"], temps["pieces"]):
        assert (a is None and b is None) or np.array_equal(a, b)
    cuda.gehtp_cuda_set_fusion(1)
    cuda.gehtp_cuda_set_graph(1)
    cuda.wt_exec_state_reset()


def test_fused_plan_survives_piecewise_and_hooked_runs(cuda):
    """With fusion on, chains run as single kernels and their inner temps have
    no memory; asking for one of those ops alone makes the engine plan again
    unfused, and results stay the same."""
    buf, man = build_decode_runlist(TINY, 2, 32, seed=5, quant="w4")
    face = decode_face(man, [3, 4], 0, TINY.head_dim, TINY.rope_theta)
    cuda.gehtp_cuda_set_fusion(1)
    cuda.gehtp_cuda_set_graph(0)
    cuda.wt_exec_state_reset()
    eng = Engine(cuda, buf)
    eng.run_io(face, man["token_temp"], None)
    assert cuda.gehtp_cuda_fused_ops() >= TINY.layers * (25 + 5 + 2)
    fused_logits = eng.temp(man["logits_temp"]).copy()
    cuda.wt_exec_state_reset()
    for i in range(man["n_ops"]):
        eng.run_range(i, 1)
    assert cuda.gehtp_cuda_fused_ops() == 0
    piece_logits = eng.temp(man["logits_temp"]).copy()
    eng.shutdown()
    cuda.wt_exec_state_reset()
    assert_fp16_close(fused_logits, piece_logits, "fused vs piecewise")
    cuda.gehtp_cuda_set_graph(1)


@pytest.mark.parametrize("seq", [48, 200])
def test_prefill_runlist_matches_reference(cuda, ref, seq):
    """Causal prefill (rotary and attention chains fused into their kernels) against the
    reference executor on the same graph with dequantised weights; 200 tokens span
    several 64-row tiles with a ragged last one and skipped (fully masked) tiles."""
    cfg = DecoderConfig(256, 2, 4, 2, 128, 512, 512, 1e6, "tiny")
    buf_w4, man = build_prefill_runlist(cfg, seq, seed=21, quant="w4")
    buf_f16, man2 = build_prefill_runlist(cfg, seq, seed=21, quant="f16")
    ids = (np.arange(seq, dtype=np.int32) * 37 + 11) % cfg.vocab
    outs = []
    for lib, buf, m in ((cuda, buf_w4, man), (ref, buf_f16, man2)):
        eng = Engine(lib, buf)
        eng.run_io(ids, m["logits_temp"], None)
        outs.append(eng.temp(m["logits_temp"]).reshape(seq, -1))
        eng.shutdown()
    assert_fp16_close(outs[0], outs[1], "prefill logits")
    assert (outs[0].argmax(1) == outs[1].argmax(1)).mean() > 0.9
    # 2 layers x (3 splits + 2 rotary chains of 7 ops in one kernel, the attention chain of 9 ops, the 5-op
    # SwiGLU: one GEMV up to 64 rows, two GEMMs + one elementwise kernel beyond) must have been replaced
    assert cuda.gehtp_cuda_fused_ops() >= 2 * (17 + 9 + 5)
    # and the op-by-op plan gives the same answer within the same gate
    cuda.gehtp_cuda_set_fusion(0)
    eng = Engine(cuda, buf_w4)
    eng.run_io(ids, man["logits_temp"], None)
    unfused = eng.temp(man["logits_temp"]).reshape(seq, -1).copy()
    eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    assert_fp16_close(outs[0], unfused, "fused vs op-by-op prefill")


def test_kernel_family_switches_agree(cuda, tmp_path):
    """The environment switches that put an older kernel form back in (read once per process, hence child processes):
    prefill attention on mma.sync instead of tcgen05 ($GEHTP_CUDA_PREFILL_SM100=0) and the W4A16 GEMM without split K
    ($GEHTP_CUDA_SPLITK=0). Each gives the logits of the default build within the fp16 gate, and not the same bits
    (so the switch did change the kernel)."""
    import os
    import subprocess
    import sys
    script = (
        "import sys, numpy as np\n"
        "sys.path.insert(0, %r)\n"
        "import gehtp_b200\n"
        "from gehtp_b200.runlists import DecoderConfig, build_prefill_runlist\n"
        "from gehtp_b200.wtop import Engine\n"
        "cfg = DecoderConfig(1024, 1, 8, 4, 128, 2048, 512, 1e6, 'switch')   # K = 2048 of the down projection: 32 k blocks on 16 tiles, split\n"
        "buf, man = build_prefill_runlist(cfg, 200, seed=21, quant='w4')\n"
        "ids = (np.arange(200, dtype=np.int32) * 37 + 11) %% cfg.vocab\n"
        "eng = Engine(gehtp_b200.lib(), buf)\n"
        "eng.run_io(ids, man['logits_temp'], None)\n"
        "np.save(sys.argv[1], eng.temp(man['logits_temp']).copy())\n"
        "eng.shutdown()\n") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = {}
    for name, env in (("default", {}), ("mma_attention", {"GEHTP_CUDA_PREFILL_SM100": "0"}), ("no_split_k", {"GEHTP_CUDA_SPLITK": "0"})):
        out = tmp_path / (name + ".npy")
        r = subprocess.run([sys.executable, "-c", script, str(out)], env=dict(os.environ, **env), capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        outs[name] = np.load(out)
    for name in ("mma_attention", "no_split_k"):
        assert_fp16_close(outs[name], outs["default"], name)
        assert not np.array_equal(outs[name].view(np.uint16), outs["default"].view(np.uint16)), name + ": the switch changed nothing"


@pytest.mark.parametrize("tokens,F,hd", [(70, 512, 128), (133, 512, 128), (300, 9728, 128), (133, 320, 128), (70, 512, 24)])
def test_prefill_split_rotary_and_swiglu_tail_bit_equal(cuda, tokens, F, hd):
    """The head of a prefill block (3 SPLITs + 2 rotary chains, 17 ops, one kernel) and a SwiGLU over
    64 rows or more keep every fp16 rounding point of the ops they replace: fused and op-by-op plans agree
    bit for bit. The SwiGLU runs as one tcgen05 launch (gate and up accumulators side by side in TMEM, the
    three elementwise ops in the epilogue; 128-row tiles, and 256-row tiles at the 9728-wide case) or, where
    the width is no multiple of 128 (320), as two GEMMs and one elementwise kernel. Head size 24 takes the split +
    rotary kernel's 4-byte form, the others its 16-byte form."""
    from gehtp_b200.runlists import Emitter, rand_w4, rope_tables
    rng = np.random.default_rng(31)
    H, nh, kvh = 256, 4, 2
    e = Emitter("w4")
    face = e.b.add_ext_in(tokens * H * 2)
    cos, sin = rope_tables(hd, np.arange(tokens), 1e6)
    cq, sq = (S(e.b.add_slot(np.repeat(t, nh, axis=0))) for t in (cos, sin))
    ck, sk = (S(e.b.add_slot(np.repeat(t, kvh, axis=0))) for t in (cos, sin))
    qkv = e.linear(S(face), *rand_w4(rng, H, (nh + 2 * kvh) * hd), tokens)
    sizes = [nh * hd, kvh * hd, kvh * hd]
    q = e.rope(e.split(qkv, sizes, 0), tokens * nh, hd, cq, sq)
    k = e.rope(e.split(qkv, sizes, 1), tokens * kvh, hd, ck, sk)
    v = e.split(qkv, sizes, 2)
    d = e.swiglu(S(face), tokens, rand_w4(rng, H, F), rand_w4(rng, H, F), rand_w4(rng, F, H))
    buf = e.b.build()
    x = rng.standard_normal((tokens, H)).astype(np.float16)
    res = []
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        eng.run_io(x, d, None)
        res.append([eng.temp(t, np.uint16).copy() for t in (q, k, v, d)])
        if fusion:
            assert cuda.gehtp_cuda_fused_ops() == 17 + 5
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    for a, b2, name in zip(res[0], res[1], "qkvd"):
        assert a.size and np.array_equal(a, b2), name


@pytest.mark.parametrize("M,K,F", [(64, 64, 128), (65, 128, 256), (257, 64, 128), (128, 2560, 256), (384, 192, 9728)])
def test_gate_up_gemm_edge_shapes_bit_equal(cuda, M, K, F):
    """The gate | up GEMM at its smallest shape (64 rows, one k block, one tile), with ragged last row tiles, a long K
    and enough tiles for the 256-row form: the fused plan's SwiGLU output agrees bit for bit with the op-by-op plan
    wherever the two separate GEMMs of that plan walk K in one run (fewer than 8 k blocks: nothing to split). With
    a long K and two tiles they split K into runs and add fp32 partial sums in another order than the one-launch
    form does: the fp16 gate there."""
    from gehtp_b200.runlists import Emitter, rand_w4
    rng = np.random.default_rng(5)
    e = Emitter("w4")
    face = e.b.add_ext_in(M * K * 2)
    d = e.swiglu(S(face), M, rand_w4(rng, K, F), rand_w4(rng, K, F), rand_w4(rng, F, 64))
    act = d - 1            # the SwiGLU product feeding the down projection (the temp made right before its output)
    buf = e.b.build()
    x = rng.standard_normal((M, K)).astype(np.float16)
    res = []
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        eng.run_io(x, d, None)
        res.append([eng.temp(t, np.uint16).copy() for t in (act, d)])
        if fusion:
            assert cuda.gehtp_cuda_fused_ops() == 5
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    for a, b2, name in zip(res[0], res[1], ("swiglu", "down")):
        assert a.size == b2.size and a.size
        if K // 64 < 8:
            assert np.array_equal(a, b2), name
        else:
            assert_fp16_close(a.view(np.float16), b2.view(np.float16), name)
    assert np.isfinite(res[0][0].view(np.float16).astype(np.float32)).all()


@pytest.mark.parametrize("H,rows,D,N", [(4, 64, 64, 128), (16, 64, 128, 1024), (3, 200, 128, 256)])
def test_gemm_reads_per_head_tensor_without_transposition(cuda, H, rows, D, N):
    """[heads][rows][d] -> TRANSPOSE_GEN -> W4A16 GEMM at GEMM row counts: the fused plan gives the GEMM the
    untransposed tensor through a three-dimensional tensor map (one box of 64 columns lies in one head). Bit for bit
    the op-by-op plan's result; the second shape is the out-projection of the delta-rule layer."""
    from gehtp_b200.runlists import Emitter, rand_w4
    rng = np.random.default_rng(21)
    e = Emitter("w4")
    face = e.b.add_ext_in(H * rows * D * 2)
    x = e.face(S(face), 0, H * rows * D, H * rows * D)
    xt = e.transpose3(x, (H, rows, D), (1, 0, 2))
    y = e.linear(xt, *rand_w4(rng, H * D, N), rows)
    buf = e.b.build()
    inp = rng.standard_normal(H * rows * D).astype(np.float16)
    res = []
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        eng.run_io(inp, y, None)
        res.append(eng.temp(y, np.uint16).copy())
        if fusion:
            assert cuda.gehtp_cuda_fused_ops() == 2
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    assert res[0].size == rows * N and np.array_equal(res[0], res[1])


def test_constant_ops_run_once(cuda):
    """A slice of a table that lives in a weight slot and a transposition of that slice give the same bytes on every
    run: the fused engine executes them on the first run and skips them afterwards (also in the captured graph); a
    slice of the input face next to them is not a constant. Results equal the one-kernel-per-op engine's on every run."""
    from gehtp_b200.runlists import Emitter
    rng = np.random.default_rng(12)
    e = Emitter("w4")
    n = 8 * 16
    face = e.b.add_ext_in(2 * n * 2)
    table = e.b.add_slot(rng.standard_normal((8, 32)).astype(np.float16))
    win = e.slice2(S(table), 8, 32, 8, 24)                  # constant: [8][16]
    win_t = e.transpose3(win, (1, 8, 16), (0, 2, 1))        # constant through its input: [16][8]
    x = e.face(S(face), n, n, 2 * n)                        # second half of the input: not a constant
    y = e.binary(win_t, x, n, 0)
    buf = e.b.build()
    inputs = [rng.standard_normal(2 * n).astype(np.float16) for _ in range(4)]
    outs = {}
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        res, launches = [], []
        for inp in inputs:
            before = cuda.gehtp_cuda_launch_count()
            eng.run_io(inp, y, None)
            launches.append(cuda.gehtp_cuda_launch_count() - before)
            res.append(eng.temp(y, np.uint16).copy())
        if fusion:
            assert cuda.gehtp_cuda_const_ops() == 2
            assert launches[0] == 4 and launches[1] == 2 and launches[3] == 2, launches
        else:
            assert cuda.gehtp_cuda_const_ops() == 0 and launches == [4, 4, 4, 4], launches
        outs[fusion] = res
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    for a, b2 in zip(outs[1], outs[0]):
        assert a.size == n and np.array_equal(a, b2)
    assert not np.array_equal(outs[1][0], outs[1][1])


def test_gate_up_gemm_epilogue_on_every_fp16_gate_value(cuda):
    """The SwiGLU epilogue of the gate | up GEMM forms its roundings on packed pairs (half2 conversions and
    multiplies, a correctly rounded reciprocal, NaNs redone apart) where the ops it replaces work value by value. Row m of the activations carries the fp16 value with bit pattern m in its
    first column and the weights pick it out (one weight 1.0 per column, the rest 0), so the 65536 rows put every fp16
    value - subnormals, infinities and NaNs included - through the epilogue as the gate, with an up value that is the
    gate itself in half of the columns and 60000 times the gate (mostly infinite) in the others: bit for bit the
    op-by-op plan's result."""
    from gehtp_b200.runlists import Emitter
    M, K, F = 65536, 64, 128
    nib = np.full((K, F // 2), 0x88, np.uint8)
    nib[0, :] = 0x99                                   # (9 - 8) * scale in row 0 of every column
    ones = np.ones((K // 64, F), np.float16)
    up_scale = ones.copy()
    up_scale[0, F // 2:] = np.float16(60000.0)         # second half of the columns: up = 60000 gate, infinite beyond |gate| = 1.09
    e = Emitter("w4")
    face = e.b.add_ext_in(M * K * 2)
    rng = np.random.default_rng(9)
    from gehtp_b200.runlists import rand_w4
    d = e.swiglu(S(face), M, (nib, ones), (nib, up_scale), rand_w4(rng, F, 64))
    act = d - 1
    buf = e.b.build()
    x = np.zeros((M, K), np.uint16)
    x[:, 0] = np.arange(M, dtype=np.uint32).astype(np.uint16)
    res = []
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        eng.run_io(x, d, None)
        res.append(eng.temp(act, np.uint16).copy())
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    assert res[0].size == M * F and np.array_equal(res[0], res[1])
    got = res[0].reshape(M, F)
    g = x[:, 0].view(np.float16).astype(np.float64)
    ok = np.isfinite(g) & (np.abs(g) < 100)
    want = g[ok] / (1.0 + np.exp(-g[ok])) * g[ok]
    assert_fp16_close(got[ok, 0].view(np.float16), want.astype(np.float16), "silu(g) * g")


@pytest.mark.parametrize("tokens,K,N", [(70, 1024, 1024), (133, 256, 2560), (600, 256, 9728)])
def test_gemm_with_add_and_norm_in_its_epilogue_bit_equal(cuda, tokens, K, N):
    """W4A16 GEMM -> residual ADD -> RMSNORM2 at GEMM row counts runs as the GEMM plus one kernel that adds
    the split-K runs, the residual, and normalises (first two shapes: fewer tiles than SMs, K split), or as the
    GEMM plus the add + norm kernel (third shape: tiles fill the SMs). GEMM output, sum and norm agree bit for bit
    with the one-kernel-per-op plan."""
    from gehtp_b200.runlists import Emitter, rand_w4
    rng = np.random.default_rng(77)
    e = Emitter("w4")
    face = e.b.add_ext_in(tokens * (K + N) * 2)
    x = e.face(S(face), 0, tokens * K, tokens * (K + N))
    res = e.face(S(face), tokens * K, tokens * N, tokens * (K + N))
    lin = e.linear(x, *rand_w4(rng, K, N), tokens)
    summed = e.binary(res, lin, tokens * N, 0)
    normed = e.rmsnorm(summed, rng.normal(1.0, 0.1, N), tokens * N)
    buf = e.b.build()
    inp = np.concatenate([rng.standard_normal(tokens * K), rng.standard_normal(tokens * N)]).astype(np.float16)
    out = []
    for fusion in (1, 0):
        cuda.gehtp_cuda_set_fusion(fusion)
        eng = Engine(cuda, buf)
        eng.run_io(inp, normed, None)
        out.append([eng.temp(t, np.uint16).copy() for t in (lin, summed, normed)])
        eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    for a, b2, name in zip(out[0], out[1], ("gemm", "sum", "norm")):
        assert a.size and np.array_equal(a, b2), name


def test_gdn_layer_runlist_matches_reference(cuda, ref):
    """Config 5 in small: W4A16 in-projection, causal conv1d, four delta-rule chunks carrying the
    fp32 state, out-projection per chunk; against the reference executor with dequantised weights."""
    from gehtp_b200.runlists import build_gdn_runlist
    kw = dict(seq=128, hidden=128, C=256, H=2, D=128, chunk=32, seed=5)
    buf_w4, man = build_gdn_runlist(quant="w4", **kw)
    buf_f16, man2 = build_gdn_runlist(quant="f16", **kw)
    h = np.random.default_rng(3).standard_normal((kw["seq"], kw["hidden"])).astype(np.float16)
    res = []
    for lib, buf, m in ((cuda, buf_w4, man), (ref, buf_f16, man2)):
        lib.wt_exec_state_reset()
        eng = Engine(lib, buf)
        eng.run_io(h, m["chunk_out"][-1], None)
        res.append([eng.temp(m["conv_temp"]).copy()] + [eng.temp(t).copy() for t in m["chunk_out"]])
        eng.shutdown()
        lib.wt_exec_state_reset()
    assert_fp16_close(res[0][0], res[1][0], "conv1d over the in-projection")
    for i in range(1, len(res[0])):
        assert_fp16_close(res[0][i], res[1][i], "delta-rule chunk %d after the out-projection" % (i - 1))


def test_static_offset_table_and_alias_hazard(cuda, ref):
    """A TEMPOFF table whose offsets are sound is honoured; one that maps two
    simultaneously live temps to the same bytes (what the reference's emitter
    produces when it recycles temp ids) must not corrupt results here."""
    rng = np.random.default_rng(2)
    n = 256
    x = rng.standard_normal(n).astype(np.float16)
    c = rng.standard_normal(n).astype(np.float16)

    def graph(entries):
        b = BlobBuilder()
        sx, sc = b.add_slot(x), b.add_slot(c)
        b.add_tempoff(4096, entries, bump_kb=64)
        b.add_op(OP.UNARY, [S(sx), 3, n, 14])            # t3 = x
        b.add_op(OP.BINARY, [3, S(sc), 1, n, 2])         # t1 = t3 * c
        b.add_op(OP.SLICE, [3, 5, n // 2, 1, 0, 0, 0, n // 2, 0, 0, 1, 1, 1, n, 1, 1])  # t5 = t3[:n/2]
        b.add_op(OP.ADD, [1, 3, 6, n])                   # t6 = t1 + t3
        return b
    want5, want6 = x[:n // 2], (x * c).astype(np.float16) + x
    sound = [(3, 0, 512), (1, 512, 512), (5, 1024, 256), (6, 2048, 512)]
    alias = [(3, 0, 512), (1, 0, 512), (5, 1024, 256), (6, 2048, 512)]
    for entries in (sound, alias):
        eng = Engine(cuda, graph(entries).build())
        eng.run()
        assert np.array_equal(eng.temp(5), want5)
        assert np.array_equal(eng.temp(6), want6.astype(np.float16))
        eng.shutdown()
    # the reference itself corrupts the aliased case (documented hazard), the sound one it runs
    eng = Engine(ref, graph(sound).build())
    eng.run()
    assert np.array_equal(eng.temp(6), want6.astype(np.float16))
    eng.shutdown()
