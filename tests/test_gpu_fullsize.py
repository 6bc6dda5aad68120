"""Parity at the benchmark's own shapes (the kernels take other template paths here than on
the toy shapes of test_gpu_hotpath.py: 5/8/10/19-warp GEMV walks, the rotary epilogue at 6144
columns, 256-wide GEMM tiles, 18 context slices per KV-head group, 64-token delta chunks on 4
CTAs per head). The reference executor's cost is bounded by giving it ONE layer of each model
(plus a 2048-column cut of the vocabulary projection) with the weights dequantised to fp16;
part_rng() in runlists.py makes that cut carry exactly the weights of the whole model's first
layer. Gate: the project's fp16 gate (max |err| <= 1e-2 max|ref|, cosine >= 0.9999)."""
import ctypes

import numpy as np
import pytest

from conftest import assert_fp16_close, cos_sim
from oracle.refexec import ptr
from gehtp_b200.runlists import (QWEN3_0P6B, QWEN3_4B, build_decode_runlist, build_gdn_runlist, build_prefill_runlist,
                                 decode_face)
from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine

pytestmark = pytest.mark.gpu


def fill_reference_ring(ref, ring, n_pos, ctx):
    """Appends rows [0, n_pos) of `ring` ([ctx][K face | V face] fp16) to state 0 of the reference
    executor through its own KV_APPEND op, one run per position (the state table is per process:
    the model blob that follows must declare the same single state)."""
    kv_elems = ring.shape[1] // 2
    b = BlobBuilder()
    face = b.add_ext_in(2 * kv_elems * 2)
    b.add_states([kv_elems * 4 * ctx])
    b.add_op(OP.SLICE, [S(face), 1, kv_elems, 1, 0, 0, 0, kv_elems, 0, 0, 1, 1, 1, 2 * kv_elems, 1, 1])
    b.add_op(OP.SLICE, [S(face), 2, kv_elems, 1, kv_elems, 0, 0, 2 * kv_elems, 0, 0, 1, 1, 1, 2 * kv_elems, 1, 1])
    b.add_op(OP.KV_APPEND, [1, 2, ST(0), KV_POS_AUTO])
    eng = Engine(ref, b.build())
    for p in range(n_pos):
        eng.run_io(ring[p], 0)
    return eng


@pytest.mark.parametrize("B", [1, 8])
def test_qwen3_4b_decode_layer_full_size(cuda, ref, orc, B):
    """Config 4: hidden 2560, 32 query / 8 KV heads of 128, FFN 9728, KV context 8192, batch 1 and 8;
    one decode step at the last position of the ring (8191 resident positions), through the fused
    engine: eager, captured and replayed runs must agree bit for bit with each other and meet the
    gate against the reference; ring slots other than the appended one keep their bytes.

    At 8192 positions the reference's op chain is the noisier side: its probabilities (~1e-4) are fp16
    temps. The attention output is therefore also measured against a float64 restatement, where the fused
    kernel must be at least as close as the chain; and the logits, which inherit the chain's noise through
    a residual stream of magnitude ~1e3 and a final norm, are gated at 2e-2 of their maximum plus cosine."""
    cfg, ctx, vs = QWEN3_4B, 8192, 2048
    buf_w4, man = build_decode_runlist(cfg, B, ctx, seed=1004, quant="w4", n_layers=1, vocab=vs)
    buf_f16, man2 = build_decode_runlist(cfg, B, ctx, seed=1004, quant="f16", n_layers=1, vocab=vs)
    assert man["layer_out"] == man2["layer_out"] and man["logits_temp"] == man2["logits_temp"]
    kv_elems, hd, pos = B * cfg.kv_heads * cfg.head_dim, cfg.head_dim, ctx - 1
    rng = np.random.default_rng(1004)
    ring = rng.standard_normal((ctx, 2 * kv_elems), dtype=np.float32).astype(np.float16)
    ids = rng.integers(0, vs, B)
    face = decode_face(man, ids, pos, hd, cfg.rope_theta)

    # reference: one layer, fp16 weights
    ref.wt_exec_state_reset()
    fill_reference_ring(ref, ring, pos, ctx)
    reng = Engine(ref, buf_f16)
    reng.run_io(face, man2["token_temp"])
    r_x = reng.temp(man2["layer_out"][0]).copy()
    r_logits = reng.temp(man2["logits_temp"]).copy()
    append = [reng.blob.ops[i] for i in range(reng.blob.n_ops) if reng.blob.ops[i].opcode == OP.KV_APPEND][0]
    r_k, r_v = reng.temp(append.args[0]).copy(), reng.temp(append.args[1]).copy()
    bmm = [reng.blob.ops[i] for i in range(reng.blob.n_ops) if reng.blob.ops[i].opcode == OP.MATMUL_F16 and reng.blob.ops[i].args[6] & 4]
    q_temp, ctx_temp = bmm[0].args[0], bmm[1].args[2]
    r_ctx = reng.temp(ctx_temp).copy()
    reng.shutdown()
    ref.wt_exec_state_reset()

    # CUDA engine: W4A16 weights, fused plan, CUDA graph from the third run on
    cuda.gehtp_cuda_set_fusion(1)
    cuda.gehtp_cuda_set_graph(1)
    cuda.wt_exec_state_reset()
    eng = Engine(cuda, buf_w4)
    err = ctypes.create_string_buffer(256)
    assert cuda.gehtp_cuda_state_load(ctypes.byref(eng.blob), 0, ring.ctypes.data, ring.nbytes, 0, kv_elems, pos, err, 256) == 0, err.value
    outs = []
    for run in range(4):
        assert cuda.gehtp_cuda_state_set_count(0, pos) == 0
        tok = np.zeros(2 * B, np.uint16)
        eng.run_io(face, man["token_temp"], tok)
        outs.append((eng.temp(man["layer_out"][0]).copy(), eng.temp(man["logits_temp"]).copy(), tok.copy()))
    assert cuda.gehtp_cuda_fused_ops() >= 25 + 5 + 2 + 2
    for x, lg, tok in outs[1:]:
        assert np.array_equal(x.view(np.uint16), outs[0][0].view(np.uint16))
        assert np.array_equal(lg.view(np.uint16), outs[0][1].view(np.uint16))
        assert np.array_equal(tok, outs[0][2])
    assert_fp16_close(outs[0][0], r_x, "layer output, batch %d" % B)
    lg, rl = outs[0][1].astype(np.float64), r_logits.astype(np.float64)
    assert np.abs(lg - rl).max() <= 2e-2 * np.abs(rl).max() and cos_sim(lg, rl) >= 0.9999, (np.abs(lg - rl).max(), np.abs(rl).max())
    got_ring = np.zeros_like(ring)
    assert cuda.gehtp_cuda_state_read(0, got_ring.ctypes.data, got_ring.nbytes) == 0
    # attention against float64 over the same rotated q and ring
    nh, kvh = B * cfg.n_heads, B * cfg.kv_heads
    g_q, g_ctx = eng.temp(q_temp).copy(), eng.temp(ctx_temp).copy()
    exact = np.zeros((nh, hd), np.float64)
    orc.orc_attn_decode_f64(ptr(g_q), ptr(got_ring), ctx, ctx, nh, kvh, hd, float(np.float16(1 / np.sqrt(hd))), None, ptr(exact))
    e_fused = np.abs(g_ctx.astype(np.float64).reshape(nh, hd) - exact).max()
    e_chain = np.abs(r_ctx.astype(np.float64).reshape(nh, hd) - exact).max()
    # both sides end in one fp16 rounding of outputs up to ~10: two fp16 steps of the largest output are allowed on top
    assert e_fused <= 1.5 * e_chain + 2.0 ** -9 * np.abs(exact).max() + 1e-3, (e_fused, e_chain, np.abs(exact).max())
    assert_fp16_close(g_ctx, r_ctx, "attention output vs the reference chain")
    assert np.array_equal(got_ring[:pos].view(np.uint16), ring[:pos].view(np.uint16)), "resident ring slots changed"
    assert_fp16_close(got_ring[pos, :kv_elems], r_k, "appended K (rotary applied)")
    assert_fp16_close(got_ring[pos, kv_elems:], r_v, "appended V")
    eng.shutdown()
    cuda.wt_exec_state_reset()


def test_qwen3_0p6b_prefill_layer_full_size(cuda, ref):
    """Config 3: one Qwen3-0.6B-shaped layer (hidden 1024, 16 query / 8 KV heads of 128, FFN 3072) over
    512 tokens with a causal mask, plus a 2048-column cut of the vocabulary projection. Under a causal
    mask the first 128 tokens do not depend on the rest, so the reference runs the 128-token prefix of
    the same layer (same weights and ids) and is compared with the first 128 rows of the 512-token run."""
    cfg, seq, cut, vs = QWEN3_0P6B, 512, 128, 2048
    buf_w4, man = build_prefill_runlist(cfg, seq, seed=1003, quant="w4", n_layers=1, vocab=vs)
    buf_f16, man2 = build_prefill_runlist(cfg, cut, seed=1003, quant="f16", n_layers=1, vocab=vs)
    ids = np.random.default_rng(1003).integers(0, vs, seq).astype(np.int32)
    reng = Engine(ref, buf_f16)
    reng.run_io(ids[:cut], man2["logits_temp"])
    r_x = reng.temp(man2["layer_out"][0]).reshape(cut, -1).copy()
    r_logits = reng.temp(man2["logits_temp"]).reshape(cut, -1).copy()
    reng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    eng = Engine(cuda, buf_w4)
    outs = []
    for run in range(3):
        eng.run_io(ids, man["logits_temp"])
        outs.append((eng.temp(man["layer_out"][0]).reshape(seq, -1).copy(), eng.temp(man["logits_temp"]).reshape(seq, -1).copy()))
    eng.shutdown()
    assert np.array_equal(outs[0][1].view(np.uint16), outs[2][1].view(np.uint16)), "eager and replayed runs differ"
    assert np.isfinite(outs[0][1].astype(np.float32)).all()
    assert_fp16_close(outs[0][0][:cut], r_x, "prefill layer output, first 128 of 512 tokens")
    assert_fp16_close(outs[0][1][:cut], r_logits, "prefill logits, first 128 of 512 tokens")


def test_gated_delta_layer_full_size(cuda, ref):
    """Config 5 at its own size: 2048 tokens, 4096 conv channels, 16 heads of 128, chunks of 64 (the
    kernel's widest form: 4 CTAs per head, 64-row chunk matrices). The reference runs the 256-token
    prefix of the same layer (build_gdn_runlist draws every part from its own generator, so the prefix
    has the same weights, conv taps and q/k/v/beta/g): in-projection, conv and the first 4 chunks with
    their out-projections; the state is carried from chunk to chunk, so an error in one shows in the
    next. The remaining 28 chunks and the final fp32 state must stay finite."""
    buf_w4, man = build_gdn_runlist(quant="w4")
    assert (man["seq"], man["C"], man["H"], man["D"], man["chunk"]) == (2048, 4096, 16, 128, 64)
    n_chunks, k_conv = 4, 4
    cut = n_chunks * man["chunk"]
    buf_f16, man2 = build_gdn_runlist(seq=cut, quant="f16")
    h = np.random.default_rng(1005).standard_normal((man["seq"], man["hidden"]), dtype=np.float32).astype(np.float16)
    ref.wt_exec_state_reset()
    reng = Engine(ref, buf_f16)
    reng.run_io(h[:cut], 0)
    want = [reng.temp(man2["conv_temp"]).reshape(cut, -1).copy()] + [reng.temp(t).copy() for t in man2["chunk_out"]]
    reng.shutdown()
    ref.wt_exec_state_reset()

    cuda.wt_exec_state_reset()
    eng = Engine(cuda, buf_w4)
    eng.run_io(h, man["chunk_out"][-1], None)
    got = [eng.temp(man["conv_temp"]).reshape(man["seq"], -1).copy()] + [eng.temp(t).copy() for t in man["chunk_out"]]
    state = np.zeros(man["H"] * man["D"] * man["D"], np.float32)
    assert cuda.gehtp_cuda_state_read(0, state.ctypes.data, state.nbytes) == 0
    eng.shutdown()
    cuda.wt_exec_state_reset()
    # the op treats the last k-1 input rows of its sequence as the zero flush: rows that see them differ in the cut
    rows = cut - (k_conv - 1)
    assert_fp16_close(got[0][:rows], want[0][:rows], "conv1d over 4096 channels")
    for i in range(n_chunks):
        assert_fp16_close(got[1 + i], want[1 + i], "delta-rule chunk %d (64 tokens, 16 heads)" % i)
    for g in got:
        assert np.isfinite(g.astype(np.float32)).all()
    assert np.isfinite(state).all() and np.abs(state).max() > 0
