"""Hand-built WTOP runlists for the LLM hot path.

The reference compiles ONNX graphs into runlists with `hnnx_compile` +
`wtop_emit`; Qwen-shaped graphs cannot be produced in this environment (no
ONNX converter, no checkpoints), so the runlists here are written out op by op
in the form that emitter produces: the same opcodes, argument layouts, operand
encodings, rotary / attention / SwiGLU decompositions (one op per ONNX node,
reference blob of test_models/qnn_probe, ops 5-47) and decode-state ops
(compiler/tools/wtop_ops/op_decode_state.cpp). Weights are seeded synthetic
tensors of the named architecture's shapes.

`quant="w4"` emits opcode 1 with group-64 W4A16 weight slots; `quant="f16"`
emits the same graph with the dequantised fp16 weights and opcode 24, which
the reference executor can run, so that it can serve as the oracle.
"""
from dataclasses import dataclass

import numpy as np

from .wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, pack_w4a16


@dataclass
class DecoderConfig:
    hidden: int
    layers: int
    n_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 1e6
    name: str = "custom"


QWEN3_0P6B = DecoderConfig(1024, 28, 16, 8, 128, 3072, 151936, 1e6, "qwen3-0.6b-shape")
QWEN3_4B = DecoderConfig(2560, 36, 32, 8, 128, 9728, 151936, 1e6, "qwen3-4b-shape")


def rand_w4(rng, K, N):
    """Uniform int4 weights and U[0.005, 0.02] fp16 scales, as slot bytes parts."""
    nib = rng.integers(0, 256, size=(K, N // 2), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(K // 64, N)).astype(np.float16)
    return nib, scales


def nib_to_q(nib):
    K, N2 = nib.shape
    q = np.empty((K, N2 * 2), np.uint8)
    q[:, 0::2] = nib & 15
    q[:, 1::2] = nib >> 4
    return q


def dequant_f16(nib, scales):
    """fp16((q - 8) * scale): the weights opcode 1 multiplies by."""
    q = nib_to_q(nib).astype(np.float32) - 8.0
    s = np.repeat(scales.astype(np.float32), 64, axis=0)
    return (q * s).astype(np.float16)


def rope_tables(hd, pos, theta):
    """cos/sin rows [len(pos), hd] for split-half rotation (the layout of
    hvhx_v2_rope_neox_f32, kernels/src/hvx/hvx_rope.c:288)."""
    inv = 1.0 / (theta ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ang = np.asarray(pos, dtype=np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1)
    return cos.astype(np.float16), sin.astype(np.float16)


class Emitter:
    """Op-by-op runlist writer with fresh temp ids (temp 0 is never used: the
    KV gather op treats an output id of 0 as "skip this face")."""

    def __init__(self, quant="w4"):
        self.b = BlobBuilder()
        self.quant = quant
        self.t = 0
        self.zero_bias = {}
        self.consts = {}
        self.row_parallel_ops = []   # op indices whose output is a partial sum under tensor parallelism

    def fresh(self):
        self.t += 1
        assert self.t < 4096
        return self.t

    def const_f16(self, value):
        key = float(value)
        if key not in self.consts:
            self.consts[key] = self.b.add_slot(np.array([value], np.float16))
        return S(self.consts[key])

    # ---- single ops
    def linear(self, a_ref, nib, scales, M, row_parallel=False):
        K, N = nib.shape[0], nib.shape[1] * 2
        y = self.fresh()
        if self.quant == "w4":
            w = self.b.add_slot(np.concatenate([nib.reshape(-1), scales.view(np.uint8).reshape(-1)]), count=K * N)
            i = self.b.add_op(OP.MATMUL_W4A16, [a_ref, S(w), y, M, K, N])
        else:
            # FullyConnected weights are stored [N, K] with the transposed-weight bit, as the reference's
            # emitter stores them (compiler/tools/wtop_ops/op_matmul.cpp:50)
            w = self.b.add_slot(np.ascontiguousarray(dequant_f16(nib, scales).T))
            i = self.b.add_op(OP.MATMUL_F16, [a_ref, S(w), y, M, K, N, 2])
        if row_parallel:
            self.row_parallel_ops.append(i)
        return y

    def rmsnorm(self, x_ref, gamma, n):
        w = self.b.add_slot(np.asarray(gamma, np.float16))
        width = len(gamma)
        if width not in self.zero_bias:
            self.zero_bias[width] = self.b.add_slot(np.zeros(width, np.float16))
        y = self.fresh()
        self.b.add_op(OP.RMSNORM2, [x_ref, S(w), S(self.zero_bias[width]), y, n])
        return y

    def unary(self, x, n, sub):
        y = self.fresh()
        self.b.add_op(OP.UNARY, [x, y, n, sub])
        return y

    def binary(self, a, c, n, sub):
        y = self.fresh()
        if sub == 0:
            self.b.add_op(OP.ADD, [a, c, y, n])
        else:
            self.b.add_op(OP.BINARY, [a, c, y, n, sub])
        return y

    def broadcast(self, x, in_d, out_d):
        n = int(np.prod(out_d))
        y = self.fresh()
        self.b.add_op(OP.BROADCAST, [x, y, n, int(np.prod(in_d))] + list(in_d) + list(out_d))
        return y

    def slice2(self, x, rows, width, c0, c1):
        y = self.fresh()
        self.b.add_op(OP.SLICE, [x, y, rows * (c1 - c0), 2, 0, c0, 0, rows, c1, 0, 1, 1, 1, rows, width, 1])
        return y

    def face(self, x, begin, n, total):
        """rank-1 window of the merged input face (op_decode_state.cpp:27-50)."""
        y = self.fresh()
        self.b.add_op(OP.SLICE, [x, y, n, 1, begin, 0, 0, begin + n, 0, 0, 1, 1, 1, total, 1, 1])
        return y

    def concat(self, parts, sizes, n_elems):
        y = self.fresh()
        ins = list(parts) + [0] * (8 - len(parts))
        sz = list(sizes) + [0] * (4 - len(sizes))
        self.b.add_op(OP.CONCAT, ins + [y, 0, len(parts), n_elems] + sz)
        return y

    def split(self, x, sizes, index):
        y = self.fresh()
        sz = list(sizes) + [0] * (4 - len(sizes))
        self.b.add_op(OP.SPLIT, [x, y] + [0] * 7 + [0, len(sizes)] + sz + [index])
        return y

    def transpose3(self, x, dims, perm):
        y = self.fresh()
        p = perm[0] | perm[1] << 8 | perm[2] << 16
        self.b.add_op(OP.TRANSPOSE_GEN, [x, y, 3, dims[0], dims[1], dims[2], 1, p])
        return y

    def softmax(self, x, rows, n):
        y = self.fresh()
        self.b.add_op(OP.SOFTMAX, [x, y, rows, n])
        return y

    def bmm(self, a, w, Bn, M, K, N, t1=False):
        y = self.fresh()
        self.b.add_op(OP.MATMUL_F16, [a, w, y, M, K, N, 4 | (2 if t1 else 0) | (Bn << 16)])
        return y

    # ---- composite pieces, decomposed as the emitter decomposes the ONNX graph
    def rope(self, x, rows, hd, cos_b, sin_b):
        """x*cos + rotate_half(x)*sin with rotate_half = concat(-x2, x1)."""
        n, h = rows * hd, hd // 2
        xc = self.binary(x, cos_b, n, 2)
        x1 = self.slice2(x, rows, hd, 0, h)
        x2 = self.slice2(x, rows, hd, h, hd)
        nx2 = self.unary(x2, rows * h, 0)
        rot = self.concat([nx2, x1], [h, h], n)
        xs = self.binary(rot, sin_b, n, 2)
        return self.binary(xc, xs, n, 0)

    def swiglu(self, h2, M, wg, wu, wd):
        ffn = wg[0].shape[1] * 2
        gate = self.linear(h2, *wg, M)
        sig = self.unary(gate, M * ffn, 8)
        act = self.binary(gate, sig, M * ffn, 2)
        up = self.linear(h2, *wu, M)
        prod = self.binary(act, up, M * ffn, 2)
        return self.linear(prod, *wd, M, row_parallel=True)


def synth_embedding(rng, V, H):
    """fp16 ~ N(0, 0.02) [V, H]. Tables of more than 1024 rows are tiled from a
    1024-row block: converting hundreds of millions of floats on the host takes
    longer than the whole benchmark, and a decode step reads only one row per
    sequence. Row r is block[r % 1024] whatever V is, so models that differ only
    in their vocabulary size embed the same id (below 1024) the same way."""
    block = (rng.standard_normal((min(V, 1024), H), dtype=np.float32) * 0.02).astype(np.float16)
    if V <= 1024:
        return block
    return np.tile(block, ((V + 1023) // 1024, 1))[:V]


def part_rng(seed, part):
    """Independent generator per model part (layer index, or a name's number), so that a
    one-layer or small-vocabulary cut of a model carries the same weights as the whole."""
    return np.random.default_rng([int(seed), int(part)])


EMB_PART, HEAD_PART = 100000, 100001


def synth_head(rng, H, V):
    """Vocabulary projection [H, V] in W4 form. The first 2048 columns are drawn first, the rest
    after them, so a 2048-column cut of a model is the head of the whole model's projection."""
    first = rand_w4(rng, H, min(V, 2048))
    if V <= 2048:
        return first
    return hcat(first, rand_w4(rng, H, V - 2048))


def cols(w, c0, c1):
    """Column slice [c0, c1) of a (nibbles, scales) weight pair (c0, c1 even)."""
    nib, sc = w
    return np.ascontiguousarray(nib[:, c0 // 2:c1 // 2]), np.ascontiguousarray(sc[:, c0:c1])


def rows(w, r0, r1):
    """Row (K) slice [r0, r1) of a weight pair; r0 and r1 are multiples of the group size 64."""
    nib, sc = w
    return np.ascontiguousarray(nib[r0:r1]), np.ascontiguousarray(sc[r0 // 64:r1 // 64])


def hcat(*ws):
    return np.concatenate([w[0] for w in ws], axis=1), np.concatenate([w[1] for w in ws], axis=1)


def synth_layer(rng, cfg, tp=1, rank=0):
    """Seeded weights of one decoder layer. With tp > 1 every rank draws the
    same full matrices and keeps its shard: q/k/v heads and gate/up columns are
    column-parallel, o and down are row-parallel (their K slices fall on
    multiples of the scale group)."""
    H, hd = cfg.hidden, cfg.head_dim
    NH, KVH, F = cfg.n_heads, cfg.kv_heads, cfg.ffn
    full = dict(
        g1=rng.normal(1.0, 0.1, H).astype(np.float16),
        g2=rng.normal(1.0, 0.1, H).astype(np.float16),
        qkv=rand_w4(rng, H, (NH + 2 * KVH) * hd),
        o=rand_w4(rng, NH * hd, H),
        gate=rand_w4(rng, H, F),
        up=rand_w4(rng, H, F),
        down=rand_w4(rng, F, H),
    )
    if tp == 1:
        return full
    nh, kvh, f = NH // tp, KVH // tp, F // tp
    assert NH % tp == 0 and KVH % tp == 0 and F % tp == 0 and (nh * hd) % 64 == 0 and f % 64 == 0
    q0, k0, v0 = 0, NH * hd, (NH + KVH) * hd
    full["qkv"] = hcat(cols(full["qkv"], q0 + rank * nh * hd, q0 + (rank + 1) * nh * hd),
                       cols(full["qkv"], k0 + rank * kvh * hd, k0 + (rank + 1) * kvh * hd),
                       cols(full["qkv"], v0 + rank * kvh * hd, v0 + (rank + 1) * kvh * hd))
    full["o"] = rows(full["o"], rank * nh * hd, (rank + 1) * nh * hd)
    full["gate"] = cols(full["gate"], rank * f, (rank + 1) * f)
    full["up"] = cols(full["up"], rank * f, (rank + 1) * f)
    full["down"] = rows(full["down"], rank * f, (rank + 1) * f)
    return full


def build_decode_runlist(cfg, B, nslots, seed=1004, quant="w4", n_layers=None, with_lm_head=True,
                         vocab=None, tp=1, rank=0, scale_div=False):
    """One decode step for B sequences that share a position: token ids and the
    rotary / mask faces come in through the EXT_IN face, K/V of the new token are
    appended to one KV state per layer (batch folded into the head dim) and
    attention runs over the whole ring.

    Returns (blob bytes as uint8 array, manifest dict).
    Input face, in fp16-sized units: ids (int32 x B) | cos[hd] | sin[hd] | mask[nslots].
    """
    L = cfg.layers if n_layers is None else n_layers
    V = cfg.vocab if vocab is None else vocab
    H, hd = cfg.hidden, cfg.head_dim
    nh, kvh = cfg.n_heads // tp, cfg.kv_heads // tp
    e = Emitter(quant)
    ids_u16 = (2 * B + 31) // 32 * 32
    face_total = ids_u16 + 2 * hd + nslots
    face = e.b.add_ext_in(face_total * 2)
    e.b.add_states([B * kvh * hd * 4 * nslots] * L)
    emb_s = e.b.add_slot(synth_embedding(part_rng(seed, EMB_PART), V, H))

    ids = e.face(S(face), 0, 2 * B, face_total)
    cos = e.face(S(face), ids_u16, hd, face_total)
    sin = e.face(S(face), ids_u16 + hd, hd, face_total)
    mask = e.face(S(face), ids_u16 + 2 * hd, nslots, face_total)
    x = e.fresh()
    e.b.add_op(OP.GATHER, [S(emb_s), ids, x, B * H, 0 | 1 << 8 | 2 << 16, V, H, 1, 1, 1, B, 1, 1, 1, 1])
    cos_q = e.broadcast(cos, (1, 1, 1, hd), (1, 1, B * nh, hd))
    sin_q = e.broadcast(sin, (1, 1, 1, hd), (1, 1, B * nh, hd))
    cos_k = e.broadcast(cos, (1, 1, 1, hd), (1, 1, B * kvh, hd))
    sin_k = e.broadcast(sin, (1, 1, 1, hd), (1, 1, B * kvh, hd))
    mask_b = e.broadcast(mask, (1, 1, 1, nslots), (1, 1, B * nh, nslots))
    sc = float(np.sqrt(hd)) if scale_div else float(1.0 / np.sqrt(hd))
    scale_b = e.broadcast(e.const_f16(sc), (1, 1, 1, 1), (1, 1, 1, B * nh * nslots))

    layer_out = []
    for li in range(L):
        w = synth_layer(part_rng(seed, li), cfg, tp, rank)
        h1 = e.rmsnorm(x, w["g1"], B * H)
        qkv = e.linear(h1, *w["qkv"], B)
        sizes = [nh * hd, kvh * hd, kvh * hd]
        q = e.split(qkv, sizes, 0)
        k = e.split(qkv, sizes, 1)
        v = e.split(qkv, sizes, 2)
        qr = e.rope(q, B * nh, hd, cos_q, sin_q)
        kr = e.rope(k, B * kvh, hd, cos_k, sin_k)
        e.b.add_op(OP.KV_APPEND, [kr, v, ST(li), KV_POS_AUTO])
        kT, vv = e.fresh(), e.fresh()
        e.b.add_op(OP.KV_GATHER, [ST(li), kT, 0, KV_POS_AUTO, B * nh, B * kvh, hd])
        e.b.add_op(OP.KV_GATHER, [ST(li), 0, vv, KV_POS_AUTO, B * nh, B * kvh, hd])
        scores = e.bmm(qr, kT, B * nh, 1, hd, nslots)
        scaled = e.binary(scores, scale_b, B * nh * nslots, 3 if scale_div else 2)
        masked = e.binary(scaled, mask_b, B * nh * nslots, 0)
        probs = e.softmax(masked, B * nh, nslots)
        ctx = e.bmm(probs, vv, B * nh, 1, nslots, hd)
        o = e.linear(ctx, *w["o"], B, row_parallel=True)
        x = e.binary(x, o, B * H, 0)
        h2 = e.rmsnorm(x, w["g2"], B * H)
        d = e.swiglu(h2, B, w["gate"], w["up"], w["down"])
        x = e.binary(x, d, B * H, 0)
        layer_out.append(x)

    rng = part_rng(seed, HEAD_PART)
    gf = rng.normal(1.0, 0.1, H).astype(np.float16)
    hn = e.rmsnorm(x, gf, B * H)
    man = dict(config=cfg.name, B=B, nslots=nslots, layers=L, hidden=H, face_u16=face_total, ids_u16=ids_u16,
               cos_off=ids_u16, sin_off=ids_u16 + hd, mask_off=ids_u16 + 2 * hd, hidden_temp=hn,
               input_slot=face, quant=quant, tp=tp, rank=rank, layer_out=layer_out)
    if with_lm_head:
        Vs = V // tp
        # column c of the vocabulary projection is the same whatever V is (drawn in blocks of 2048 columns)
        logits = e.linear(hn, *cols(synth_head(rng, H, V), rank * Vs, (rank + 1) * Vs), B)
        toks = []
        for bi in range(B):
            row = e.slice2(logits, B, Vs, 0, Vs) if B == 1 else e.fresh()
            if B > 1:
                e.b.add_op(OP.SLICE, [logits, row, Vs, 2, bi, 0, 0, bi + 1, Vs, 0, 1, 1, 1, B, Vs, 1])
            am = e.fresh()
            e.b.add_op(OP.ARGMAX, [row, am, Vs])
            toks.append(am)
        toks = [(t, 2) for t in toks]   # int32 results, joined as pairs of fp16-sized elements
        while len(toks) > 1:
            nxt = []
            for i in range(0, len(toks), 4):
                grp = toks[i:i + 4]
                if len(grp) == 1:
                    nxt.append(grp[0])
                    continue
                total = sum(w for _, w in grp)
                nxt.append((e.concat([t for t, _ in grp], [w for _, w in grp], total), total))
            toks = nxt
        toks = [toks[0][0]]
        if tp > 1:
            # row maxima next to the shard-local argmax, so that ranks can be merged: [tokens int32 x B | max f16 x B]
            mx = e.fresh()
            e.b.add_op(OP.REDUCE, [logits, mx, B * Vs, 1, 2, B, Vs, 1, 1])
            toks = [e.concat([toks[0], mx], [2 * B, B], 3 * B)]
        man.update(logits_temp=logits, token_temp=toks[0], vocab_shard=Vs)
    man["row_parallel_ops"] = e.row_parallel_ops
    man["n_ops"] = len(e.b.ops)
    return e.b.build(), man


def decode_face(man, token_ids, pos, hd, theta, n_valid=None):
    """The EXT_IN face of one decode step at position `pos` (same for all sequences)."""
    face = np.zeros(man["face_u16"], np.uint16)
    ids = np.asarray(token_ids, np.int32)
    face[:2 * ids.size] = ids.view(np.uint16)
    cos, sin = rope_tables(hd, [pos], theta)
    face[man["cos_off"]:man["cos_off"] + hd] = cos[0].view(np.uint16)
    face[man["sin_off"]:man["sin_off"] + hd] = sin[0].view(np.uint16)
    mask = np.full(man["nslots"], -np.inf, np.float16)
    mask[:(pos + 1 if n_valid is None else n_valid)] = 0
    face[man["mask_off"]:man["mask_off"] + man["nslots"]] = mask.view(np.uint16)
    return face


def build_prefill_runlist(cfg, seq, seed=1003, quant="w4", n_layers=None, with_lm_head=True, vocab=None):
    """Causal prefill of `seq` tokens, batch 1. Input face: ids int32 x seq.
    cos/sin tables and the causal mask are baked constant slots, as in the
    reference's prefill graphs."""
    L = cfg.layers if n_layers is None else n_layers
    V = cfg.vocab if vocab is None else vocab
    H, hd, nh, kvh = cfg.hidden, cfg.head_dim, cfg.n_heads, cfg.kv_heads
    rep = nh // kvh
    e = Emitter(quant)
    face = e.b.add_ext_in(seq * 4)
    emb_s = e.b.add_slot(synth_embedding(part_rng(seed, EMB_PART), V, H))
    cos, sin = rope_tables(hd, np.arange(seq), cfg.rope_theta)
    # rows of q are (token, head): the table row of a (token, head) pair is the token's
    cos_q = S(e.b.add_slot(np.repeat(cos, nh, axis=0)))
    sin_q = S(e.b.add_slot(np.repeat(sin, nh, axis=0)))
    cos_k = S(e.b.add_slot(np.repeat(cos, kvh, axis=0)))
    sin_k = S(e.b.add_slot(np.repeat(sin, kvh, axis=0)))
    causal = np.where(np.tril(np.ones((seq, seq), bool)), 0.0, -np.inf).astype(np.float16)
    mask_s = S(e.b.add_slot(causal))
    x = e.fresh()
    e.b.add_op(OP.GATHER, [S(emb_s), S(face), x, seq * H, 0 | 1 << 8 | 2 << 16, V, H, 1, 1, 1, seq, 1, 1, 1, 1])
    mask_b = e.broadcast(mask_s, (1, 1, seq, seq), (1, nh, seq, seq))
    scale_b = e.broadcast(e.const_f16(1.0 / np.sqrt(hd)), (1, 1, 1, 1), (1, 1, 1, nh * seq * seq))
    layer_out = []
    for li in range(L):
        w = synth_layer(part_rng(seed, li), cfg)
        h1 = e.rmsnorm(x, w["g1"], seq * H)
        qkv = e.linear(h1, *w["qkv"], seq)
        sizes = [nh * hd, kvh * hd, kvh * hd]
        q = e.rope(e.split(qkv, sizes, 0), seq * nh, hd, cos_q, sin_q)
        k = e.rope(e.split(qkv, sizes, 1), seq * kvh, hd, cos_k, sin_k)
        v = e.split(qkv, sizes, 2)
        qh = e.transpose3(q, (seq, nh, hd), (1, 0, 2))      # [nh, seq, hd] = [kvh, rep*seq, hd]
        kh = e.transpose3(k, (seq, kvh, hd), (1, 2, 0))     # [kvh, hd, seq]
        vh = e.transpose3(v, (seq, kvh, hd), (1, 0, 2))     # [kvh, seq, hd]
        scores = e.bmm(qh, kh, kvh, rep * seq, hd, seq)
        scaled = e.binary(scores, scale_b, nh * seq * seq, 2)
        masked = e.binary(scaled, mask_b, nh * seq * seq, 0)
        probs = e.softmax(masked, nh * seq, seq)
        ctx = e.bmm(probs, vh, kvh, rep * seq, seq, hd)     # [nh, seq, hd]
        ctx = e.transpose3(ctx, (nh, seq, hd), (1, 0, 2))   # [seq, nh*hd]
        o = e.linear(ctx, *w["o"], seq, row_parallel=True)
        x = e.binary(x, o, seq * H, 0)
        h2 = e.rmsnorm(x, w["g2"], seq * H)
        d = e.swiglu(h2, seq, w["gate"], w["up"], w["down"])
        x = e.binary(x, d, seq * H, 0)
        layer_out.append(x)
    rng = part_rng(seed, HEAD_PART)
    hn = e.rmsnorm(x, rng.normal(1.0, 0.1, H).astype(np.float16), seq * H)
    man = dict(config=cfg.name, seq=seq, layers=L, hidden_temp=hn, input_slot=face, quant=quant, layer_out=layer_out)
    if with_lm_head:
        man["logits_temp"] = e.linear(hn, *synth_head(rng, H, V), seq)
    man["n_ops"] = len(e.b.ops)
    return e.b.build(), man


def build_gdn_runlist(seq=2048, hidden=1024, C=4096, k_conv=4, H=16, D=128, chunk=64, seed=1005, quant="w4"):
    """One gated-delta-rule linear-attention layer over `seq` tokens, batch 1
    (baseline config 5): W4A16 in-projection hidden -> C channels, causal
    depthwise conv1d (OP_CONV1D_SSM), the delta rule chunk by chunk
    (OP_DELTA_CHUNK, fp32 state [H, D, D] carried in persistent state 0) on
    independent synthetic q/k/v/beta/g slots, and a W4A16 out-projection
    H*D -> hidden of every chunk's output. Input face: h fp16 [seq, hidden].

    Returns (blob, manifest); manifest["chunk_out"] lists the temps holding
    the out-projection of each chunk ([chunk, hidden] fp16). Weights and the
    per-chunk q/k/v/beta/g are drawn from one generator per part, so a layer
    built with a shorter `seq` is the prefix of the longer one."""
    assert seq % chunk == 0 and chunk <= 64
    e = Emitter(quant)
    face = e.b.add_ext_in(seq * hidden * 2)
    e.b.add_states([H * D * D * 4])
    xin = e.linear(S(face), *rand_w4(part_rng(seed, 0), hidden, C), seq)
    conv_w = e.b.add_slot(part_rng(seed, 1).normal(0.0, 0.5, (k_conv, C)).astype(np.float16))
    conv = e.fresh()
    e.b.add_op(OP.CONV1D_SSM, [xin, conv_w, conv, seq, C, k_conv])
    parts = [[], [], [], [], []]
    for ci in range(seq // chunk):
        rng = part_rng(seed, 10 + ci)
        kc = rng.standard_normal((H, chunk, D)).astype(np.float32)
        parts[0].append((kc / np.linalg.norm(kc, axis=-1, keepdims=True)).astype(np.float16))
        parts[1].append(rng.standard_normal((H, chunk, D)).astype(np.float16))
        parts[2].append(rng.standard_normal((H, chunk, D)).astype(np.float16))
        parts[3].append((1.0 / (1.0 + np.exp(-rng.standard_normal((H, chunk))))).astype(np.float16))
        parts[4].append(np.log(1.0 / (1.0 + np.exp(-rng.standard_normal((H, chunk))))).astype(np.float16))
    kk, vv, qq, beta, gg = (np.ascontiguousarray(np.concatenate(p, axis=1)) for p in parts)
    sk, sv, sq, sb, sg = (S(e.b.add_slot(a)) for a in (kk, vv, qq, beta, gg))
    nib_o, sc_o = rand_w4(part_rng(seed, 2), H * D, hidden)
    if quant == "w4":
        w_out = S(e.b.add_slot(np.concatenate([nib_o.reshape(-1), sc_o.view(np.uint8).reshape(-1)]), count=H * D * hidden))
    else:
        w_out = S(e.b.add_slot(np.ascontiguousarray(dequant_f16(nib_o, sc_o).T)))     # [N, K], as the emitter stores weights
    outs = []
    for ci in range(seq // chunk):
        t0, t1 = ci * chunk, (ci + 1) * chunk
        parts = []
        for src in (sk, sv, sq):
            y = e.fresh()
            e.b.add_op(OP.SLICE, [src, y, H * chunk * D, 3, 0, t0, 0, H, t1, D, 1, 1, 1, H, seq, D])
            parts.append(y)
        for src in (sb, sg):
            y = e.fresh()
            e.b.add_op(OP.SLICE, [src, y, H * chunk, 2, 0, t0, 0, H, t1, 0, 1, 1, 1, H, seq, 1])
            parts.append(y)
        yc = e.fresh()
        e.b.add_op(OP.DELTA_CHUNK, parts + [yc, ST(0), chunk, chunk, H, D, 0])
        yt = e.transpose3(yc, (H, chunk, D), (1, 0, 2))            # [chunk, H*D]
        yo = e.fresh()
        if quant == "w4":
            e.b.add_op(OP.MATMUL_W4A16, [yt, w_out, yo, chunk, H * D, hidden])
        else:
            e.b.add_op(OP.MATMUL_F16, [yt, w_out, yo, chunk, H * D, hidden, 2])
        outs.append(yo)
    man = dict(seq=seq, hidden=hidden, C=C, H=H, D=D, chunk=chunk, conv_temp=conv, chunk_out=outs,
               input_slot=face, quant=quant, n_ops=len(e.b.ops))
    return e.b.build(), man
