"""Writes a decoder-only transformer as a `net.json` + weight archive in the
dialect the reference's graph compiler reads, so that runlists for this engine
can be COMPILED by the reference's own tools (hnnx_compile -> wtop_emit)
instead of packed by hand.

The dialect is what compiler/src/frontend/qnn_ir_loader.cpp accepts
(parse_tensors :99, parse_nodes :174, build_graph :217) and what
test_models/qnn_probe/model_float_net.json uses:

    graph.tensors{name: {id, type, data_type, dims}}     type 0 input, 1 output,
                                                         3 activation, 4 static
    graph.nodes{name: {type, input_names, output_names,
                       tensor_params{param: {tensor: {id,type,data_type,dims,data}}},
                       scalar_params{param: {"<dtype id>": value}}}}

Nodes must appear in execution order and tensor ids must grow along it (the
loader creates ops sorted by the id of their output tensor). Static tensors
carry no data in the JSON; their float32 values travel in a TAR archive with
one `<tensor name>.raw` member each (hnnx_compile.cpp:143 passes a TAR
through unchanged).

One block, in the probe's own node vocabulary:

    RmsNorm -> FullyConnected(qkv) -> Split -> [rotate-half RoPE on q and k]
    -> Transpose -> MatMul(q, k^T) -> Div(sqrt(hd)) -> Add(causal mask)
    -> Softmax -> MatMul(p, v) -> Transpose -> FullyConnected(o) -> Add
    -> RmsNorm -> FullyConnected(gate) * sigmoid * FullyConnected(up)
    -> FullyConnected(down) -> Add

Nothing here touches the GPU or the engine: the output is two files.
"""
import io
import json
import tarfile
from dataclasses import dataclass

import numpy as np

F32, U32, I32, BOOL, STR = 562, 306, 50, 1288, 1544      # data_type ids of the dialect
T_IN, T_OUT, T_ACT, T_STATIC = 0, 1, 3, 4
OP_ADD, OP_DIV, OP_MUL = 0, 2, 13   # Eltwise_Binary "operation"
OP_NEG = 8                          # Eltwise_Unary "operation"
OP_SIGMOID = 6                      # ElementWiseNeuron "operation"


@dataclass
class DecoderShape:
    """Sizes of the synthesised model; `heads * head_dim` need not equal `hidden`."""
    layers: int = 2
    hidden: int = 256
    heads: int = 4
    head_dim: int = 64
    ffn: int = 512
    vocab: int = 512
    seq: int = 64
    rope_theta: float = 1.0e6
    eps: float = 1e-6


class _Net:
    def __init__(self):
        self.tensors, self.nodes, self.weights = {}, {}, {}
        self.next_id = 1

    def _id(self):
        i = self.next_id
        self.next_id += 1
        return i

    def tensor(self, name, ttype, dtype, dims):
        if name not in self.tensors:
            self.tensors[name] = {"id": self._id(), "type": ttype, "data_type": dtype, "dims": [int(d) for d in dims]}
        return name

    def static(self, name, values):
        values = np.ascontiguousarray(values, np.float32)
        self.weights[name] = values
        return self.tensor(name, T_STATIC, F32, values.shape)

    def node(self, name, ntype, inputs, outputs, scalars=None, tparams=None):
        """`outputs` = [(name, dims)] (the last node's output may already exist as the graph
        output); `scalars` = {param: (dtype id, value)}; `tparams` = {param: (dtype id, array)}."""
        tp = {}
        for pname, (dtype, arr) in (tparams or {}).items():
            arr = np.asarray(arr)
            tname = "%s_%s" % (name, pname)
            tp[pname] = {tname: {"id": self._id(), "type": T_STATIC, "data_type": dtype, "dims": list(arr.shape),
                                 "data": arr.tolist()}}
        for oname, dims in outputs:
            self.tensor(oname, T_ACT, F32, dims)
        self.nodes[name] = {
            "package": "qti.aisw", "type": ntype, "tensor_params": tp,
            "scalar_params": dict({k: {str(dt): v} for k, (dt, v) in (scalars or {}).items()},
                                  packageName={str(STR): "qti.aisw"}),
            "input_names": list(inputs), "output_names": [o for o, _ in outputs]}
        return outputs[0][0]


def _rope_tables(shape):
    half = shape.head_dim // 2
    inv = shape.rope_theta ** (-np.arange(half, dtype=np.float64) / half)
    ang = np.arange(shape.seq, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=1)
    return (np.cos(ang).astype(np.float32).reshape(1, shape.seq, 1, shape.head_dim),
            np.sin(ang).astype(np.float32).reshape(1, shape.seq, 1, shape.head_dim))


def synth_decoder(shape: DecoderShape, seed: int = 0):
    """Returns (net dict ready for json.dump, {static tensor name: float32 array})."""
    s, h, nh, hd = shape.seq, shape.hidden, shape.heads, shape.head_dim
    qd = nh * hd
    rng = np.random.default_rng(seed)
    n = _Net()

    def w(rows, cols):
        return (rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32)

    def gamma():
        return (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)

    def fc(prefix, x, x_dims, weight, n_out):
        """[1, s, k] -> Reshape [s, k] -> FullyConnected with a [n_out, k] weight -> Reshape [1, s, n_out]"""
        k = x_dims[-1]
        a = n.node(prefix + "_pre_reshape", "Reshape", [x], [(prefix + "_pre_reshape", [s, k])])
        wname = n.static(prefix + "_weight", weight)
        b = n.node(prefix, "FullyConnected", [a, wname], [(prefix + "_output_0_fc", [s, n_out])])
        return n.node(prefix + "_post_reshape", "Reshape", [b], [(prefix + "_output_0", [1, s, n_out])])

    def rms(prefix, x, g):
        gname = n.static(prefix + "_weight", g)
        bname = n.static(prefix + "_bias", np.zeros(h, np.float32))
        return n.node("rms_norm_" + prefix, "RmsNorm", [x, gname, bname], [(prefix + "_output_0", [1, s, h])],
                      scalars={"epsilon": (F32, float(np.float32(shape.eps)))}, tparams={"axes": (U32, [2])})

    def rope(prefix, x, cos, sin):
        """x * cos + concat(-x[..., hd/2:], x[..., :hd/2]) * sin on [1, s, nh, hd]"""
        full, half = [1, s, nh, hd], [1, s, nh, hd // 2]
        masks = {"begin_mask": (U32, 0), "end_mask": (U32, 0), "new_axes_mask": (U32, 0), "shrink_axes": (U32, 0)}
        a = n.node(prefix + "_Mul", "Eltwise_Binary", [x, cos], [(prefix + "_Mul_output_0", full)],
                   scalars={"operation": (U32, OP_MUL)})
        hi = n.node(prefix + "_Slice", "StridedSlice", [x], [(prefix + "_Slice_output_0", half)], scalars=masks,
                    tparams={"ranges": (I32, [[0, 1, 1], [0, s, 1], [0, nh, 1], [hd // 2, hd, 1]])})
        neg = n.node(prefix + "_Neg", "Eltwise_Unary", [hi], [(prefix + "_Neg_output_0", half)],
                     scalars={"operation": (U32, OP_NEG)})
        lo = n.node(prefix + "_Slice_1", "StridedSlice", [x], [(prefix + "_Slice_1_output_0", half)], scalars=masks,
                    tparams={"ranges": (I32, [[0, 1, 1], [0, s, 1], [0, nh, 1], [0, hd // 2, 1]])})
        rot = n.node(prefix + "_Concat", "Concat", [neg, lo], [(prefix + "_Concat_output_0", full)],
                     scalars={"axis": (U32, 3)})
        b = n.node(prefix + "_Mul_1", "Eltwise_Binary", [rot, sin], [(prefix + "_Mul_1_output_0", full)],
                   scalars={"operation": (U32, OP_MUL)})
        return n.node(prefix + "_Add", "Eltwise_Binary", [a, b], [(prefix + "_Add_output_0", full)],
                      scalars={"operation": (U32, OP_ADD)})

    n.tensor("tokens", T_IN, I32, [1, s])
    emb = n.static("embed_weight", rng.standard_normal((shape.vocab, h)).astype(np.float32))
    x = n.node("_embed_Gather", "Gather", [emb, "tokens"], [("_embed_Gather_output_0", [1, s, h])],
               scalars={"axis": (I32, 0)})
    cos_t, sin_t = _rope_tables(shape)
    mask = np.where(np.arange(s)[None, :] > np.arange(s)[:, None], -10000.0, 0.0).astype(np.float32)
    cos = sin = mname = sname = None
    for li in range(shape.layers):
        p = "_blocks_%d" % li
        y = rms(p + "_norm1", x, gamma())
        qkv = fc(p + "_attn_qkv_MatMul", y, [1, s, h], w(3 * qd, h), 3 * qd)
        n.node(p + "_attn_Split", "Split", [qkv], [(p + "_attn_Split_output_%d" % i, [1, s, qd]) for i in range(3)],
               scalars={"axis": (U32, 2)}, tparams={"split_index": (U32, [qd, 2 * qd])})
        q4, k4, v4 = [n.node(p + "_attn_Reshape%s" % suf, "Reshape", [p + "_attn_Split_output_%d" % i],
                             [(p + "_attn_Reshape%s_output_0" % suf, [1, s, nh, hd])])
                      for i, suf in enumerate(("", "_1", "_2"))]
        if cos is None:
            cos, sin = n.static("rope_cos", cos_t), n.static("rope_sin", sin_t)
        qr = rope(p + "_attn_rope", q4, cos, sin)
        kr = rope(p + "_attn_rope_1", k4, cos, sin)
        qt = n.node(p + "_attn_Transpose", "Transpose", [qr], [(p + "_attn_Transpose_output_0", [1, nh, s, hd])],
                    tparams={"perm": (U32, [0, 2, 1, 3])})
        vt = n.node(p + "_attn_Transpose_1", "Transpose", [v4], [(p + "_attn_Transpose_1_output_0", [1, nh, s, hd])],
                    tparams={"perm": (U32, [0, 2, 1, 3])})
        kt = n.node(p + "_attn_Transpose_2", "Transpose", [kr], [(p + "_attn_Transpose_2_output_0", [1, nh, hd, s])],
                    tparams={"perm": (U32, [0, 2, 3, 1])})
        mm = {"transpose_in0": (BOOL, 0), "transpose_in1": (BOOL, 0)}
        sc = n.node(p + "_attn_MatMul", "MatMul", [qt, kt], [(p + "_attn_MatMul_output_0", [1, nh, s, s])], scalars=mm)
        if sname is None:
            sname = n.static("attn_scale_div", np.array([np.sqrt(hd)], np.float32))
        sc = n.node(p + "_attn_Div", "Eltwise_Binary", [sc, sname], [(p + "_attn_Div_output_0", [1, nh, s, s])],
                    scalars={"operation": (U32, OP_DIV)})
        if mname is None:
            mname = n.static("causal_mask", mask)
        sc = n.node(p + "_attn_Add", "Eltwise_Binary", [sc, mname], [(p + "_attn_Add_output_0", [1, nh, s, s])],
                    scalars={"operation": (U32, OP_ADD)})
        pr = n.node(p + "_attn_Softmax", "Softmax", [sc], [(p + "_attn_Softmax_output_0", [1, nh, s, s])],
                    scalars={"axis": (U32, 3), "beta": (F32, 1.0)})
        o = n.node(p + "_attn_MatMul_1", "MatMul", [pr, vt], [(p + "_attn_MatMul_1_output_0", [1, nh, s, hd])], scalars=mm)
        o = n.node(p + "_attn_Transpose_3", "Transpose", [o], [(p + "_attn_Transpose_3_output_0", [1, s, nh, hd])],
                   tparams={"perm": (U32, [0, 2, 1, 3])})
        o = n.node(p + "_attn_Reshape_3", "Reshape", [o], [(p + "_attn_Reshape_3_output_0", [1, s, qd])])
        o = fc(p + "_attn_out_MatMul", o, [1, s, qd], w(h, qd), h)
        x = n.node(p + "_Add", "Eltwise_Binary", [x, o], [(p + "_Add_output_0", [1, s, h])],
                   scalars={"operation": (U32, OP_ADD)})
        y = rms(p + "_norm2", x, gamma())
        g = fc(p + "_ffn_gate_MatMul", y, [1, s, h], w(shape.ffn, h), shape.ffn)
        sg = n.node(p + "_ffn_Sigmoid", "ElementWiseNeuron", [g], [(p + "_ffn_Sigmoid_output_0", [1, s, shape.ffn])],
                    scalars={"operation": (U32, OP_SIGMOID)})
        g = n.node(p + "_ffn_Mul", "Eltwise_Binary", [g, sg], [(p + "_ffn_Mul_output_0", [1, s, shape.ffn])],
                   scalars={"operation": (U32, OP_MUL)})
        u = fc(p + "_ffn_up_MatMul", y, [1, s, h], w(shape.ffn, h), shape.ffn)
        g = n.node(p + "_ffn_Mul_1", "Eltwise_Binary", [g, u], [(p + "_ffn_Mul_1_output_0", [1, s, shape.ffn])],
                   scalars={"operation": (U32, OP_MUL)})
        d = fc(p + "_ffn_down_MatMul", g, [1, s, shape.ffn], w(h, shape.ffn), h)
        x = n.node(p + "_Add_1", "Eltwise_Binary", [x, d], [(p + "_Add_1_output_0", [1, s, h])],
                   scalars={"operation": (U32, OP_ADD)})
    y = rms("_norm_out", x, gamma())
    a = n.node("_lm_head_MatMul_pre_reshape", "Reshape", [y], [("_lm_head_MatMul_pre_reshape", [s, h])])
    wname = n.static("lm_head_weight", w(shape.vocab, h))
    b = n.node("_lm_head_MatMul", "FullyConnected", [a, wname], [("logits_fc", [s, shape.vocab])])
    n.tensor("logits", T_OUT, F32, [1, s, shape.vocab])
    n.node("_lm_head_MatMul_post_reshape", "Reshape", [b], [("logits", [1, s, shape.vocab])])
    net = {"model.cpp": "", "model.bin": "", "converter_command": "gehtp_b200.netjson.synth_decoder",
           "op_types": sorted({v["type"] for v in n.nodes.values()}),
           "graph": {"tensors": n.tensors, "nodes": n.nodes}}
    return net, n.weights


def write_net(net, weights, json_path, tar_path):
    """net.json plus the weight TAR (`<tensor>.raw`, float32, in tensor order)."""
    with open(json_path, "w") as f:
        json.dump(net, f)
    with tarfile.open(tar_path, "w", format=tarfile.USTAR_FORMAT) as tar:
        for name, arr in weights.items():
            raw = np.ascontiguousarray(arr, np.float32).tobytes()
            info = tarfile.TarInfo(name + ".raw")
            info.size = len(raw)
            tar.addfile(info, io.BytesIO(raw))


def decoder_f32(shape: DecoderShape, weights, ids):
    """The synthesised graph in float64 numpy (what the compiled runlist approximates in fp16):
    logits [seq, vocab] for `ids`. Used by tests to check that the compiled model still is this model."""
    s, nh, hd = shape.seq, shape.heads, shape.head_dim
    W = {k: v.astype(np.float64) for k, v in weights.items()}

    def rms(x, prefix):
        r = np.sqrt((x * x).mean(-1, keepdims=True) + shape.eps)
        return x / r * W[prefix + "_weight"] + W[prefix + "_bias"]

    def rope(x):
        rot = np.concatenate([-x[..., hd // 2:], x[..., :hd // 2]], -1)
        return x * W["rope_cos"][0] + rot * W["rope_sin"][0]

    x = W["embed_weight"][np.asarray(ids).reshape(-1)]
    for li in range(shape.layers):
        p = "_blocks_%d" % li
        qkv = rms(x, p + "_norm1") @ W[p + "_attn_qkv_MatMul_weight"].T
        q, k, v = [t.reshape(s, nh, hd) for t in np.split(qkv, 3, axis=1)]
        q, k = rope(q), rope(k)
        sc = np.einsum("qhd,khd->hqk", q, k) / W["attn_scale_div"][0] + W["causal_mask"][None]
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        sc /= sc.sum(-1, keepdims=True)
        o = np.einsum("hqk,khd->qhd", sc, v).reshape(s, nh * hd)
        x = x + o @ W[p + "_attn_out_MatMul_weight"].T
        y = rms(x, p + "_norm2")
        g = y @ W[p + "_ffn_gate_MatMul_weight"].T
        g = g / (1.0 + np.exp(-g)) * (y @ W[p + "_ffn_up_MatMul_weight"].T)
        x = x + g @ W[p + "_ffn_down_MatMul_weight"].T
    return rms(x, "_norm_out") @ W["lm_head_weight"].T
