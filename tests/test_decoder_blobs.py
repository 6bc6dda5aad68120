"""A decoder written by gehtp_b200.netjson and compiled by the reference's chain.

tests/golden/decoder/ holds a 2-layer Qwen3-shaped model (hidden 128, 4 heads of 64,
FFN 256, 64 tokens) that gehtp_b200.netjson.synth_decoder wrote as net.json + weight
archive and the reference's `hnnx_compile` + `wtop_emit` compiled
(compiler/tools/hnnx_compile.cpp:286 main, compiler/tools/wtop_emit.cpp:74 emit),
without and with `--ddr-budget`, together with the f32 logits of the reference's
`host_run` (tests/golden/make_decoder_blobs.py wrote them). The CPU tests tie the
synthesiser, the float64 restatement of the graph and the fixtures to each other
and run the blob on the reference executor; the GPU tests run both blobs through
the CUDA engine unchanged.
"""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

from conftest import cos_sim
from gehtp_b200.netjson import DecoderShape, decoder_f32, synth_decoder, write_net
from gehtp_b200.wtop import OP, Engine, parse_blob

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoder")
sys.path.insert(0, os.path.dirname(HERE))
import make_decoder_blobs as gen  # noqa: E402

SHAPE = gen.SHAPE


def load(name):
    buf = np.fromfile(os.path.join(HERE, name + ".wtop"), np.uint8)
    man = json.load(open(os.path.join(HERE, name + ".manifest.json")))
    return buf, man


def ids():
    return np.fromfile(os.path.join(HERE, "ids.i32.raw"), np.int32)


def host_logits():
    return np.fromfile(os.path.join(HERE, "host_run.f32.raw"), np.float32).reshape(SHAPE.seq, SHAPE.vocab)


def check_logits(got_f16, what):
    got = np.asarray(got_f16, np.float16).astype(np.float64).reshape(SHAPE.seq, SHAPE.vocab)
    want = host_logits().astype(np.float64)
    assert cos_sim(got, want) >= 0.9999, what
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), what
    assert (got.argmax(1) == want.argmax(1)).all(), what + ": top-1 differs"


def test_dialect_of_the_synthesised_net():
    """Ids grow along the node order, every input exists before its consumer, node types are the
    probe model's vocabulary, and one weight array exists per static graph tensor."""
    net, weights = synth_decoder(SHAPE, gen.SEED)
    tensors, nodes = net["graph"]["tensors"], net["graph"]["nodes"]
    assert set(net["op_types"]) <= {"Concat", "ElementWiseNeuron", "Eltwise_Binary", "Eltwise_Unary", "FullyConnected",
                                    "Gather", "MatMul", "Reshape", "RmsNorm", "Softmax", "Split", "StridedSlice",
                                    "Transpose"}
    seen, last = {n for n, t in tensors.items() if t["type"] in (0, 4)}, 0
    for name, node in nodes.items():
        for i in node["input_names"]:
            assert i in seen, (name, i)
        for o in node["output_names"]:
            assert tensors[o]["id"] > last, name
            last = tensors[o]["id"]
            seen.add(o)
        for tp in node["tensor_params"].values():
            (t,) = tp.values()
            assert t["type"] == 4 and np.asarray(t["data"]).shape == tuple(t["dims"])
    all_ids = [t["id"] for t in tensors.values()] + [t["id"] for n in nodes.values() for tp in n["tensor_params"].values()
                                                     for t in tp.values()]
    assert len(set(all_ids)) == len(all_ids)
    assert {n for n, t in tensors.items() if t["type"] == 4} == set(weights)
    for n, a in weights.items():
        assert list(a.shape) == tensors[n]["dims"] and a.dtype == np.float32
    assert [n for n, t in tensors.items() if t["type"] == 1] == ["logits"]
    assert len(nodes) == 5 + 50 * SHAPE.layers


def test_fixture_is_this_model(tmp_path):
    """The synthesiser still writes the files the fixture was compiled from, and the reference's
    f32 host executor computed what the float64 restatement of the graph computes."""
    net, weights = synth_decoder(SHAPE, gen.SEED)
    write_net(net, weights, tmp_path / "net.json", tmp_path / "weights.tar")
    h = hashlib.sha256((tmp_path / "net.json").read_bytes() + (tmp_path / "weights.tar").read_bytes()).hexdigest()
    assert h == open(os.path.join(HERE, "net.sha256")).read().strip()
    want = decoder_f32(SHAPE, weights, ids())
    assert np.abs(host_logits() - want).max() <= 1e-4 * np.abs(want).max()


def test_recompile_reproduces_the_fixture(tmp_path):
    """With the reference's tools at hand (make -C oracle compiler) the chain gives the committed bytes again."""
    if not os.path.exists(os.path.join(gen.TOOLS, "hnnx_compile")):
        pytest.skip("reference compiler not built here")
    gen.compile_decoder(str(tmp_path))
    for name in ("decoder_noplan", "decoder_plan"):
        assert (tmp_path / (name + ".wtop")).read_bytes() == open(os.path.join(HERE, name + ".wtop"), "rb").read(), name


def test_compiled_decoder_parses(cuda):
    for name in ("decoder_noplan", "decoder_plan"):
        buf, man = load(name)
        rc, blob = parse_blob(cuda, buf)
        assert rc == 0 and blob.n_ops == man["n_ops"] and blob.n_slots == man["n_slots"]
        assert [blob.ops[i].opcode for i in range(blob.n_ops)] == man["opcodes"]
        assert man["input_elems"] == SHAPE.seq
        codes = set(man["opcodes"])
        assert {OP.GATHER, OP.RMSNORM2, OP.MATMUL_F16, OP.SOFTMAX, OP.TRANSPOSE_GEN} <= codes


def test_reference_executor_on_the_compiled_decoder(ref):
    buf, man = load("decoder_noplan")
    eng = Engine(ref, buf)
    eng.run_io(ids(), 0)
    check_logits(eng.temp(man["output_temp"]), "reference executor")
    eng.shutdown()


@pytest.mark.gpu
def test_compiled_decoder_runs_unchanged(cuda, ref):
    """Both blobs through the CUDA engine, one kernel per op and fused, eager and replayed: the host_run
    gate holds, the planned blob gives the unplanned one's bits, and the one-kernel-per-op logits stay
    within the fp16 gate of the reference executor's."""
    eng = Engine(ref, load("decoder_noplan")[0])
    eng.run_io(ids(), 0)
    ref_logits = eng.temp(load("decoder_noplan")[1]["output_temp"]).astype(np.float64)
    eng.shutdown()
    logits = {}
    for name in ("decoder_noplan", "decoder_plan"):
        buf, man = load(name)
        for fusion in (1, 0):
            cuda.gehtp_cuda_set_fusion(fusion)
            eng = Engine(cuda, buf)
            out = np.zeros(SHAPE.seq * SHAPE.vocab, np.float16)
            runs = []
            for _ in range(4):
                out[:] = 0
                eng.run_io(ids(), man["output_temp"], out)
                check_logits(out, "%s fusion=%d" % (name, fusion))
                runs.append(out.copy())
            assert all(np.array_equal(runs[0].view(np.uint16), r.view(np.uint16)) for r in runs[1:])
            # slices of tables in weight slots are made once in the fused plan of the unplanned blob; the planned
            # blob's temps share memory (static table), nothing is kept across runs there
            consts = cuda.gehtp_cuda_const_ops()
            assert consts >= 1 if (fusion and name == "decoder_noplan") else consts == 0, (name, fusion, consts)
            logits[(name, fusion)] = runs[0]
            eng.shutdown()
    cuda.gehtp_cuda_set_fusion(1)
    for fusion in (0, 1):
        assert np.array_equal(logits[("decoder_noplan", fusion)].view(np.uint16),
                              logits[("decoder_plan", fusion)].view(np.uint16))
        got = logits[("decoder_noplan", fusion)].astype(np.float64)
        assert np.abs(got - ref_logits).max() <= 1e-2 * np.abs(ref_logits).max()
        assert cos_sim(got, ref_logits) >= 0.9999
