"""Generates tests/golden/decoder/: a Qwen3-shaped decoder synthesised by
gehtp_b200.netjson (heads * head_dim != hidden, rotate-half RoPE, causal
softmax attention, gated FFN) and compiled by the reference's own tool chain

    net.json + weights.tar --hnnx_compile--> tagged .bin --wtop_emit--> WTOP blob

without and with `--ddr-budget` (decoder_noplan.wtop / decoder_plan.wtop), plus

    ids.i32.raw          the input token ids, (7*i) mod vocab
    host_run.f32.raw     logits of the reference's f32 host executor (`host_run`)
    net.sha256           digest of the synthesised net.json and weight archive,
                         so a test can tell that the synthesiser still writes
                         the model these blobs were compiled from

The tools are built by `make -C oracle compiler` from where the reference tree
lies; run in a container that has that tree.

    GEHTP_REFERENCE_DIR=<reference tree> python tests/golden/make_decoder_blobs.py
"""
import hashlib
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gehtp_b200.netjson import DecoderShape, synth_decoder, write_net  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "decoder")
TOOLS = os.path.join(ROOT, "oracle", "_ref")
SHAPE = DecoderShape(layers=2, hidden=128, heads=4, head_dim=64, ffn=256, vocab=256, seq=64)
SEED = 20
DDR_BUDGET = 67108864


def sh(*cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise SystemExit("failed: " + " ".join(cmd))
    return r.stdout + r.stderr


def digest(*paths):
    h = hashlib.sha256()
    for p in paths:
        h.update(open(p, "rb").read())
    return h.hexdigest()


def compile_decoder(tmp, shape=SHAPE, seed=SEED, out=None):
    """Synthesises, compiles and emits both blobs into `out`; returns the net digest."""
    out = out or tmp
    net, weights = synth_decoder(shape, seed)
    nj, tar = os.path.join(tmp, "net.json"), os.path.join(tmp, "weights.tar")
    write_net(net, weights, nj, tar)
    for name, extra in (("decoder_noplan", []), ("decoder_plan", ["--ddr-budget", str(DDR_BUDGET)])):
        tagged = os.path.join(tmp, name + ".bin")
        sh(os.path.join(TOOLS, "hnnx_compile"), "--net-json", nj, "--weights-bin", tar, "--format", "tagged", *extra,
           "--output", tagged)
        print(sh(os.path.join(TOOLS, "wtop_emit"), "--bin", tagged, "--out", os.path.join(out, name + ".wtop"),
                 "--manifest", os.path.join(out, name + ".manifest.json")).strip())
    return digest(nj, tar)


def main():
    ref_root = os.environ.get("GEHTP_REFERENCE_DIR") or sys.exit("set GEHTP_REFERENCE_DIR to the reference tree")
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-j8", "compiler", "REF=" + ref_root], check=True)
    os.makedirs(OUT, exist_ok=True)
    ids = (np.arange(SHAPE.seq) * 7 % SHAPE.vocab).astype(np.int32)
    ids.tofile(os.path.join(OUT, "ids.i32.raw"))
    with tempfile.TemporaryDirectory() as tmp:
        d = compile_decoder(tmp, out=OUT)
        open(os.path.join(OUT, "net.sha256"), "w").write(d + "\n")
        sh(os.path.join(TOOLS, "host_run"), "--bin", os.path.join(tmp, "decoder_plan.bin"), "--input-f32",
           os.path.join(OUT, "ids.i32.raw"), "--out", os.path.join(OUT, "host_run.f32.raw"))


if __name__ == "__main__":
    main()
