"""Generates tests/golden/probe/: the reference's own `qnn_probe` model compiled
by the reference's own tool chain, and what the reference computes for it.

    net.json + weights --hnnx_compile--> tagged .bin --wtop_emit--> WTOP blob

twice: without a memory plan (`probe_noplan.wtop`) and with `--ddr-budget`
(`probe_plan.wtop`: carries the TAG_MEM_PLAN offsets as a TEMPOFF slot). Beside
the blobs and their manifests it stores

    ids.i32.raw          the 32 input token ids, (7*i) mod 256
    host_run.f32.raw     logits of the reference's f32 host executor (`host_run`)
    probe_ext_v2.wtop    the unplanned model again, emitted with --ext-weights --force-v2:
                         descriptors only, weights in probe_ext_v2.weights.bin
    ref_ops.npz          every op's output as the reference's device executor
                         compiled for the host leaves it (dump hook, no-plan blob),
                         key "op<idx>_t<temp>", fp16 bits

The tools are built by `make -C oracle compiler` from where the reference tree
lies. Run in a container that has that tree; the outputs are committed
so that any other machine can run the compiled blobs and compare.

    GEHTP_REFERENCE_DIR=<reference tree> python tests/golden/make_probe_blobs.py
"""
import glob
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gehtp_b200.wtop import Engine, op_out_temps  # noqa: E402
from oracle.refexec import ref_lib  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "probe")
TOOLS = os.path.join(ROOT, "oracle", "_ref")
DDR_BUDGET = 67108864


def sh(*cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise SystemExit("failed: " + " ".join(cmd))
    return r.stdout + r.stderr


def main():
    ref_root = os.environ.get("GEHTP_REFERENCE_DIR") or sys.exit("set GEHTP_REFERENCE_DIR to the reference tree")
    probe = os.path.join(ref_root, "test_models", "qnn_probe")
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-j8", "compiler", "ref", "REF=" + ref_root], check=True)
    os.makedirs(OUT, exist_ok=True)
    ids = (np.arange(32) * 7 % 256).astype(np.int32)
    ids.tofile(os.path.join(OUT, "ids.i32.raw"))
    with tempfile.TemporaryDirectory() as tmp:
        for name, extra in (("probe_noplan", []), ("probe_plan", ["--ddr-budget", str(DDR_BUDGET)])):
            tagged = os.path.join(tmp, name + ".bin")
            sh(os.path.join(TOOLS, "hnnx_compile"), "--net-json", os.path.join(probe, "model_float_net.json"),
               "--weights-bin", os.path.join(probe, "model_float.bin"), "--format", "tagged", *extra, "--output", tagged)
            print(sh(os.path.join(TOOLS, "wtop_emit"), "--bin", tagged, "--out", os.path.join(OUT, name + ".wtop"),
                     "--manifest", os.path.join(OUT, name + ".manifest.json")).strip())
        # the same model with the weights outside the blob (EXT_WGT slots + <blob>.weights.bin,
        # wtop_emit.cpp:700-711) and 24-byte v2 slot records with 64-bit offsets
        print(sh(os.path.join(TOOLS, "wtop_emit"), "--bin", os.path.join(tmp, "probe_noplan.bin"), "--out",
                 os.path.join(OUT, "probe_ext_v2.wtop"), "--manifest", os.path.join(OUT, "probe_ext_v2.manifest.json"),
                 "--ext-weights", "--force-v2").strip())
        sh(os.path.join(TOOLS, "host_run"), "--bin", os.path.join(tmp, "probe_plan.bin"), "--input-f32",
           os.path.join(OUT, "ids.i32.raw"), "--out", os.path.join(OUT, "host_run.f32.raw"))

        # per-op outputs of the reference's device executor (scalar CPU paths) on the no-plan blob
        buf = np.fromfile(os.path.join(OUT, "probe_noplan.wtop"), np.uint8)
        lib = ref_lib(private_dir=tmp)
        eng = Engine(lib, buf)
        pairs = [(i, t) for i in range(eng.blob.n_ops) for t in op_out_temps(eng.blob.ops[i])]
        spec = ",".join("%d:%d" % p for p in pairs).encode()
        for f in glob.glob("/tmp/hook_*_*.f16.raw"):
            os.remove(f)
        lib.wt_exec_set_hook(spec)
        eng.run_io(ids, 0)
        lib.wt_exec_set_hook(None)
        dumps = {}
        for i, t in pairs:
            fn = "/tmp/hook_%d_%d.f16.raw" % (i, t)
            dumps["op%d_t%d" % (i, t)] = np.fromfile(fn, np.uint16)
            os.remove(fn)
        eng.shutdown()
        np.savez_compressed(os.path.join(OUT, "ref_ops.npz"), **dumps)
        print("ref_ops.npz: %d op outputs, %d bytes" % (len(dumps), os.path.getsize(os.path.join(OUT, "ref_ops.npz"))))


if __name__ == "__main__":
    main()
