"""Generates tests/golden/golden_ops.npz: outputs of the reference executor
(compiled for the host from the reference tree by oracle/Makefile) on seeded
inputs, one entry per hot-path op. Run in a container that has the reference
tree; the .npz is committed so that every other machine can check the C oracle
and the CUDA kernels against the reference's own results.

    python tests/golden/make_golden.py
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine  # noqa: E402
from oracle.refexec import ref_lib  # noqa: E402


def cases():
    """name -> (builder fn(rng) -> (BlobBuilder, [out temps], {input arrays}))."""
    def r16(rng, shape, s=1.0):
        return (rng.standard_normal(shape) * s).astype(np.float16)

    def matmul(flags, M, K, N, Bn=0):
        def f(rng):
            nb = max(Bn, 1)
            a = r16(rng, (nb, K, M) if (flags & 1 and not Bn) else (nb, M, K))
            w = r16(rng, (nb, N, K) if flags & 2 else (nb, K, N), 0.2)
            b = BlobBuilder()
            sa, sw = b.add_slot(a), b.add_slot(w)
            b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, flags | ((4 | Bn << 16) if Bn else 0)])
            return b, [1], dict(a=a, w=w, dims=np.array([M, K, N, flags & 1, (flags >> 1) & 1, Bn]))
        return f

    def rms(rng):
        x, g, be = r16(rng, (6, 160)), rng.normal(1, 0.1, 160).astype(np.float16), r16(rng, 160, 0.1)
        x[0] *= np.float16(1e-4)
        b = BlobBuilder()
        sx, sg, sb = b.add_slot(x), b.add_slot(g), b.add_slot(be)
        b.add_op(OP.RMSNORM2, [S(sx), S(sg), S(sb), 1, x.size])
        return b, [1], dict(x=x, g=g, b=be)

    def softmax(rows, n):
        def f(rng):
            x = r16(rng, (rows, n), 4.0)
            b = BlobBuilder()
            b.add_op(OP.SOFTMAX, [S(b.add_slot(x)), 1, rows, n])
            return b, [1], dict(x=x)
        return f

    def kv(rng):
        nh, kvh, hd, nslots, steps = 8, 2, 64, 8, 11   # wraps the ring
        ks, vs = r16(rng, (steps, kvh * hd)), r16(rng, (steps, kvh * hd))
        b = BlobBuilder()
        b.add_states([kvh * hd * 4 * nslots])
        for i in range(steps):
            b.add_op(OP.KV_APPEND, [S(b.add_slot(ks[i])), S(b.add_slot(vs[i])), ST(0), i])
        # after wrapping, positions 3..10 are resident; gather needs [0, n_kv): use a second pass at small n
        b2 = BlobBuilder()
        b2.add_states([kvh * hd * 4 * nslots])
        for i in range(6):
            b2.add_op(OP.KV_APPEND, [S(b2.add_slot(ks[i])), S(b2.add_slot(vs[i])), ST(0), KV_POS_AUTO])
        b2.add_op(OP.KV_GATHER, [ST(0), 1, 2, KV_POS_AUTO, nh, kvh, hd])
        b2.add_op(OP.KV_GATHER, [ST(0), 3, 4, 5, nh, kvh, hd])
        return b2, [1, 2, 3, 4], dict(k=ks[:6], v=vs[:6], dims=np.array([nh, kvh, hd, nslots]))

    def conv(rng):
        seq, C, k = 19, 48, 4
        x, w = r16(rng, (seq, C)), r16(rng, (k, C), 0.5)
        b = BlobBuilder()
        b.add_states([(k - 1) * C * 4])
        sx, sw = b.add_slot(x), b.add_slot(w)
        b.add_op(OP.CONV1D_SSM, [S(sx), sw, 1, seq, C, k])
        for i in range(4):
            b.add_op(OP.CONV1D_SSM_STEP, [S(b.add_slot(x[i])), S(sw), 2 + i, ST(0), C, k])
        return b, [1, 2, 3, 4, 5], dict(x=x, w=w)

    def delta(rng):
        H, D, c, ntok = 2, 64, 16, 32
        k = r16(rng, (H, ntok, D))
        k = (k / np.linalg.norm(k.astype(np.float32), axis=-1, keepdims=True)).astype(np.float16)
        v, q = r16(rng, (H, ntok, D)), r16(rng, (H, ntok, D))
        beta = (1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16)
        g = np.log(1 / (1 + np.exp(-rng.standard_normal((H, ntok))))).astype(np.float16)
        b = BlobBuilder()
        b.add_states([H * D * D * 4])
        sl = [S(b.add_slot(a)) for a in (k, v, q, beta, g)]
        b.add_op(OP.DELTA_CHUNK, sl + [1, ST(0), c, ntok, H, D, 0])
        b.add_op(OP.DELTA_CHUNK, sl + [2, ST(0), c, ntok, H, D, 1])
        return b, [1, 2], dict(k=k, v=v, q=q, beta=beta, g=g, dims=np.array([H, D, c, ntok]))

    def unary(rng):
        x = r16(rng, 200, 2.0)
        b = BlobBuilder()
        sx = b.add_slot(x)
        for sub in range(17):
            b.add_op(OP.UNARY, [S(sx), 1 + sub, 200, sub])
        return b, list(range(1, 18)), dict(x=x)

    def binary(rng):
        a, c = r16(rng, 100, 3.0), r16(rng, 100, 3.0)
        b = BlobBuilder()
        sa, sc = b.add_slot(a), b.add_slot(c)
        for sub in range(6):
            b.add_op(OP.BINARY, [S(sa), S(sc), 1 + sub, 100, sub])
        return b, list(range(1, 7)), dict(a=a, b=c)

    return {
        "matmul_plain": matmul(0, 5, 96, 40), "matmul_t0": matmul(1, 8, 64, 33), "matmul_t1": matmul(2, 3, 80, 50),
        "matmul_t0t1": matmul(3, 16, 32, 32), "matmul_batched": matmul(0, 1, 64, 24, Bn=5),
        "matmul_batched_t1": matmul(2, 2, 48, 16, Bn=3),
        "rmsnorm2": rms, "softmax_wide": softmax(4, 64), "softmax_narrow": softmax(3, 21),
        "kv": kv, "conv": conv, "delta": delta, "unary": unary, "binary": binary,
    }


def main():
    out = {}
    for i, (name, fn) in enumerate(sorted(cases().items())):
        rng = np.random.default_rng(9000 + i)
        builder, temps, inputs = fn(rng)
        with tempfile.TemporaryDirectory() as d:
            lib = ref_lib(private_dir=d)
            assert lib is not None, "build oracle/_ref first (make -C oracle)"
            eng = Engine(lib, builder.build())
            eng.run()
            for t in temps:
                out["%s/out%d" % (name, t)] = eng.temp(t, np.uint16)
            eng.shutdown()
        for k, v in inputs.items():
            out["%s/in_%s" % (name, k)] = v
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_ops.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
