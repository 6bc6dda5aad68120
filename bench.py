"""Decode throughput of a Qwen3-4B-shaped W4A16 decoder runlist on B200.

    python bench.py --gpus N --steps K --warmup W            (our arm)
    python bench.py --impl reference --gpus N --steps K ...   (the reference's CPU path)

One step = one decode step of the whole runlist (36 layers + lm_head) for a
batch of sequences that all sit at a KV context of about 8192 positions.
Rank 0 prints one JSON line. `value` is measured with the step's input face
already in HBM; `e2e` goes through wt_exec_run_io with host buffers (host to
device copy of the face, device to host read of the chosen tokens inside the
timed region). With N > 1 the projections are tensor-parallel (column / row
sharded runlists per rank, NCCL all-reduce inside the engine after the
row-parallel ones).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "qwen3_4b_shape_w4a16_decode_tokens_per_s"
UNIT = "tok/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--shard-of", type=int, default=1,
                    help="profiling aid for 1 GPU: run rank 0's shard of an N-way tensor-parallel split without the "
                         "all-reduces (shapes and timing of one rank; the numbers it prints are not bench values)")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--micro", default=None, choices=["gemv", "lmhead", "gemm", "gemm1", "gemm512", "headline", "gemmtiles", "attn", "attn8", "norm", "prefill", "gdn", "all"],
                    help="time single kernels (device-resident operands, graph replay) instead of the decode step")
    return ap.parse_args()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (keyed by kernel group, batch, context, GPUs); None for other workloads.
NCU_TRAFFIC = {
    # attn_decode_tma_kernel, batch 8, ctx 8192, 1 GPU: 268.56 MB read + 4.31 MB written per launch
    # (profiles/attn_decode_tma_b8_ctx8192.md); the rotary/append and merge kernels of the unit are not included
    ("attn_decode", 8, 8192, 1): 268555264 + 4312320,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 8 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 8:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def w4_bytes(M, K, N):
    """Algorithmic bytes of one W4A16 matmul: nibbles + scales + activations in + out."""
    return K * N // 2 + 2 * (K // 64) * N + 2 * M * K + 2 * M * N


def classify_units(blob, op_ms, man, n_kv):
    """Groups the launch units of one profiled step: name -> [launches, total ms, algorithmic bytes]."""
    from gehtp_b200.wtop import OP
    groups = {}

    def add(name, ms, nbytes):
        g = groups.setdefault(name, [0, 0.0, 0])
        g[0] += 1
        g[1] += ms
        g[2] += nbytes
    B = man["B"]
    i, n = 0, blob.n_ops
    while i < n:
        ms = op_ms[i]
        op = blob.ops[i]
        if ms <= 0.0:
            i += 1
            continue
        if op.opcode == OP.MATMUL_W4A16 and i + 1 < n and blob.ops[i + 1].opcode == OP.SPLIT and op_ms[i + 1] <= 0.0:
            # the q|k|v projection heads the attention unit (rotary + append in its epilogue, then attention + merge);
            # the unit is filed under attention, whose KV bytes dominate it
            add("attn_decode", ms, 2 * n_kv * man["kv_elems"] * 2 + 4 * man["q_elems"])
        elif op.opcode == OP.MATMUL_W4A16:
            M, K, N = op.args[3], op.args[4], op.args[5]
            nb = w4_bytes(M, K, N)
            dual = (i + 3 < n and blob.ops[i + 1].opcode == OP.UNARY and blob.ops[i + 3].opcode == OP.MATMUL_W4A16
                    and op_ms[i + 3] <= 0.0)
            if dual:
                nb += K * N // 2 + 2 * (K // 64) * N
            add("w4a16_gemv", ms, nb)
        elif op.opcode == OP.SPLIT and i + 1 < n and op_ms[i + 1] <= 0.0:
            kv_elems = man["kv_elems"]
            add("attn_decode", ms, 2 * n_kv * kv_elems * 2 + 4 * man["q_elems"])
        elif op.opcode == OP.ADD and i + 1 < n and op_ms[i + 1] <= 0.0:
            add("add_rmsnorm", ms, 4 * op.args[3] * 2)
        elif op.opcode == OP.RMSNORM2:
            add("rmsnorm", ms, 2 * op.args[4] * 2)
        else:
            add("other", ms, 0)
        i += 1
    return groups


def run_ours(args, rank, world):
    import torch
    import gehtp_b200
    from gehtp_b200.runlists import QWEN3_4B, build_decode_runlist, decode_face
    from gehtp_b200.wtop import Engine

    cfg = QWEN3_4B
    B, ctx, K, W = args.batch, args.ctx, args.steps, args.warmup
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    lib = gehtp_b200.lib()
    assert lib.gehtp_cuda_set_device(local) == 0, "no CUDA device"
    if world > 1:
        init_tp(lib, rank, world)

    t0 = time.time()
    shard = world if world > 1 else max(args.shard_of, 1)
    buf, man = build_decode_runlist(cfg, B, ctx, seed=1004, quant="w4", n_layers=args.layers, tp=shard, rank=rank)
    kvh, nh, hd = cfg.kv_heads // shard, cfg.n_heads // shard, cfg.head_dim
    man["kv_elems"], man["q_elems"] = B * kvh * hd, B * nh * hd
    eng = Engine(lib, buf)
    err = ctypes.create_string_buffer(256)
    if world > 1:
        idx = (ctypes.c_uint32 * len(man["row_parallel_ops"]))(*man["row_parallel_ops"])
        assert lib.gehtp_cuda_tp_allreduce_after(idx, len(man["row_parallel_ops"])) == 0
    total_steps = max(W + K, 6)
    p0 = max(ctx - total_steps, 0)

    # KV rings ~ N(0,1) for positions [0, ctx), generated on the device
    ring_elems = ctx * 2 * man["kv_elems"]
    for li in range(man["layers"]):
        kv = torch.randn(ring_elems, device="cuda", dtype=torch.float16)
        rc = lib.gehtp_cuda_state_load(ctypes.byref(eng.blob), li, kv.data_ptr(), ring_elems * 2, 1, man["kv_elems"], p0, err, 256)
        assert rc == 0, err.value
        del kv
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    rng = np.random.default_rng(4)
    faces = [decode_face(man, rng.integers(0, cfg.vocab, B), p0 + s, hd, cfg.rope_theta) for s in range(total_steps)]
    out_host = np.zeros(2 * B, np.uint16)
    stream = torch.cuda.ExternalStream(lib.gehtp_cuda_stream())
    tok_temp = man["token_temp"]

    def reset_positions():
        for li in range(man["layers"]):
            assert lib.gehtp_cuda_state_set_count(li, p0) == 0

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn):
        """W warm-up steps, then exactly K steps between two CUDA events on the engine stream; max over ranks."""
        reset_positions()
        for s in range(W):
            step_fn(s)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        for s in range(W, W + K):
            step_fn(s)
        with torch.cuda.stream(stream):
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # first runs: plan build, weight upload and repack, graph capture
    reset_positions()
    for s in range(2):
        eng.run_io(faces[s], tok_temp, out_host)

    # ---- e2e: host face in, tokens out, through wt_exec_run_io
    def step_e2e(s):
        eng.run_io(faces[s], tok_temp, out_host)
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = lib.gehtp_cuda_launch_count()
    e2e_ms = timed(step_e2e)
    launches_e2e = lib.gehtp_cuda_launch_count() - launches0

    # ---- device-resident: faces already in HBM, tokens stay on the device
    faces_dev = [torch.from_numpy(f.view(np.int16).copy()).cuda() for f in faces]
    out_dev = torch.zeros(2 * B, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()

    def step_dev(s):
        rc = lib.gehtp_cuda_run_dev(ctypes.byref(eng.blob), faces_dev[s].data_ptr(), out_dev.data_ptr(), tok_temp, err, 256)
        assert rc == 0, err.value
    reset_positions()
    for s in range(2):          # re-capture of the graph for the device-resident binding
        step_dev(s)
    lib.gehtp_cuda_sync()
    launches0 = lib.gehtp_cuda_launch_count()
    dev_ms = timed(step_dev)
    launches_dev = lib.gehtp_cuda_launch_count() - launches0
    clocks = sampler.stop()
    assert lib.gehtp_cuda_sync() == 0

    # ---- per-kernel device times of a few steps (CUDA events around every launch unit)
    reset_positions()
    op_ms = (ctypes.c_float * eng.blob.n_ops)()
    acc = None
    attn_ms, attn_n = 0.0, 0
    prof_steps = 3
    for s in range(prof_steps + 1):
        rc = lib.gehtp_cuda_run_profiled(ctypes.byref(eng.blob), faces[s].ctypes.data, tok_temp, op_ms, eng.blob.n_ops, err, 256)
        assert rc == 0, err.value
        if s == 0:
            continue        # first eager pass after graph mode: warm-up
        cur = np.array(op_ms[:], dtype=np.float64)
        acc = cur if acc is None else acc + cur
        a_ms, a_n = ctypes.c_float(), ctypes.c_uint32()
        lib.gehtp_cuda_profiled_attn(ctypes.byref(a_ms), ctypes.byref(a_n))
        attn_ms += a_ms.value
        attn_n += a_n.value
    acc /= prof_steps
    groups = classify_units(eng.blob, acc, man, p0 + 2)
    fused_ops = int(lib.gehtp_cuda_fused_ops())
    eng.shutdown()
    attn_kernel_us = attn_ms * 1e3 / attn_n if attn_n else None
    return dict(attn_kernel_us=attn_kernel_us, e2e_ms=e2e_ms, dev_ms=dev_ms, launches=int(launches_dev), launches_e2e=int(launches_e2e), clocks=clocks,
                groups=groups, man=man, face_bytes=int(faces[0].nbytes), out_bytes=int(out_host.nbytes),
                setup_s=setup_s, fused_ops=fused_ops, blob_bytes=int(buf.size))


def run_micro(which):
    """Single-kernel timings through the device-pointer C entry points: operands
    live in HBM, `copies` rotating weight sets larger than L2 defeat cache reuse,
    launches are captured into one CUDA graph and replayed (no host overhead).
    Returns a list of dicts."""
    import torch
    import gehtp_b200
    lib = gehtp_b200.lib()
    assert lib.gehtp_cuda_set_device(0) == 0
    peak_hbm, _ = load_peaks()
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak_tf = float(peaks.get("bf16_tflops", 1590.0))
    out = []

    def timeit(fn, n=32, warm=3):
        for i in range(warm):
            fn(i)
        lib.gehtp_cuda_sync()
        torch.cuda.synchronize()
        assert lib.gehtp_cuda_capture_begin() == 0
        for i in range(n):
            fn(i + warm)
        ms = ctypes.c_float()
        assert lib.gehtp_cuda_capture_end_replay(5, ctypes.byref(ms)) == 0, lib.gehtp_cuda_last_error()
        return ms.value * 1e3 / n

    def w4(M, K, N, path, dual=False, n=32):
        nb = K * N // 2
        copies = min(max(2, int(300e6 // nb) + 1), 64)
        packed = torch.randint(0, 2 ** 31 - 1, (copies, nb // 4), dtype=torch.int32, device="cuda")
        scales = (torch.rand(copies, K // 64, N, device="cuda") * 0.015 + 0.005).half()
        a = torch.randn(M, K, device="cuda").half()
        y = torch.zeros(M, N, dtype=torch.half, device="cuda")

        def f(i):
            c, c2 = i % copies, (i + 1) % copies
            if dual:
                rc = lib.gehtp_dev_w4a16_swiglu(a.data_ptr(), packed[c].data_ptr(), scales[c].data_ptr(), packed[c2].data_ptr(),
                                                scales[c2].data_ptr(), y.data_ptr(), M, K, N)
            else:
                rc = lib.gehtp_dev_w4a16_matmul(a.data_ptr(), packed[c].data_ptr(), scales[c].data_ptr(), y.data_ptr(), M, K, N, path)
            assert rc == 0, lib.gehtp_cuda_last_error()
        us = timeit(f, n=n)
        nbytes = (nb + 2 * (K // 64) * N) * (2 if dual else 1) + 2 * M * K + 2 * M * N
        flops = 2.0 * M * K * N * (2 if dual else 1)
        return us, nbytes, flops

    if which in ("gemv", "all"):
        for M in (1, 8):
            for (K, N, dual) in ((1024, 3072, False), (2560, 6144, False), (4096, 2560, False), (2560, 9728, True),
                                 (9728, 2560, False), (2560, 151936, False)):
                us, nbytes, _ = w4(M, K, N, 1, dual)
                out.append({"kernel": "w4a16_gemv" + ("_swiglu" if dual else ""), "M": M, "K": K, "N": N, "us": us,
                            "GBps": nbytes / us / 1e3, "frac_of_measured_hbm": nbytes / us / 1e3 / peak_hbm})
    if which == "headline":   # the two kernel figures of the headline metric, for the bench line
        us, nbytes, _ = w4(1, 2560, 151936, 1, False, n=8)
        out.append({"kernel": "w4a16_gemv", "M": 1, "K": 2560, "N": 151936, "us": us, "GBps": nbytes / us / 1e3,
                    "frac_of_measured_hbm": nbytes / us / 1e3 / peak_hbm})
        us, _, flops = w4(8192, 2560, 9728, 2, n=8)
        out.append({"kernel": "w4a16_gemm_tcgen05", "M": 8192, "K": 2560, "N": 9728, "us": us, "TFLOPs": flops / us / 1e6,
                    "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which == "gemmtiles":   # the tile configurations of the tcgen05 GEMM side by side (path 3 / 4 / 5)
        for (M, K, N) in ((2048, 2560, 9728), (4096, 2560, 9728), (8192, 2560, 9728), (8192, 9728, 2560), (8192, 2560, 6144)):
            for path, name in ((3, "128x128"), (4, "256x128"), (5, "256x256")):
                us, _, flops = w4(M, K, N, path, n=8)
                out.append({"kernel": "w4a16_gemm_tcgen05", "tile": name, "M": M, "K": K, "N": N, "us": us,
                            "TFLOPs": flops / us / 1e6, "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which == "gemm1":    # one mid-size GEMM: a small case for profiler captures
        M, K, N = 2048, 2560, 9728
        us, _, flops = w4(M, K, N, 2, n=4)
        out.append({"kernel": "w4a16_gemm_tcgen05", "M": M, "K": K, "N": N, "us": us, "TFLOPs": flops / us / 1e6,
                    "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which == "gemm512":  # one prefill-size GEMM (512 tokens, q|k|v of the 0.6B shape) per tile configuration that takes it
        M, K, N = 512, 1024, 4096
        for path, name in ((3, "128x128"), (4, "256x128")):
            us, _, flops = w4(M, K, N, path, n=4)
            out.append({"kernel": "w4a16_gemm_tcgen05", "tile": name, "M": M, "K": K, "N": N, "us": us, "TFLOPs": flops / us / 1e6,
                        "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which == "lmhead":   # the vocabulary projection alone: a small case for profiler captures
        for M in (1, 8):
            us, nbytes, _ = w4(M, 2560, 151936, 1, False, n=8)
            out.append({"kernel": "w4a16_gemv", "M": M, "K": 2560, "N": 151936, "us": us, "GBps": nbytes / us / 1e3,
                        "frac_of_measured_hbm": nbytes / us / 1e3 / peak_hbm})
    if which in ("gemm", "all"):
        for (M, K, N) in ((128, 1024, 3072), (512, 1024, 4096), (512, 1024, 3072), (512, 3072, 1024), (2048, 2560, 9728),
                          (4096, 2560, 9728), (8192, 2560, 9728), (8192, 9728, 2560)):
            us, _, flops = w4(M, K, N, 2, n=8)
            out.append({"kernel": "w4a16_gemm_tcgen05", "M": M, "K": K, "N": N, "us": us, "TFLOPs": flops / us / 1e6,
                        "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which in ("attn", "attn8", "all"):
        # attn8: the batch-8 shape of the decode bench alone, a small case for profiler captures
        for (nh, kvh, n_kv) in (((256, 64, 8192),) if which == "attn8" else ((256, 64, 8192), (32, 8, 8192), (16, 8, 4096))):
            hd = 128
            ring = torch.randn(n_kv, 2, kvh * hd, device="cuda").half()
            q = torch.randn(nh, hd, device="cuda").half()
            o = torch.zeros_like(q)
            mask = torch.zeros(n_kv, device="cuda").half()

            def f(i):
                rc = lib.gehtp_attn_decode_noalloc(q.data_ptr(), ring.data_ptr(), mask.data_ptr(), o.data_ptr(), nh, kvh, hd,
                                                   n_kv, n_kv, 0.088, lib.gehtp_cuda_stream())
                assert rc == 0, lib.gehtp_cuda_last_error()
            us = timeit(f, n=8)
            nbytes = ring.numel() * 2
            out.append({"kernel": "attn_decode (split + merge)", "n_heads": nh, "kv_heads": kvh, "n_kv": n_kv, "us": us,
                        "GBps": nbytes / us / 1e3, "frac_of_measured_hbm": nbytes / us / 1e3 / peak_hbm})
    if which in ("norm", "all"):
        for rows, width in ((1, 1024), (8, 2560), (64, 2560), (512, 1024)):
            x = torch.randn(64, rows, width, device="cuda").half()
            r = torch.randn_like(x)
            gam = torch.ones(width, device="cuda").half()
            y, sm = torch.zeros_like(x[0]), torch.zeros_like(x[0])
            us = timeit(lambda i: lib.gehtp_dev_rmsnorm(x[i % 64].data_ptr(), r[i % 64].data_ptr(), gam.data_ptr(), None,
                                                        sm.data_ptr(), y.data_ptr(), rows, width))
            out.append({"kernel": "add_rmsnorm", "rows": rows, "width": width, "us": us, "GBps": 8.0 * rows * width / us / 1e3})
    if which == "gdn":
        # gated-delta-rule layer (config 5): in-projection, conv1d over 4096 channels, 32 chunks of 64 tokens, out-projection
        from gehtp_b200.runlists import build_gdn_runlist
        from gehtp_b200.wtop import Engine
        buf, man = build_gdn_runlist()
        eng = Engine(lib, buf)
        h = np.random.default_rng(1005).standard_normal((man["seq"], man["hidden"])).astype(np.float16)
        last = man["chunk_out"][-1]
        for _ in range(3):
            lib.wt_exec_state_reset()
            eng.run_io(h, last, None)
        stream = torch.cuda.ExternalStream(lib.gehtp_cuda_stream())
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        for _ in range(reps):
            eng.run_io(h, last, None)
        with torch.cuda.stream(stream):
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        op_ms = (ctypes.c_float * eng.blob.n_ops)()
        err = ctypes.create_string_buffer(256)
        assert lib.gehtp_cuda_run_profiled(ctypes.byref(eng.blob), h.ctypes.data, last, op_ms, eng.blob.n_ops, err, 256) == 0, err.value
        from gehtp_b200.wtop import OP as _OP
        by = {}
        for i in range(eng.blob.n_ops):
            by[eng.blob.ops[i].opcode] = by.get(eng.blob.ops[i].opcode, 0.0) + op_ms[i]
        H, D, seq, C = man["H"], man["D"], man["seq"], man["C"]
        out.append({"workload": "gated delta-rule layer, seq 2048, 16 heads x 128, conv 4096 channels, W4A16 in/out projections",
                    "ms": ms, "tokens_per_s": seq / ms * 1e3,
                    "conv1d_ms": by.get(_OP.CONV1D_SSM, 0.0), "conv1d_GBps": 2.0 * seq * C * 2 / max(by.get(_OP.CONV1D_SSM, 1e-9), 1e-9) / 1e6,
                    "delta_chunks_ms": by.get(_OP.DELTA_CHUNK, 0.0), "delta_qkvy_GBps": 4.0 * H * seq * D * 2 / max(by.get(_OP.DELTA_CHUNK, 1e-9), 1e-9) / 1e6,
                    "projections_ms": by.get(_OP.MATMUL_W4A16, 0.0)})
        eng.shutdown()
    if which == "prefill":
        # Qwen3-0.6B-shaped causal prefill of 512 tokens, batch 1, through the engine (graph replay after warm-up)
        from gehtp_b200.runlists import QWEN3_0P6B, build_prefill_runlist
        from gehtp_b200.wtop import Engine
        seq = 512
        cfg = QWEN3_0P6B
        buf, man = build_prefill_runlist(cfg, seq, seed=1003, quant="w4")
        eng = Engine(lib, buf)
        ids = np.random.default_rng(1003).integers(0, cfg.vocab, seq).astype(np.int32)
        tok = np.zeros(8, np.uint16)
        for _ in range(3):
            eng.run_io(ids, man["hidden_temp"], None)
        lib.gehtp_cuda_sync()
        stream = torch.cuda.ExternalStream(lib.gehtp_cuda_stream())
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        for _ in range(reps):
            eng.run_io(ids, man["hidden_temp"], None)
        with torch.cuda.stream(stream):
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        H, F, L, V = cfg.hidden, cfg.ffn, cfg.layers, cfg.vocab
        nh, kvh, hd = cfg.n_heads, cfg.kv_heads, cfg.head_dim
        lin = 2.0 * seq * (H * (nh + 2 * kvh) * hd + nh * hd * H + 3 * H * F) * L + 2.0 * seq * H * V
        att = 4.0 * nh * seq * seq * hd / 2 * L
        op_ms = (ctypes.c_float * eng.blob.n_ops)()
        perr = ctypes.create_string_buffer(256)
        by = {}
        if lib.gehtp_cuda_run_profiled(ctypes.byref(eng.blob), ids.ctypes.data, man["hidden_temp"], op_ms, eng.blob.n_ops, perr, 256) == 0:
            for i in range(eng.blob.n_ops):
                if op_ms[i] > 0:
                    k = int(eng.blob.ops[i].opcode)
                    by[k] = [by.get(k, [0, 0.0])[0] + 1, by.get(k, [0, 0.0])[1] + op_ms[i]]
        out.append({"workload": "qwen3-0.6b-shape prefill, 512 tokens, batch 1, 28 layers + lm_head", "ms": ms,
                    "units_ms_by_first_opcode": {str(k): [v[0], round(v[1], 3)] for k, v in sorted(by.items(), key=lambda kv: -kv[1][1])},
                    "tokens_per_s": seq / ms * 1e3, "TFLOPs": (lin + att) / ms / 1e9, "fused_ops": int(lib.gehtp_cuda_fused_ops()),
                    "frac_of_measured_bf16_peak": (lin + att) / ms / 1e9 / peak_tf})
        eng.shutdown()
    return out


def reference_sample(args, reps):
    """Times the reference's own executor (compiled for the host, scalar code,
    one thread as the reference runs it) on a bounded sample of the workload:
    one decoder layer at the full batch and KV context plus a 2048-column slice
    of lm_head, weights dequantised to fp16 because the reference has no
    group-64 W4A16 op. The step time of the whole model is extrapolated linearly
    (layers x layer time + vocab/2048 x head-slice time)."""
    from gehtp_b200.runlists import QWEN3_4B, build_decode_runlist, decode_face
    from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine
    from oracle.refexec import ref_lib
    import tempfile
    cfg, B, ctx = QWEN3_4B, args.batch, args.ctx
    tmp = tempfile.mkdtemp()
    lib = ref_lib(private_dir=tmp)
    if lib is None:
        return None
    vs = 2048
    buf, man = build_decode_runlist(cfg, B, ctx, seed=1004, quant="f16", n_layers=1, vocab=vs)
    kv_elems = B * cfg.kv_heads * cfg.head_dim
    # fill the KV ring through the reference's own append op
    fill = BlobBuilder()
    fill.add_states([kv_elems * 4 * ctx])
    rng = np.random.default_rng(1)
    kslot = fill.add_slot(rng.standard_normal(kv_elems).astype(np.float16))
    n_fill = ctx - 1 - reps
    for _ in range(n_fill):
        fill.add_op(OP.KV_APPEND, [S(kslot), S(kslot), ST(0), KV_POS_AUTO])
    feng = Engine(lib, fill.build())
    feng.run()
    eng = Engine(lib, buf)
    n_ops = eng.blob.n_ops
    op_us = (ctypes.c_int64 * n_ops)()
    err = ctypes.create_string_buffer(256)
    from gehtp_b200.wtop import OP as _OP
    head_ops = [i for i in range(n_ops) if eng.blob.ops[i].opcode == _OP.MATMUL_F16 and eng.blob.ops[i].args[5] == vs]
    times = []
    for r in range(reps):
        face = decode_face(man, rng.integers(0, vs, B), n_fill + r, cfg.head_dim, cfg.rope_theta)
        t0 = time.time()
        rc = lib.wt_exec_run_io(ctypes.byref(eng.blob), face.ctypes.data, None, man["token_temp"], None, op_us, err, 256)
        wall = time.time() - t0
        assert rc == 0, err.value
        us = np.array(op_us[:], dtype=np.float64)
        head = us[head_ops].sum() if head_ops else 0.0
        layer = us.sum() - head
        full_s = (layer * args.layers + head * (cfg.vocab / vs)) * 1e-6
        times.append((wall, full_s))
    eng.shutdown()
    wall = float(np.mean([t[0] for t in times]))
    full = float(np.mean([t[1] for t in times]))
    return dict(tok_s=B / full, step_s_extrapolated=full, sample_wall_s=wall, reps=reps,
                sample="1 of %d layers at batch %d, KV ctx %d, plus a %d-column slice of lm_head; fp16 weights; "
                       "step time extrapolated linearly; %d repetition(s) of %.1f s" % (args.layers, B, ctx, vs, reps, wall))


def init_tp(lib, rank, world):
    """NCCL communicator of the engine: rank 0 makes the id, torch.distributed carries it."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        dist.init_process_group("nccl")
    idb = (ctypes.c_uint8 * 128)()
    if rank == 0:
        assert lib.gehtp_cuda_tp_unique_id(idb, 128) == 0
    t = torch.tensor(list(idb), dtype=torch.uint8, device="cuda")
    dist.broadcast(t, 0)
    raw = bytes(t.cpu().tolist())
    cbuf = (ctypes.c_uint8 * 128).from_buffer_copy(raw)
    assert lib.gehtp_cuda_tp_init(rank, world, cbuf, 128) == 0, lib.gehtp_cuda_last_error()
    if os.environ.get("GEHTP_TP_P2P", "1") != "0":
        # mailboxes for the one-kernel all-reduce over peer memory: gather the IPC handles in rank order
        hb = (ctypes.c_uint8 * 64)()
        ok = lib.gehtp_cuda_tp_p2p_export(hb, 64) == 0
        mine = torch.tensor(list(hb), dtype=torch.uint8, device="cuda")
        allh = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        raw = b"".join(bytes(h.cpu().tolist()) for h in allh)
        hbuf = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(raw)
        ok = ok and lib.gehtp_cuda_tp_p2p_import(hbuf, 64, world) == 0
        # every rank uses the peer-memory kernels or none does
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if not ok:
                print("[tp] rank %d: peer-memory mailboxes unavailable (%s); all ranks use NCCL all-reduces"
                      % (rank, lib.gehtp_cuda_last_error().decode(errors="replace")), file=sys.stderr)
            lib.gehtp_cuda_tp_p2p_disable()
        dist.barrier()


def main():
    args = parse_args()
    # stdout carries the JSON line(s) only: libraries that print banners there (NCCL's
    # version line) are pointed at stderr while the run lasts.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        lines = run_main(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    for ln in lines:
        print(ln)
    sys.stdout.flush()


def run_main(args):
    out = []
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    B = args.batch
    config = {"workload": "Qwen3-4B-shaped decoder decode step, W4A16 group-64, batch %d, KV context %d, %d layers + lm_head 151936"
                          % (B, args.ctx, args.layers),
              "batch": B, "kv_context": args.ctx, "layers": args.layers,
              "parallelism": "tp%d" % world if world > 1 else
                             ("single GPU" if args.shard_of <= 1 else "rank 0's shard of tp%d, no all-reduce (profiling aid)" % args.shard_of),
              "l2": "inputs larger than L2: every step streams the weights and the KV rings (GBs) once"}

    if args.micro:
        if rank == 0:
            for row in run_micro(args.micro):
                out.append(json.dumps(row))
        return out

    if args.impl == "reference":
        if rank != 0:
            return out
        probe = reference_sample(args, 1)
        if probe is None:
            out.append(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libgehtp_ref.so was not built"}))
            return out
        reps = int(max(1, min(args.steps, 150.0 // max(probe["sample_wall_s"], 1e-3)))) - 1
        res = reference_sample(args, reps) if reps >= 1 else probe
        line = {"impl": "reference", "metric": METRIC, "value": res["tok_s"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["step_s_extrapolated"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": config, "gpu_launches": 0,
                "cpu_baseline": {"value": res["tok_s"], "unit": UNIT, "cores": 1, "kind": "reference", "sample": res["sample"]},
                "e2e": {"value": res["tok_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        out.append(json.dumps(line))
        return out

    r = run_ours(args, rank, world)
    if rank != 0:
        return out
    K = args.steps
    peak, peak_src = load_peaks()
    value = B * K / (r["dev_ms"] * 1e-3)
    e2e = B * K / (r["e2e_ms"] * 1e-3)
    groups = r["groups"]
    kernels = {}
    for name, (n, ms, nb) in groups.items():
        kernels[name] = {"launches_per_step": n, "ms_per_step": ms, "avg_us": ms * 1e3 / max(n, 1),
                         "achieved_gbs": (nb / (ms * 1e-3) / 1e9) if ms > 0 and nb else None}
    dom = max((k for k in groups if groups[k][2] > 0), key=lambda k: groups[k][1])
    dn, dms, dbytes = groups[dom]
    achieved = dbytes / (dms * 1e-3) / 1e9
    dom_kernel, dom_us = dom, dms * 1e3 / dn
    if dom == "attn_decode" and r.get("attn_kernel_us"):
        # the unit holds three kernels (q|k|v projection with rotary/append, attention, merge); the roofline is the attention kernel's,
        # timed by its own event pair inside the same profiled steps
        dom_kernel, dom_us = "attn_decode_tma_kernel", r["attn_kernel_us"]
        achieved = (dbytes / dn) / (dom_us * 1e-6) / 1e9
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": r["dev_ms"] / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": config, "clocks": r["clocks"],
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": r["e2e_ms"] / K, "h2d_bytes_per_step": r["face_bytes"],
                    "d2h_bytes_per_step": r["out_bytes"]},
            "gpu_launches": r["launches"],
            "roofline": {"bound": "hbm", "kernel": dom_kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC.get((dom, B, args.ctx, world)), "peak_source": peak_src,
                         "bytes_per_launch": dbytes / dn, "avg_launch_us": dom_us, "launch_unit_us": dms * 1e3 / dn},
            "kernels": kernels, "fused_ops": r["fused_ops"], "setup_s": r["setup_s"]}
    if world == 1 and args.shard_of <= 1:
        # the kernel halves of the headline metric: streaming GEMV (vocabulary projection, M = 1) and prefill GEMM
        try:
            hv, hm = run_micro("headline")
            line["w4a16_gemv"] = {"shape": [hv["M"], hv["K"], hv["N"]], "GBps": hv["GBps"], "frac_of_measured_hbm": hv["frac_of_measured_hbm"]}
            line["w4a16_gemm"] = {"shape": [hm["M"], hm["K"], hm["N"]], "TFLOPs": hm["TFLOPs"],
                                  "frac_of_measured_bf16_peak": hm["frac_of_measured_bf16_peak"]}
        except Exception as ex:      # never lose the bench line over the extra figures
            line["w4a16_kernels_error"] = str(ex)[:200]
    if world == 1 and not args.no_cpu_baseline:
        cb = reference_sample(args, 1)
        if cb:
            line["cpu_baseline"] = {"value": cb["tok_s"], "unit": UNIT, "cores": 1, "kind": "reference", "sample": cb["sample"]}
    out.append(json.dumps(line))
    return out


if __name__ == "__main__":
    main()
