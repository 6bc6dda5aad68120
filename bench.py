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
    ap.add_argument("--config", type=int, default=None, choices=[1, 2, 3, 5],
                    help="one line for another baseline configuration (1: single W4A16 matmul, 2: RMSNorm + decode attention, "
                         "3: 0.6B-shape prefill, 5: gated delta-rule layer) with its roofline and the reference's CPU time")
    ap.add_argument("--micro", default=None, choices=["gemv", "lmhead", "gemm", "swiglu", "swiglu512", "gemm1", "gemm512", "f16gemm", "headline", "gemmtiles", "attn", "attn8", "norm", "prefill", "gdn", "all"],
                    help="time single kernels (device-resident operands, graph replay) instead of the decode step")
    return ap.parse_args()


# roofline.traffic = dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel. It is not
# measured by this program (no profiler runs inside a bench): it is read from the ncu summary under profiles/
# that covers the workload, whose "bench-traffic" line records the byte count and the sha256 of the kernel's
# source file at capture time. A summary taken from another version of the kernel is not quoted.
TRAFFIC_PROFILES = {("attn_decode", 8, 8192, 1): "profiles/attn_decode_tma_b8_ctx8192.md"}


def profile_traffic(key):
    """(bytes per launch or None, provenance dict) for a workload key (kernel group, batch, context, GPUs)."""
    import hashlib
    import re
    rel = TRAFFIC_PROFILES.get(key)
    if not rel or not os.path.exists(os.path.join(ROOT, rel)):
        return None, {"traffic_source": None}
    m = re.search(r"bench-traffic:\s*bytes_per_launch=(\d+)\s+source=(\S+)\s+sha256=([0-9a-f]{64})", open(os.path.join(ROOT, rel)).read())
    if not m:
        return None, {"traffic_source": rel, "traffic_note": "summary has no bench-traffic line"}
    src = os.path.join(ROOT, m.group(2))
    now = hashlib.sha256(open(src, "rb").read()).hexdigest() if os.path.exists(src) else ""
    if now != m.group(3):
        return None, {"traffic_source": rel, "traffic_note": "summary was captured from another version of %s" % m.group(2)}
    return int(m.group(1)), {"traffic_source": rel, "traffic_kernel_sha256": now[:16]}


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
    check = None
    for li in range(man["layers"]):
        kv = torch.randn(ring_elems, device="cuda", dtype=torch.float16)
        rc = lib.gehtp_cuda_state_load(ctypes.byref(eng.blob), li, kv.data_ptr(), ring_elems * 2, 1, man["kv_elems"], p0, err, 256)
        assert rc == 0, err.value
        if li == 0 and world == 1 and args.shard_of <= 1 and not args.no_cpu_baseline:
            # kept for the self-check: the reference runs layer 0 of step 0 on the same ring
            check = {"ring": kv.cpu().numpy().view(np.float16).reshape(ctx, 2 * man["kv_elems"]).copy(), "p0": p0}
        del kv
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    rng = np.random.default_rng(4)
    faces = [decode_face(man, rng.integers(0, cfg.vocab, B), p0 + s, hd, cfg.rope_theta) for s in range(total_steps)]
    # the step's result: B int32 tokens; a tensor-parallel shard adds the B fp16 row maxima its argmax goes with
    out_units = (3 if shard > 1 else 2) * B
    out_host = np.zeros(out_units, np.uint16)
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
        if s == 0 and check is not None:
            check["face"] = faces[0].copy()
            check["layer_out"] = eng.temp(man["layer_out"][0]).copy()

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
    out_dev = torch.zeros(out_units, dtype=torch.int16, device="cuda")
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
                groups=groups, man=man, face_bytes=int(faces[0].nbytes), out_bytes=int(out_host.nbytes), check=check,
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
    if which in ("gemm", "swiglu", "all"):   # gate | up of a gated FFN as one tcgen05 launch (product in the epilogue) beside one of its two GEMMs
        for (M, K, N) in ((64, 2560, 9728), (512, 1024, 3072), (2048, 2560, 9728)):
            # graphs of 4 launches: in a longer chain of this one kernel the early CTAs of the next launches (released at
            # kernel entry) hold SMs while they wait for their predecessors and the figure stops describing a launch
            us, _, flops = w4(M, K, N, 0, dual=True, n=4)
            us1, _, _ = w4(M, K, N, 2, n=4)
            out.append({"kernel": "w4a16_gemm_tcgen05_swiglu", "M": M, "K": K, "N": N, "us": us, "TFLOPs": flops / us / 1e6,
                        "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf, "one_projection_alone_us": us1})
    if which == "swiglu512":   # the gate | up launch of the 0.6B-shape prefill alone: a small case for profiler captures
        M, K, N = 512, 1024, 3072
        us, _, flops = w4(M, K, N, 0, dual=True, n=4)
        out.append({"kernel": "w4a16_gemm_tcgen05_swiglu", "M": M, "K": K, "N": N, "us": us, "TFLOPs": flops / us / 1e6,
                    "frac_of_measured_bf16_peak": flops / us / 1e6 / peak_tf})
    if which in ("f16gemm", "all"):   # OP_MATMUL_F16 with weights stored [N, K]: tcgen05 GEMM (M >= 128) and streaming GEMV (M < 32)
        for (M, K, N) in ((1, 1024, 151936), (8, 2560, 9728), (128, 1024, 3072), (512, 1024, 4096), (2048, 2560, 9728), (8192, 2560, 9728)):
            copies = min(max(2, int(300e6 // (2 * K * N)) + 1), 16)
            w = (torch.randn(copies, N, K, device="cuda") * 0.05).half()
            a = torch.randn(M, K, device="cuda").half()
            y = torch.zeros(M, N, dtype=torch.half, device="cuda")

            def f(i):
                assert lib.gehtp_dev_matmul_f16_nk(a.data_ptr(), w[i % copies].data_ptr(), y.data_ptr(), M, K, N) == 0, lib.gehtp_cuda_last_error()
            us = timeit(f, n=8)
            flops, nbytes = 2.0 * M * K * N, 2.0 * (K * N + M * K + M * N)
            row = {"kernel": "f16_gemm_sm100" if M >= 128 else "f16_gemv_nk", "M": M, "K": K, "N": N, "us": us}
            if M >= 128:
                row.update(TFLOPs=flops / us / 1e6, frac_of_measured_bf16_peak=flops / us / 1e6 / peak_tf)
            else:
                row.update(GBps=nbytes / us / 1e3, frac_of_measured_hbm=nbytes / us / 1e3 / peak_hbm)
            out.append(row)
            del w
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


def _time_graph(lib, torch, fn, n=16, warm=3):
    """Mean microseconds of one call of fn(i), n calls captured into a CUDA graph and replayed."""
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


def _ref_op_us(ref, buf, inp, reps=1):
    """Per-op microseconds of the reference executor on one blob (its own op_us clock), last of `reps` runs."""
    from gehtp_b200.wtop import Engine
    eng = Engine(ref, buf)
    op_us = (ctypes.c_int64 * eng.blob.n_ops)()
    err = ctypes.create_string_buffer(256)
    keep = np.ascontiguousarray(inp) if inp is not None else None
    for _ in range(reps):
        rc = ref.wt_exec_run_io(ctypes.byref(eng.blob), keep.ctypes.data if keep is not None else None, None, 0, None, op_us, err, 256)
        assert rc == 0, err.value
    us = np.array(op_us[:], dtype=np.float64)
    ops = [(int(eng.blob.ops[i].opcode), list(eng.blob.ops[i].args)) for i in range(eng.blob.n_ops)]
    return us, ops, eng


def run_config(args):
    """Baseline configurations 1, 2, 3 and 5: the same contract as the decode line (value = device-resident
    figure by graph replay or CUDA events, e2e = through the C ABI with host buffers, roofline against the
    measured peaks, cpu_baseline = the reference's executor on this box's host cores, one thread, on a
    bounded sample that `sample` describes)."""
    import tempfile
    import torch
    import gehtp_b200
    from gehtp_b200.runlists import QWEN3_0P6B, build_gdn_runlist, build_prefill_runlist, dequant_f16, rand_w4
    from gehtp_b200.wtop import KV_POS_AUTO, OP, S, ST, BlobBuilder, Engine
    from oracle.refexec import orc_lib, ptr, ref_lib
    lib = gehtp_b200.lib()
    assert lib.gehtp_cuda_set_device(0) == 0, "no CUDA device"
    peak_hbm, peak_src = load_peaks()
    pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak_tf = float(pk.get("bf16_tflops", 1590.0))
    ref = None if args.no_cpu_baseline else ref_lib(private_dir=tempfile.mkdtemp())
    sampler = ClockSampler(0)
    sampler.start()
    stream = torch.cuda.ExternalStream(lib.gehtp_cuda_stream())

    def events(fn, reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        lib.gehtp_cuda_sync()
        with torch.cuda.stream(stream):
            e0.record()
        for i in range(reps):
            fn(i)
        with torch.cuda.stream(stream):
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    line = {"n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic"}
    c = args.config
    if c == 1:
        # ---- single W4A16 matmul, M128 K1024 N3072 (GEMM) and the same weights at M = 1 (GEMV)
        M, K, N = 128, 1024, 3072
        rng = np.random.default_rng(1001)
        a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
        nib, sc = rand_w4(rng, K, N)
        slot = np.concatenate([nib.reshape(-1), sc.view(np.uint8).reshape(-1)])
        copies = 128            # 208 MB of weights in rotation: larger than L2
        packed = torch.randint(0, 2 ** 31 - 1, (copies, K * N // 8), dtype=torch.int32, device="cuda")
        scales = (torch.rand(copies, K // 64, N, device="cuda") * 0.015 + 0.005).half()
        da = torch.from_numpy(a.view(np.int16)).cuda()
        dy = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        res = {}
        for name, m, path in (("gemm", M, 2), ("gemv", 1, 1)):
            us = _time_graph(lib, torch, lambda i: lib.gehtp_dev_w4a16_matmul(da.data_ptr(), packed[i % copies].data_ptr(), scales[i % copies].data_ptr(),
                                                                              dy.data_ptr(), m, K, N, path), n=32)
            res[name] = us
        got = np.zeros((M, N), np.float16)
        e2e_ms = events(lambda i: lib.gehtp_w4a16_matmul(ptr(a), ptr(slot), ptr(got), M, K, N, 0), max(args.steps, 5))
        flops, gemm_bytes, gemv_bytes = 2.0 * M * K * N, w4_bytes(M, K, N), w4_bytes(1, K, N)
        line.update(metric="w4a16_matmul_m128_k1024_n3072_tflops", value=flops / res["gemm"] / 1e6, unit="TFLOP/s",
                    ms_per_step=res["gemm"] * 1e-3, gpu_launches=32 * 5,
                    config={"workload": "config 1: one W4A16 group-64 matmul, M128 K1024 N3072; weights rotate through %d copies (208 MB > L2)" % copies},
                    e2e={"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": int(a.nbytes + slot.nbytes), "d2h_bytes_per_step": int(got.nbytes)},
                    roofline={"bound": "tensor", "kernel": "w4a16_gemm_sm100_kernel", "achieved": flops / res["gemm"] / 1e6, "peak": peak_tf,
                              "unit": "TFLOP/s", "frac": flops / res["gemm"] / 1e6 / peak_tf, "traffic": None, "peak_source": peak_src,
                              "note": "0.8 GFLOP: the ideal math time is 0.5 us, the launch is latency bound; HBM floor %d bytes = %.2f us" % (gemm_bytes, gemm_bytes / peak_hbm / 1e3)},
                    gemv={"M": 1, "us": res["gemv"], "GBps": gemv_bytes / res["gemv"] / 1e3, "frac_of_measured_hbm": gemv_bytes / res["gemv"] / 1e3 / peak_hbm})
        if ref is not None:
            orc = orc_lib()
            want = np.zeros((M, N), np.float16)
            t0 = time.time()
            orc.orc_w4a16_matmul(ptr(a), ptr(slot), ptr(want), M, K, N)
            t_rest = time.time() - t0
            b = BlobBuilder()
            sa, sw = b.add_slot(a), b.add_slot(dequant_f16(nib, sc))
            b.add_op(OP.MATMUL_F16, [S(sa), S(sw), 1, M, K, N, 0])
            us, _, reng = _ref_op_us(ref, b.build(), None)
            err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
            line["checked"] = bool(err <= 1e-2 * np.abs(want.astype(np.float64)).max())
            line["cpu_baseline"] = {"value": flops / (us.sum() * 1e-6) / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "reference",
                                    "sample": "the whole matmul once: reference OP_MATMUL_F16 on the dequantised fp16 weights %.2f s; "
                                              "this repo's C restatement of the group-64 op %.2f s" % (us.sum() * 1e-6, t_rest)}
    elif c == 2:
        # ---- RMSNorm [1,1024] + decode attention 16 q / 8 kv heads of 128 over 4096 positions
        nh, kvh, hd, n_kv, W = 16, 8, 128, 4096, 1024
        rng = np.random.default_rng(1002)
        x = rng.standard_normal((1, W), dtype=np.float32).astype(np.float16)
        gam = rng.normal(1, 0.1, W).astype(np.float16)
        q = rng.standard_normal((nh, hd), dtype=np.float32).astype(np.float16)
        ring = rng.standard_normal((n_kv, 2, kvh * hd), dtype=np.float32).astype(np.float16)
        mask = np.zeros(n_kv, np.float16)
        scale = float(np.float16(1 / np.sqrt(hd)))
        copies = 12            # 200 MB of rings in rotation
        rings = torch.randn(copies, n_kv * 2 * kvh * hd, device="cuda").half()
        dq, dm = torch.from_numpy(q.view(np.int16)).cuda(), torch.zeros(n_kv, dtype=torch.int16, device="cuda")
        do = torch.zeros(nh * hd, dtype=torch.int16, device="cuda")
        dx, dg = torch.from_numpy(x.view(np.int16)).cuda(), torch.from_numpy(gam.view(np.int16)).cuda()
        dyn = torch.zeros(W, dtype=torch.int16, device="cuda")
        st = lib.gehtp_cuda_stream()
        us_attn = _time_graph(lib, torch, lambda i: lib.gehtp_attn_decode_noalloc(dq.data_ptr(), rings[i % copies].data_ptr(), dm.data_ptr(), do.data_ptr(),
                                                                                   nh, kvh, hd, n_kv, n_kv, scale, st), n=24)
        us_norm = _time_graph(lib, torch, lambda i: lib.gehtp_dev_rmsnorm(dx.data_ptr(), None, dg.data_ptr(), None, None, dyn.data_ptr(), 1, W), n=24)
        got = np.zeros((nh, hd), np.float16)
        yn = np.zeros((1, W), np.float16)

        def e2e_step(i):
            assert lib.gehtp_rmsnorm(ptr(x), ptr(gam), None, ptr(yn), 1, W) == 0
            assert lib.gehtp_attn_decode(ptr(q), ptr(ring), ptr(mask), ptr(got), nh, kvh, hd, n_kv, n_kv, scale) == 0
        e2e_ms = events(e2e_step, max(args.steps, 5))
        kv_bytes = ring.nbytes
        line.update(metric="decode_attention_16q8kv_ctx4096_GBps", value=kv_bytes / us_attn / 1e3, unit="GB/s", ms_per_step=(us_attn + us_norm) * 1e-3,
                    gpu_launches=24 * 5 * 2,
                    config={"workload": "config 2: RMSNorm [1,1024] + decode GQA attention, 16 q / 8 kv heads of 128, KV context 4096; %d rings in rotation (200 MB > L2)" % copies},
                    e2e={"value": kv_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": int(ring.nbytes + q.nbytes + mask.nbytes + x.nbytes + gam.nbytes), "d2h_bytes_per_step": int(got.nbytes + yn.nbytes)},
                    roofline={"bound": "hbm", "kernel": "attn_decode (split-KV + merge)", "achieved": kv_bytes / us_attn / 1e3, "peak": peak_hbm, "unit": "GB/s",
                              "frac": kv_bytes / us_attn / 1e3 / peak_hbm, "traffic": None, "peak_source": peak_src, "bytes_per_launch": kv_bytes, "avg_launch_us": us_attn},
                    rmsnorm={"rows": 1, "width": W, "us": us_norm, "bytes": 6 * W, "note": "6 KB: latency of one launch, not a bandwidth figure"})
        if ref is not None:
            # the reference's op chain on its own KV ring: appends untimed, then gather / scores / scale / mask / softmax / PV timed
            b = BlobBuilder()
            b.add_states([kvh * hd * 4 * n_kv])
            face = b.add_ext_in(2 * kvh * hd * 2)
            b.add_op(OP.SLICE, [S(face), 1, kvh * hd, 1, 0, 0, 0, kvh * hd, 0, 0, 1, 1, 1, 2 * kvh * hd, 1, 1])
            b.add_op(OP.SLICE, [S(face), 2, kvh * hd, 1, kvh * hd, 0, 0, 2 * kvh * hd, 0, 0, 1, 1, 1, 2 * kvh * hd, 1, 1])
            b.add_op(OP.KV_APPEND, [1, 2, ST(0), KV_POS_AUTO])
            feng = Engine(ref, b.build())
            for p in range(n_kv):
                feng.run_io(ring[p].reshape(-1), 0)
            b = BlobBuilder()
            b.add_states([kvh * hd * 4 * n_kv])
            sx, sg, sz, sq = b.add_slot(x), b.add_slot(gam), b.add_slot(np.zeros(W, np.float16)), b.add_slot(q)
            ssc, smk = b.add_slot(np.array([scale], np.float16)), b.add_slot(mask)
            b.add_op(OP.RMSNORM2, [S(sx), S(sg), S(sz), 1, W])
            b.add_op(OP.KV_GATHER, [ST(0), 2, 0, n_kv, nh, kvh, hd])
            b.add_op(OP.KV_GATHER, [ST(0), 0, 3, n_kv, nh, kvh, hd])
            b.add_op(OP.MATMUL_F16, [S(sq), 2, 4, 1, hd, n_kv, 4 | nh << 16])
            b.add_op(OP.BROADCAST, [S(ssc), 5, nh * n_kv, 1, 1, 1, 1, 1, 1, 1, 1, nh * n_kv])
            b.add_op(OP.BINARY, [4, 5, 6, nh * n_kv, 2])
            b.add_op(OP.BROADCAST, [S(smk), 7, nh * n_kv, n_kv, 1, 1, 1, n_kv, 1, 1, nh, n_kv])
            b.add_op(OP.ADD, [6, 7, 8, nh * n_kv])
            b.add_op(OP.SOFTMAX, [8, 9, nh, n_kv])
            b.add_op(OP.MATMUL_F16, [9, 3, 10, 1, n_kv, hd, 4 | nh << 16])
            us, _, reng = _ref_op_us(ref, b.build(), None, reps=3)
            want = reng.temp(10).astype(np.float64).reshape(nh, hd)
            err = np.abs(got.astype(np.float64) - want).max()
            line["checked"] = bool(err <= 1e-2 * np.abs(want).max())
            line["cpu_baseline"] = {"value": kv_bytes / (us[1:].sum() * 1e-6) / 1e9, "unit": "GB/s", "cores": 1, "kind": "reference",
                                    "sample": "the whole op chain (KV_GATHER x2, scores, scale, mask, SOFTMAX, PV) %.1f ms and RMSNORM2 %.1f us, "
                                              "third of 3 runs; the 4096 appends are set-up" % (us[1:].sum() * 1e-3, us[0])}
    elif c == 3:
        # ---- Qwen3-0.6B-shaped prefill, 512 tokens, 28 layers + lm_head
        cfg, seq = QWEN3_0P6B, 512
        buf, man = build_prefill_runlist(cfg, seq, seed=1003, quant="w4")
        eng = Engine(lib, buf)
        ids = np.random.default_rng(1003).integers(0, cfg.vocab, seq).astype(np.int32)
        out_h = np.zeros(seq * cfg.hidden, np.float16)
        for _ in range(max(args.warmup, 3)):
            eng.run_io(ids, man["hidden_temp"], out_h)
        dids = torch.from_numpy(ids).cuda()
        dout = torch.zeros(seq * cfg.hidden, dtype=torch.int16, device="cuda")
        err = ctypes.create_string_buffer(256)
        l0 = lib.gehtp_cuda_launch_count()
        e2e_ms = events(lambda i: eng.run_io(ids, man["hidden_temp"], out_h), max(args.steps, 5))

        def dev_step(i):
            assert lib.gehtp_cuda_run_dev(ctypes.byref(eng.blob), dids.data_ptr(), dout.data_ptr(), man["hidden_temp"], err, 256) == 0, err.value
        for i in range(3):
            dev_step(i)
        l0 = lib.gehtp_cuda_launch_count()
        ms = events(dev_step, max(args.steps, 5))
        launches = int(lib.gehtp_cuda_launch_count() - l0)
        H, F, L, V = cfg.hidden, cfg.ffn, cfg.layers, cfg.vocab
        nh, kvh, hd = cfg.n_heads, cfg.kv_heads, cfg.head_dim
        lin = 2.0 * seq * (H * (nh + 2 * kvh) * hd + nh * hd * H + 3 * H * F) * L + 2.0 * seq * H * V
        att = 4.0 * nh * seq * seq * hd / 2 * L
        tf = (lin + att) / ms / 1e9
        line.update(metric="qwen3_0p6b_shape_prefill_512_tokens_per_s", value=seq / ms * 1e3, unit="tok/s", ms_per_step=ms, gpu_launches=launches,
                    config={"workload": "config 3: Qwen3-0.6B-shaped prefill, 512 tokens, batch 1, 28 layers + lm_head 151936, W4A16 group-64; 298 MB of weights per pass (> L2)"},
                    e2e={"value": seq / e2e_ms * 1e3, "unit": "tok/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(ids.nbytes), "d2h_bytes_per_step": int(out_h.nbytes)},
                    roofline={"bound": "tensor", "kernel": "whole pass (w4a16_gemm_sm100_kernel dominates)", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s",
                              "frac": tf / peak_tf, "traffic": None, "peak_source": peak_src, "flops_per_step": lin + att})
        eng.shutdown()
        if ref is not None:
            # one layer over the 128-token causal prefix + a 2048-column cut of lm_head on the reference; every op scaled by its own work ratio
            cut, vs = 128, 2048
            work = {}
            for s_ in (cut, seq):
                bb, mm = build_prefill_runlist(cfg, s_, seed=1003, quant="f16", n_layers=1, vocab=vs)
                if s_ == cut:
                    us, ops, reng = _ref_op_us(ref, bb, ids[:cut])
                work[s_] = [_op_work(o, a_) for o, a_ in (ops if s_ == cut else [(int(x_[0]), x_[1]) for x_ in _blob_ops(lib, bb)])]
            head_i = [i for i, (o, a_) in enumerate(ops) if o == OP.MATMUL_F16 and a_[5] == vs]
            tot = 0.0
            for i in range(len(ops)):
                ratio = work[seq][i] / work[cut][i] if work[seq][i] and work[cut][i] else seq / cut
                t = us[i] * ratio
                tot += t * (V / vs if i in head_i else L) if (i in head_i or i > 2) else t
            line["cpu_baseline"] = {"value": seq / (tot * 1e-6), "unit": "tok/s", "cores": 1, "kind": "reference",
                                    "sample": "one of 28 layers over the first 128 of 512 tokens plus a 2048-column cut of lm_head, fp16 weights (%.1f s); "
                                              "each op scaled by its work ratio to 512 tokens, x28 layers, x74 for the vocabulary: extrapolated" % (us.sum() * 1e-6)}
    elif c == 5:
        # ---- gated delta-rule layer: in-projection, conv1d 4096 channels, 32 chunks of 64 tokens x 16 heads, out-projection
        buf, man = build_gdn_runlist()
        eng = Engine(lib, buf)
        h = np.random.default_rng(1005).standard_normal((man["seq"], man["hidden"]), dtype=np.float32).astype(np.float16)
        last = man["chunk_out"][-1]
        out_h = np.zeros(man["chunk"] * man["hidden"], np.float16)
        for _ in range(max(args.warmup, 3)):
            lib.wt_exec_state_reset()
            eng.run_io(h, last, out_h)
        l0 = lib.gehtp_cuda_launch_count()
        reps = max(args.steps, 5)
        e2e_ms = events(lambda i: eng.run_io(h, last, out_h), reps)
        launches = int(lib.gehtp_cuda_launch_count() - l0) // reps
        dh = torch.from_numpy(h.view(np.int16)).cuda()
        dout = torch.zeros(out_h.size, dtype=torch.int16, device="cuda")
        err = ctypes.create_string_buffer(256)

        def dev_step(i):
            assert lib.gehtp_cuda_run_dev(ctypes.byref(eng.blob), dh.data_ptr(), dout.data_ptr(), last, err, 256) == 0, err.value
        for i in range(3):
            dev_step(i)
        ms = events(dev_step, reps)
        op_ms = (ctypes.c_float * eng.blob.n_ops)()
        assert lib.gehtp_cuda_run_profiled(ctypes.byref(eng.blob), h.ctypes.data, last, op_ms, eng.blob.n_ops, err, 256) == 0, err.value
        by = {}
        for i in range(eng.blob.n_ops):
            by[eng.blob.ops[i].opcode] = by.get(eng.blob.ops[i].opcode, 0.0) + op_ms[i]
        H, D, seq, C = man["H"], man["D"], man["seq"], man["C"]
        conv_bytes, qkvy_bytes = 2.0 * seq * C * 2, 4.0 * H * seq * D * 2
        conv_ms, delta_ms = by.get(OP.CONV1D_SSM, 0.0), by.get(OP.DELTA_CHUNK, 0.0)
        line.update(metric="gated_delta_layer_seq2048_tokens_per_s", value=seq / ms * 1e3, unit="tok/s", ms_per_step=ms, gpu_launches=launches,
                    config={"workload": "config 5: gated delta-rule layer, 2048 tokens, conv1d k=4 over 4096 channels, 16 heads of 128, 32 chunks of 64, W4A16 in/out projections from hidden 1024"},
                    e2e={"value": seq / e2e_ms * 1e3, "unit": "tok/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(h.nbytes), "d2h_bytes_per_step": int(out_h.nbytes)},
                    roofline={"bound": "hbm", "kernel": "delta_chunk_mma_kernel (32 sequential launches)", "achieved": qkvy_bytes / max(delta_ms, 1e-9) / 1e6, "peak": peak_hbm,
                              "unit": "GB/s", "frac": qkvy_bytes / max(delta_ms, 1e-9) / 1e6 / peak_hbm, "traffic": None, "peak_source": peak_src,
                              "note": "q/k/v/y traffic of the 32 chunks against HBM; the chunks are sequential per head (the state carries) and latency bound: "
                                      "seven dependent small products per chunk, 10.5 MFLOP per head and chunk on mma.sync"},
                    kernels={"conv1d_ssm": {"ms": conv_ms, "GBps": conv_bytes / max(conv_ms, 1e-9) / 1e6, "frac_of_measured_hbm": conv_bytes / max(conv_ms, 1e-9) / 1e6 / peak_hbm},
                             "delta_chunk_x32": {"ms": delta_ms}, "w4a16_projections": {"ms": by.get(OP.MATMUL_W4A16, 0.0)}})
        eng.shutdown()
        if ref is not None:
            # the reference's conv op over the whole sequence and its delta-chunk op over all 32 chunks (no projections)
            rng = np.random.default_rng(1005)
            b = BlobBuilder()
            b.add_states([H * D * D * 4])
            sx = b.add_slot(rng.standard_normal((seq, C), dtype=np.float32).astype(np.float16))
            sw = b.add_slot(rng.normal(0, 0.5, (4, C)).astype(np.float16))
            b.add_op(OP.CONV1D_SSM, [S(sx), sw, 1, seq, C, 4])
            ck = man["chunk"]
            kk = rng.standard_normal((H, ck, D), dtype=np.float32)
            kk = (kk / np.linalg.norm(kk, axis=-1, keepdims=True)).astype(np.float16)
            sl = [b.add_slot(kk), b.add_slot(rng.standard_normal((H, ck, D), dtype=np.float32).astype(np.float16)),
                  b.add_slot(rng.standard_normal((H, ck, D), dtype=np.float32).astype(np.float16)),
                  b.add_slot((1 / (1 + np.exp(-rng.standard_normal((H, ck))))).astype(np.float16)),
                  b.add_slot(np.log(1 / (1 + np.exp(-rng.standard_normal((H, ck))))).astype(np.float16))]
            for ci in range(seq // ck):
                b.add_op(OP.DELTA_CHUNK, [S(s_) for s_ in sl] + [2, ST(0), ck, ck, H, D, 0])
            us, _, reng = _ref_op_us(ref, b.build(), None)
            line["cpu_baseline"] = {"value": seq / (us.sum() * 1e-6), "unit": "tok/s", "cores": 1, "kind": "reference",
                                    "sample": "OP_CONV1D_SSM over 2048 x 4096 (%.2f s) and OP_DELTA_CHUNK over 32 chunks of 64 tokens x 16 heads (%.2f s); "
                                              "the two W4A16 projections are not in the reference figure" % (us[0] * 1e-6, us[1:].sum() * 1e-6)}
    line["clocks"] = sampler.stop()
    line.setdefault("checked", False)
    return line


def _op_work(opcode, a):
    """Scalar operations of one op record, for scaling a reference timing to another sequence length."""
    from gehtp_b200.wtop import OP
    if opcode in (OP.MATMUL_F16, OP.MATMUL_W4A16):
        bn = (a[6] >> 16) if (opcode == OP.MATMUL_F16 and a[6] & 4) else 1
        return a[3] * a[4] * a[5] * max(bn, 1)
    n = {OP.ADD: 3, OP.UNARY: 2, OP.BINARY: 3, OP.BROADCAST: 2, OP.RMSNORM2: 4, OP.GATHER: 3, OP.SLICE: 2, OP.CONCAT: 11}.get(opcode, None)
    if opcode == OP.SOFTMAX:
        return a[2] * a[3]
    if opcode == OP.TRANSPOSE_GEN:
        return a[3] * a[4] * a[5] * max(a[6], 1)
    return max(a[n], 1) if n is not None else None    # None: unknown, the caller scales linearly


def _blob_ops(lib, buf):
    from gehtp_b200.wtop import parse_blob
    rc, blob = parse_blob(lib, np.ascontiguousarray(buf, dtype=np.uint8))
    assert rc == 0
    return [(int(blob.ops[i].opcode), list(blob.ops[i].args)) for i in range(blob.n_ops)]


def reference_sample(args, reps, check=None):
    """Times the reference's own executor (compiled for the host, scalar code,
    one thread as the reference runs it) on a bounded sample of the workload:
    one decoder layer at the full batch and KV context plus a 2048-column slice
    of lm_head, weights dequantised to fp16 because the reference has no
    group-64 W4A16 op. The step time of the whole model is extrapolated linearly
    (layers x layer time + vocab/2048 x head-slice time).

    With `check` (the KV ring of layer 0, the input face and the position of the GPU run's first step),
    the ring is filled with those rows and the first repetition runs that very step, so that its layer
    output can be compared with the GPU's: the one-layer model carries the weights of the whole model's
    first layer, and token ids are taken modulo 1024, the period of the synthetic embedding table."""
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
    if check is None:
        kslot = fill.add_slot(rng.standard_normal(kv_elems).astype(np.float16))
        n_fill = ctx - 1 - reps
        for _ in range(n_fill):
            fill.add_op(OP.KV_APPEND, [S(kslot), S(kslot), ST(0), KV_POS_AUTO])
        feng = Engine(lib, fill.build())
        feng.run()
    else:
        n_fill = check["p0"]
        fface = fill.add_ext_in(2 * kv_elems * 2)
        fill.add_op(OP.SLICE, [S(fface), 1, kv_elems, 1, 0, 0, 0, kv_elems, 0, 0, 1, 1, 1, 2 * kv_elems, 1, 1])
        fill.add_op(OP.SLICE, [S(fface), 2, kv_elems, 1, kv_elems, 0, 0, 2 * kv_elems, 0, 0, 1, 1, 1, 2 * kv_elems, 1, 1])
        fill.add_op(OP.KV_APPEND, [1, 2, ST(0), KV_POS_AUTO])
        feng = Engine(lib, fill.build())
        for p in range(n_fill):
            feng.run_io(check["ring"][p], 0)
    eng = Engine(lib, buf)
    n_ops = eng.blob.n_ops
    op_us = (ctypes.c_int64 * n_ops)()
    err = ctypes.create_string_buffer(256)
    from gehtp_b200.wtop import OP as _OP
    head_ops = [i for i in range(n_ops) if eng.blob.ops[i].opcode == _OP.MATMUL_F16 and eng.blob.ops[i].args[5] == vs]
    times = []
    layer_out = None
    for r in range(reps):
        face = decode_face(man, rng.integers(0, vs, B), n_fill + r, cfg.head_dim, cfg.rope_theta)
        if check is not None and r == 0:
            face = check["face"].copy()
            ids = face[:2 * B].view(np.int32) % 1024
            face[:2 * B] = ids.astype(np.int32).view(np.uint16)
        t0 = time.time()
        rc = lib.wt_exec_run_io(ctypes.byref(eng.blob), face.ctypes.data, None, man["token_temp"], None, op_us, err, 256)
        wall = time.time() - t0
        assert rc == 0, err.value
        us = np.array(op_us[:], dtype=np.float64)
        head = us[head_ops].sum() if head_ops else 0.0
        layer = us.sum() - head
        full_s = (layer * args.layers + head * (cfg.vocab / vs)) * 1e-6
        times.append((wall, full_s))
        if check is not None and r == 0:
            layer_out = eng.temp(man["layer_out"][0]).copy()
    eng.shutdown()
    wall = float(np.mean([t[0] for t in times]))
    full = float(np.mean([t[1] for t in times]))
    return dict(tok_s=B / full, step_s_extrapolated=full, sample_wall_s=wall, reps=reps, layer_out=layer_out,
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
        lib.gehtp_cuda_tp_p2p_export(hb, 64)
        mine = torch.tensor(list(hb), dtype=torch.uint8, device="cuda")
        allh = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        raw = b"".join(bytes(h.cpu().tolist()) for h in allh)
        hbuf = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(raw)
        # every rank calls import; it ends with the ranks' agreement: all use the peer-memory kernels or none does
        if lib.gehtp_cuda_tp_p2p_import(hbuf, 64, world) != 0:
            print("[tp] rank %d: peer-memory mailboxes unavailable (%s); all ranks use NCCL all-reduces"
                  % (rank, lib.gehtp_cuda_last_error().decode(errors="replace")), file=sys.stderr)
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
    if args.config:
        if rank == 0:
            out.append(json.dumps(run_config(args)))
        return out

    if args.impl == "reference":
        if rank != 0:
            return out
        probe = reference_sample(args, 1)
        if probe is None:
            out.append(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libgehtp_ref.so was not built"}))
            return out
        # the probe is the warm-up; the timed repetitions are bounded by a 150 s budget
        reps = int(max(1, min(args.steps, 150.0 // max(probe["sample_wall_s"], 1e-3)))) - 1
        res = reference_sample(args, reps) if reps >= 1 else probe
        line = {"impl": "reference", "metric": METRIC, "value": res["tok_s"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": res["reps"], "steps_requested": args.steps, "warmup": 1, "warmup_requested": args.warmup,
                "ms_per_step": res["step_s_extrapolated"] * 1e3,
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
    traffic, traffic_src = profile_traffic((dom, B, args.ctx, world))
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": r["dev_ms"] / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": config, "clocks": r["clocks"],
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": r["e2e_ms"] / K, "h2d_bytes_per_step": r["face_bytes"],
                    "d2h_bytes_per_step": r["out_bytes"]},
            "gpu_launches": r["launches"],
            "roofline": {"bound": "hbm", "kernel": dom_kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "bytes_per_launch": dbytes / dn, "avg_launch_us": dom_us, "launch_unit_us": dms * 1e3 / dn, **traffic_src},
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
    line["checked"] = False
    if world == 1 and not args.no_cpu_baseline:
        cb = reference_sample(args, 1, check=r.get("check"))
        if cb:
            line["cpu_baseline"] = {"value": cb["tok_s"], "unit": UNIT, "cores": 1, "kind": "reference", "sample": cb["sample"]}
            if cb.get("layer_out") is not None and r.get("check") and r["check"].get("layer_out") is not None:
                # output of decoder layer 0 in the GPU run's first step against the reference executor on the same
                # ring, face and weights: the project's fp16 gate (max |err| <= 1e-2 max|ref|, cosine >= 0.9999)
                got = r["check"]["layer_out"].astype(np.float64)
                want = cb["layer_out"].astype(np.float64)
                err_max, ref_max = float(np.abs(got - want).max()), float(np.abs(want).max())
                cs = float(got @ want / max(np.sqrt((got @ got) * (want @ want)), 1e-300))
                line["checked"] = bool(np.isfinite(got).all() and err_max <= 1e-2 * ref_max and cs >= 0.9999)
                line["check"] = {"what": "layer 0 output of step 0 vs the reference executor (same KV ring, face, weights)",
                                 "max_err": err_max, "ref_max": ref_max, "cosine": cs}
                assert line["checked"], "self-check failed: %r" % (line["check"],)
    out.append(json.dumps(line))
    return out


if __name__ == "__main__":
    main()
