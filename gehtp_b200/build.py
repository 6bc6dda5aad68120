"""Builds libgehtp_cuda.so for sm_100a with nvcc (cross-compiles without a GPU).

Run as `python -m gehtp_b200.build` or through `__graft_entry__.build()`.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libgehtp_cuda.so")
OBJ = os.path.join(HERE, "build")

# translation unit -> extra flags. --fmad=false keeps multiply and add as two
# roundings where the reference's scalar code has two.
UNITS = {
    "wt_parse.cpp": [],
    "executor.cu": [],
    "plan.cu": [],
    "fuse.cu": [],
    "api_kernels.cu": [],
    "ops_elem.cu": ["--fmad=false"],
    "ops_gdn.cu": ["--fmad=false"],
    "gdn_delta_mma.cu": [],
    "ops_attn.cu": [],
    "ops_attn_decode.cu": [],
    "ops_attn_prefill.cu": [],
    "attn_prefill_sm100.cu": [],
    "ops_fused.cu": [],
    "ops_matmul.cu": [],
    "ops_w4a16.cu": [],
    "w4a16_gemm_sm100.cu": [],
    "f16_gemm_sm100.cu": [],
    "tp.cu": [],
    "tp_p2p.cu": [],
}
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _nccl_dirs():
    try:
        import nvidia.nccl as n  # torch's bundled NCCL
        base = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
        return os.path.join(base, "include"), os.path.join(base, "lib")
    except Exception:
        return None, None


def _stale(src, obj):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [src] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    os.makedirs(OBJ, exist_ok=True)
    inc, lib = _nccl_dirs()
    nccl_flags = ["-I" + inc] if inc else []
    jobs = []
    objs = []
    for unit, extra in UNITS.items():
        src = os.path.join(CSRC, unit)
        obj = os.path.join(OBJ, unit.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if force or _stale(src, obj):
            cmd = ["nvcc"] + ARCH + COMMON + nccl_flags + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=8) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: " + cmd[-3])
    if jobs or not os.path.exists(OUT):
        link = ["nvcc", "-shared", "-o", OUT] + objs + ["-lcudart"] + ARCH
        if lib:
            link += ["-L" + lib, "-l:libnccl.so.2", "-Xlinker", "-rpath", "-Xlinker", lib]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    # host runner (job.txt / request-file protocols of the reference's device-side runners)
    run_src = os.path.join(CSRC, "host", "gehtp_run.cpp")
    run_bin = os.path.join(os.path.dirname(OUT), "gehtp_run")
    if force or _stale(run_src, run_bin) or os.path.getmtime(OUT) > os.path.getmtime(run_bin):
        cmd = ["g++", "-O2", "-std=c++17", "-I" + os.path.join(ROOT, "include"), run_src, "-o", run_bin,
               "-L" + os.path.dirname(OUT), "-lgehtp_cuda", "-Wl,-rpath,$ORIGIN", "-pthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("gehtp_run link failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
