"""The host runner binary (`gehtp_run`): job.txt protocol of the reference's
42_gehtp_runner and the request-file protocol of 42_gehtp_persistent."""
import json
import os
import struct
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
RUNNER = os.path.join(ROOT, "gehtp_b200", "gehtp_run")


def _tiny_blob(tmp_path):
    """y = (x + x) * x over 64 fp16 values read from the EXT_IN face."""
    from gehtp_b200.wtop import OP, S, BlobBuilder
    b = BlobBuilder()
    face = b.add_ext_in(128)
    b.add_op(OP.ADD, [S(face), S(face), 1, 64])
    b.add_op(OP.BINARY, [1, S(face), 2, 64, 2])
    path = tmp_path / "tiny.wtop"
    path.write_bytes(b.build().tobytes())
    return str(path)


def test_usage_and_missing_keys(tmp_path):
    assert os.path.exists(RUNNER), "gehtp_run is not built (python -m gehtp_b200.build)"
    assert subprocess.run([RUNNER], capture_output=True).returncode == 2
    job = tmp_path / "job.txt"
    job.write_text("blob /nonexistent\n")
    r = subprocess.run([RUNNER, "job", str(job)], capture_output=True, text=True)
    assert r.returncode == 1 and "lacks one of blob/input/output/out_temp" in r.stdout


@pytest.mark.skipif(__import__("torch").cuda.is_available(), reason="checks the behaviour without a GPU")
def test_job_fails_loudly_without_a_gpu(tmp_path):
    blob = _tiny_blob(tmp_path)
    (tmp_path / "in.raw").write_bytes(np.ones(64, np.float16).tobytes())
    job = tmp_path / "job.txt"
    job.write_text("blob %s\ninput %s\noutput %s\nout_temp 2\n" % (blob, tmp_path / "in.raw", tmp_path / "out.raw"))
    r = subprocess.run([RUNNER, "job", str(job)], capture_output=True, text=True)
    assert r.returncode == 1 and "[FAIL] wt_exec_run_io rc=-1" in r.stdout and not (tmp_path / "out.raw").exists()


@pytest.mark.gpu
def test_job_single_run_and_decode_loop(tmp_path):
    blob = _tiny_blob(tmp_path)
    x = (np.arange(64) / 8.0 - 3).astype(np.float16)
    want = ((x + x).astype(np.float16) * x).astype(np.float16)
    (tmp_path / "in.raw").write_bytes(x.tobytes())
    job = tmp_path / "job.txt"
    job.write_text("blob %s\ninput %s\noutput %s\nout_temp 2\n" % (blob, tmp_path / "in.raw", tmp_path / "out.raw"))
    r = subprocess.run([RUNNER, "job", str(job)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "[PASS] gehtp_run overall" in r.stdout and "op_timing code=7 n=1" in r.stdout
    got = np.frombuffer((tmp_path / "out.raw").read_bytes(), np.float16)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    ts = (tmp_path / "out.raw.op_ts.bin").read_bytes()
    magic, ver, n_ops = struct.unpack_from("<4sII", ts, 0)
    assert magic == b"WTS1" and ver == 2 and n_ops == 2 and len(ts) == 24 + 2 * 20
    # decode loop: inputs in.raw.<i>, outputs out.raw.<i>
    for i in range(3):
        (tmp_path / ("in.raw.%d" % i)).write_bytes((x + np.float16(i)).astype(np.float16).tobytes())
    job.write_text("blob %s\ninput %s\noutput %s\nout_temp 2\nsteps 3\n" % (blob, tmp_path / "in.raw", tmp_path / "out.raw"))
    r = subprocess.run([RUNNER, "job", str(job)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    for i in range(3):
        xi = (x + np.float16(i)).astype(np.float16)
        wi = ((xi + xi).astype(np.float16) * xi).astype(np.float16)
        gi = np.frombuffer((tmp_path / ("out.raw.%d" % i)).read_bytes(), np.float16)
        assert np.array_equal(gi.view(np.uint16), wi.view(np.uint16))


def _request(tmp_path, header, body=b""):
    h = json.dumps(header).encode()
    tmp = tmp_path / "req.tmp"
    tmp.write_bytes(struct.pack(">I", len(h)) + h + body)
    os.rename(tmp, tmp_path / "req")
    resp = tmp_path / "resp"
    for _ in range(3000):
        if resp.exists():
            raw = resp.read_bytes()
            if len(raw) >= 4 and len(raw) == 4 + struct.unpack(">I", raw[:4])[0]:
                os.unlink(resp)
                return json.loads(raw[4:])
        time.sleep(0.005)
    raise AssertionError("no response to %r" % header)


@pytest.mark.gpu
def test_serve_request_files(tmp_path):
    blob = _tiny_blob(tmp_path)
    job = tmp_path / "job.txt"
    job.write_text("blob %s\nreq %s\nresp %s\nout %s\nout_temp 2\nin_bytes 128\nidle_exit_s 20\n"
                   % (blob, tmp_path / "req", tmp_path / "resp", tmp_path / "out.raw"))
    proc = subprocess.Popen([RUNNER, "serve", str(job)], stdout=subprocess.PIPE, text=True)
    try:
        assert _request(tmp_path, {"op": "ping"}) == {"rc": 0, "pong": 1}
        x = np.zeros(64, np.float16)
        x[17] = 3.0
        r = _request(tmp_path, {"op": "run", "want_out": 1}, x.tobytes())
        assert r["rc"] == 0 and r["token"] == 17 and r["steps"] == 1
        got = np.frombuffer((tmp_path / "out.raw").read_bytes(), np.float16)
        assert got[17] == 18.0 and got.sum() == 18.0
        assert _request(tmp_path, {"op": "reset"})["reset"] == 1
        assert _request(tmp_path, {"op": "nope"})["rc"] == -1
        assert _request(tmp_path, {"op": "shutdown"})["bye"] == 1
        assert proc.wait(timeout=20) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
