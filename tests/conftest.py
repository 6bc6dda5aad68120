import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _make_oracle():
    """Builds the CPU checkers when they are missing. The reference executor can only be built
    where the reference tree is; its location comes from $GEHTP_REFERENCE_DIR (passed to the
    Makefile as REF), else the Makefile's own default is tried."""
    have_orc = os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so"))
    have_ref = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libgehtp_ref.so"))
    if have_orc and have_ref:
        return
    cmd = ["make", "-C", os.path.join(ROOT, "oracle")]
    if os.environ.get("GEHTP_REFERENCE_DIR"):
        cmd.append("REF=" + os.environ["GEHTP_REFERENCE_DIR"])
    subprocess.run(cmd, check=True, capture_output=True)


@pytest.fixture(scope="session")
def orc():
    _make_oracle()
    from oracle.refexec import orc_lib
    return orc_lib()


@pytest.fixture()
def ref(tmp_path):
    """The reference executor compiled for the host. Its persistent-state table
    is loaded once per process, so every test gets a private copy of the
    library (own globals). Skipped where the library cannot be had."""
    _make_oracle()
    from oracle.refexec import ref_lib
    lib = ref_lib(private_dir=str(tmp_path))
    if lib is None:
        pytest.skip("oracle/_ref/libgehtp_ref.so not available")
    return lib


@pytest.fixture(scope="session")
def cuda():
    import gehtp_b200
    if not os.path.exists(gehtp_b200.LIB_PATH):
        from gehtp_b200.build import build
        build()
    return gehtp_b200.lib()


def f16_bits(a):
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def cos_sim(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(a @ b / max(np.sqrt((a @ a) * (b @ b)), 1e-300))


def assert_fp16_close(got, want, what=""):
    """The fp16 gate of this project: max |err| <= 1e-2 * max|ref| and cosine >= 0.9999."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what + ": non-finite values"
    err = np.abs(got - want).max()
    ref_max = np.abs(want).max()
    cs = cos_sim(got, want)
    assert err <= 1e-2 * ref_max + 1e-12, "%s: max err %g vs 1e-2*%g" % (what, err, ref_max)
    assert cs >= 0.9999, "%s: cos %f" % (what, cs)


def ulp_diff_f16(a, b):
    """Distance in fp16 steps between two fp16 bit arrays (same-sign finite values)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(np.asarray(a, np.uint16)) - key(np.asarray(b, np.uint16)))
