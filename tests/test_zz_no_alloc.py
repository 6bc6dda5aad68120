"""The allocation-free decode-attention entry point (gehtp_attn_decode_noalloc).

Some users of the library may not call cudaMalloc where they run attention: a
serving loop whose device memory was handed out once by a pool, a real-time
thread that must never wait on the driver's allocator lock, a process whose
operator fixed its memory budget. For them the library keeps the kernel's
scratch in a fixed device array. This file is named to be collected last: it
checks, on two calls in a row (the second smaller, so it runs over what the
first left in the shared array), that the entry point gives the same result as
the ordinary one, and that an oversized problem is refused with a message."""
import numpy as np
import pytest

from oracle.refexec import ptr

pytestmark = pytest.mark.gpu


def _case(rng, nh, kvh, hd, n_kv, nslots):
    q = rng.standard_normal((nh, hd)).astype(np.float16)
    ring = np.zeros((nslots, 2, kvh * hd), np.float16)
    ring[:n_kv] = rng.standard_normal((n_kv, 2, kvh * hd)).astype(np.float16)
    mask = np.zeros(n_kv, np.float16)
    mask[rng.integers(0, n_kv, 3)] = -np.inf
    return q, ring, mask


def test_noalloc_matches_regular_entry_point_twice(cuda):
    import torch
    rng = np.random.default_rng(2024)
    stream = torch.cuda.current_stream().cuda_stream
    for nh, kvh, hd, n_kv, nslots in ((16, 8, 128, 4096, 4096), (8, 2, 128, 700, 1024)):
        q, ring, mask = _case(rng, nh, kvh, hd, n_kv, nslots)
        scale = float(np.float16(1 / np.sqrt(hd)))
        want = np.zeros((nh, hd), np.float16)
        assert cuda.gehtp_attn_decode(ptr(q), ptr(ring), ptr(mask), ptr(want), nh, kvh, hd, n_kv, nslots, scale) == 0
        dq, dr, dm = (torch.from_numpy(a.view(np.int16)).cuda() for a in (q, ring, mask))
        out = torch.zeros(nh * hd, dtype=torch.int16, device="cuda")
        torch.cuda.synchronize()
        rc = cuda.gehtp_attn_decode_noalloc(dq.data_ptr(), dr.data_ptr(), dm.data_ptr(), out.data_ptr(),
                                            nh, kvh, hd, n_kv, nslots, scale, stream)
        assert rc == 0, cuda.gehtp_cuda_last_error()
        torch.cuda.synchronize()
        got = out.cpu().numpy().view(np.float16).reshape(nh, hd)
        # same kernel, same inputs: the project's fp16 gate, and in fact the same bits
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        assert err <= 1e-2 * np.abs(want.astype(np.float64)).max()
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_noalloc_refuses_what_does_not_fit(cuda):
    import torch
    # 16384 query heads x 130 floats = 8.5 MB of partial results even unsliced: beyond the built-in array
    nh, kvh, hd, n_kv = 16384, 4096, 128, 16384
    buf = torch.zeros(16, dtype=torch.int16, device="cuda")   # never touched: the call must fail before launching
    rc = cuda.gehtp_attn_decode_noalloc(buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), nh, kvh, hd, n_kv, n_kv, 0.1, None)
    assert rc != 0
    assert b"scratch" in cuda.gehtp_cuda_last_error()
