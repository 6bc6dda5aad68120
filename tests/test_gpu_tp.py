"""Tensor-parallel decode on two GPUs against the same runlist on one GPU.

Two child processes (one per GPU) run rank 0 and rank 1 of a sharded decode
runlist through the C-ABI engine, once with NCCL all-reduces and once with the
one-kernel all-reduce over peer memory; the replicated final hidden state and
the merged greedy tokens must agree with the unsharded run. Skipped on a box
with fewer than two GPUs."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu

STEPS, B, NSLOTS = 4, 3, 64


def _cfg():
    from gehtp_b200.runlists import DecoderConfig
    return DecoderConfig(256, 2, 4, 2, 128, 512, 1024, 1e6, "tiny")


def _run_steps(lib, buf, man, cfg, merge=None):
    """STEPS decode steps on fixed input tokens; returns per step (final hidden state, merged greedy tokens, logits)."""
    from gehtp_b200.runlists import decode_face
    from gehtp_b200.wtop import Engine
    lib.wt_exec_state_reset()
    eng = Engine(lib, buf)
    hid, out_toks, logits = [], [], []
    width = 3 * B if man["tp"] > 1 else 2 * B
    for s in range(STEPS):
        ids = [(7 * s + 3 * b + 1) % 1000 for b in range(B)]
        face = decode_face(man, ids, s, cfg.head_dim, cfg.rope_theta)
        out = np.zeros(width, np.uint16)
        eng.run_io(face, man["token_temp"], out)
        hid.append(eng.temp(man["hidden_temp"]).copy())
        logits.append(eng.temp(man["logits_temp"]).reshape(B, -1).copy())
        local = out[:2 * B].view(np.int32).copy()
        out_toks.append(merge(local, out[2 * B:].view(np.float16).copy()) if merge else local)
    eng.shutdown()
    return hid, out_toks, logits


def _worker(rank, world, port, p2p, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import gehtp_b200
    from gehtp_b200.runlists import build_decode_runlist
    lib = gehtp_b200.lib()
    assert lib.gehtp_cuda_set_device(rank) == 0
    idb = (ctypes.c_uint8 * 128)()
    if rank == 0:
        assert lib.gehtp_cuda_tp_unique_id(idb, 128) == 0
    t = torch.tensor(list(idb), dtype=torch.uint8, device="cuda")
    dist.broadcast(t, 0)
    cbuf = (ctypes.c_uint8 * 128).from_buffer_copy(bytes(t.cpu().tolist()))
    assert lib.gehtp_cuda_tp_init(rank, world, cbuf, 128) == 0, lib.gehtp_cuda_last_error()
    if p2p:
        hb = (ctypes.c_uint8 * 64)()
        assert lib.gehtp_cuda_tp_p2p_export(hb, 64) == 0, lib.gehtp_cuda_last_error()
        mine = torch.tensor(list(hb), dtype=torch.uint8, device="cuda")
        allh = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        hbuf = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(b"".join(bytes(h.cpu().tolist()) for h in allh))
        if p2p == 3:
            # rank 1 is handed a handle that maps nothing: its import fails on the host (an error code of
            # cudaIpcOpenMemHandle, no GPU involved), and the agreement inside import makes rank 0 give up as well:
            # -1 on both ranks, and the run goes through NCCL
            if rank == 1:
                hbuf = (ctypes.c_uint8 * (64 * world))(*([0xA5] * (64 * world)))
            assert lib.gehtp_cuda_tp_p2p_import(hbuf, 64, world) == -1
            assert b"NCCL" in lib.gehtp_cuda_last_error() or b"cudaIpcOpenMemHandle" in lib.gehtp_cuda_last_error()
        else:
            assert lib.gehtp_cuda_tp_p2p_import(hbuf, 64, world) == 0, lib.gehtp_cuda_last_error()
        if p2p == 2:    # mailboxes mapped, then given up on every rank: the run must go through NCCL again
            lib.gehtp_cuda_tp_p2p_disable()
    cfg = _cfg()
    buf, man = build_decode_runlist(cfg, B, NSLOTS, seed=21, quant="w4", tp=world, rank=rank)
    idx = (ctypes.c_uint32 * len(man["row_parallel_ops"]))(*man["row_parallel_ops"])
    assert lib.gehtp_cuda_tp_allreduce_after(idx, len(man["row_parallel_ops"])) == 0
    vs = man["vocab_shard"]

    def merge(local_tok, local_max):
        # every rank proposes (max logit, global token id); the largest value wins, lowest rank on ties
        prop = torch.tensor(np.stack([local_max.astype(np.float32), (local_tok + rank * vs).astype(np.float32)]), device="cuda")
        allp = [torch.zeros_like(prop) for _ in range(world)]
        dist.all_gather(allp, prop)
        vals = torch.stack([p[0] for p in allp]).cpu().numpy()
        ids = torch.stack([p[1] for p in allp]).cpu().numpy()
        best = vals.argmax(0)
        return ids[best, np.arange(B)].astype(np.int32)
    hid, toks, _ = _run_steps(lib, buf, man, cfg, merge)
    if rank == 0:
        ret["hid"] = [h.view(np.uint16).tolist() for h in hid]
        ret["toks"] = [t.tolist() for t in toks]
    dist.barrier()
    lib.wt_exec_shutdown()
    lib.gehtp_cuda_tp_shutdown()
    dist.destroy_process_group()


@pytest.mark.parametrize("p2p", [0, 1, 2, 3])
def test_tp2_decode_matches_single_gpu(p2p):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import gehtp_b200
    from gehtp_b200.runlists import build_decode_runlist
    cfg = _cfg()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, 29100 + (os.getpid() + p2p) % 1500, p2p, ret), nprocs=2, join=True)
    # the unsharded run in this process
    lib = gehtp_b200.lib()
    assert lib.gehtp_cuda_set_device(0) == 0
    buf, man = build_decode_runlist(cfg, B, NSLOTS, seed=21, quant="w4")
    hid1, toks1, logits1 = _run_steps(lib, buf, man, cfg)
    lib.wt_exec_shutdown()
    for s in range(STEPS):
        got = np.array(ret["hid"][s], np.uint16).view(np.float16).astype(np.float64)
        want = hid1[s].astype(np.float64)
        err = np.abs(got - want).max()
        assert err <= 1e-2 * np.abs(want).max(), "step %d: hidden state max err %g" % (s, err)
        cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
        assert cos >= 0.9999, "step %d: cosine %g" % (s, cos)
        # greedy tokens: the merged pick of the two ranks must be (within rounding) the unsharded maximum
        lg = logits1[s].astype(np.float64)
        for b in range(B):
            t = ret["toks"][s][b]
            assert 0 <= t < lg.shape[1]
            assert lg[b, t] >= lg[b].max() - 1e-2 * np.abs(lg[b]).max(), "step %d seq %d: token %d is not the maximum" % (s, b, t)
