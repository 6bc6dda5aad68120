"""Tensor-parallel sharding of W4A16 projections, checked on CPU with two
`gloo` ranks: a row-parallel shard pair all-reduced, and a column-parallel pair
all-gathered, must reproduce the unsharded matmul of the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gehtp_b200.runlists import cols, rand_w4, rows
    from oracle.refexec import orc_lib, ptr
    orc = orc_lib()
    rng = np.random.default_rng(77)              # same draw on every rank
    M, K, N = 3, 256, 96
    a = rng.standard_normal((M, K)).astype(np.float16)
    w = rand_w4(rng, K, N)

    def mm(a_, w_):
        k, n = w_[0].shape[0], w_[0].shape[1] * 2
        slot = np.concatenate([w_[0].reshape(-1), w_[1].view(np.uint8).reshape(-1)])
        y = np.zeros((a_.shape[0], n), np.float16)
        orc.orc_w4a16_matmul(ptr(np.ascontiguousarray(a_)), ptr(slot), ptr(y), a_.shape[0], k, n)
        return y
    full = mm(a, w)
    # row parallel: K split, partial sums reduced
    ks = K // world
    part = torch.from_numpy(mm(a[:, rank * ks:(rank + 1) * ks], rows(w, rank * ks, (rank + 1) * ks)).astype(np.float32))
    dist.all_reduce(part)
    # column parallel: N split, outputs gathered
    ns = N // world
    mine = torch.from_numpy(mm(a, cols(w, rank * ns, (rank + 1) * ns)).astype(np.float32))
    parts = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    if rank == 0:
        f = full.astype(np.float32)
        out["row_err"] = float(np.abs(part.numpy() - f).max() / np.abs(f).max())
        out["col_equal"] = bool(np.array_equal(torch.cat(parts, 1).numpy(), f))
    dist.destroy_process_group()


def test_sharded_projections_reproduce_full_matmul():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, 29000 + os.getpid() % 2000, out), nprocs=2, join=True)
    assert out["col_equal"]              # column shards are exact slices of the full result
    assert out["row_err"] < 2e-3         # two fp16-rounded partial sums vs one fp16 rounding


def test_tp_runlists_shard_shapes():
    sys.path.insert(0, ROOT)
    from gehtp_b200.runlists import DecoderConfig, build_decode_runlist
    cfg = DecoderConfig(256, 2, 4, 2, 128, 512, 1024, 1e6, "tiny")
    full, mf = build_decode_runlist(cfg, 2, 32, seed=5, quant="w4")
    shards = [build_decode_runlist(cfg, 2, 32, seed=5, quant="w4", tp=2, rank=r) for r in range(2)]
    assert shards[0][1]["row_parallel_ops"] == shards[1][1]["row_parallel_ops"]
    assert len(shards[0][1]["row_parallel_ops"]) == 2 * cfg.layers
    assert shards[0][0].size < full.size and shards[0][0].size == shards[1][0].size
    assert not np.array_equal(shards[0][0], shards[1][0])
