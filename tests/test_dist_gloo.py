"""Row sharding, world size 2, gloo on CPU: the host-side logic of the multi-GPU path.

What the ranks exchange on the GPU path is (a) their distinct (feature, value) keys for the cut points, (b) per-level
node row counts and (c) per-level integer histograms.  Here two CPU processes shard the rows the way bench.py does,
exchange the same quantities with torch.distributed (gloo) and check that the union / the sums reproduce the
single-process result of the oracle: cut points identical, summed shard histograms identical (integer sums)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def shard_bounds(n_rows, rank, world):
    return n_rows * rank // world, n_rows * (rank + 1) // world


def _worker(rank, world, port, q):
    for p in (ROOT, os.path.join(ROOT, 'oracle')):
        sys.path.insert(0, p)
    import tgbm_oracle as orc
    from thundergbm_b200 import synth
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    n = 20_000
    full = synth.higgs_like(n, seed=3)
    lo, hi = shard_bounds(n, rank, world)
    mine = synth.higgs_like(n, seed=3, rows=(lo, hi))
    # the shard generator yields exactly the rows of the full data set
    ok_rows = np.array_equal(mine.val, full.val[lo * 28:hi * 28]) and np.array_equal(mine.y, full.y[lo:hi])
    # (a) union of distinct keys -> cut points: gather every rank's distinct (feature, value) pairs
    keys = np.unique(np.stack([mine.col.astype(np.int64), mine.val.view(np.int32).astype(np.int64)], 1), axis=0)
    gathered = [None] * world
    dist.all_gather_object(gathered, keys)
    allk = np.unique(np.concatenate(gathered), axis=0)
    cols = allk[:, 0].astype(np.int32)
    vals = allk[:, 1].astype(np.int32).view(np.float32)
    union = synth.CsrData(allk.shape[0], 28, np.arange(allk.shape[0] + 1, dtype=np.int32), cols, vals,
                          np.zeros(allk.shape[0], np.float32))
    cut_u, ptr_u, _ = orc.bin_only(union, 255)
    cut_f, ptr_f, bins_f = orc.bin_only(full, 255)
    ok_cuts = np.array_equal(cut_u, cut_f) and np.array_equal(ptr_u, ptr_f)
    # (c) integer histogram of the shard, summed over ranks == histogram of all rows
    rng = np.random.default_rng(0)
    gq = rng.integers(-2 ** 18, 2 ** 18, n)  # stand-in for quantised gradients, indexed by global row
    bins_mine = bins_f[lo * 28:hi * 28]
    h = np.bincount(bins_mine, weights=None, minlength=len(cut_f)) * 0
    h = np.zeros(len(cut_f), np.int64)
    np.add.at(h, bins_mine, np.repeat(gq[lo:hi], 28))
    t = torch.from_numpy(h)
    dist.all_reduce(t)
    want = np.zeros(len(cut_f), np.int64)
    np.add.at(want, bins_f, np.repeat(gq, 28))
    ok_hist = np.array_equal(t.numpy(), want)
    # (b) node row counts
    c = torch.tensor([hi - lo])
    dist.all_reduce(c)
    ok_cnt = int(c.item()) == n
    # the 128-byte communicator id travels as an object broadcast from rank 0
    uid = [bytes(range(128)) if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    ok_uid = uid[0] == bytes(range(128))
    q.put((rank, ok_rows, ok_cuts, ok_hist, ok_cnt, ok_uid))
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert len(res) == 2
    for r in res:
        assert all(r[1:]), r


def test_shard_bounds_cover_all_rows():
    for n in (0, 1, 7, 10_500_000):
        for world in (1, 2, 3, 8):
            b = [shard_bounds(n, r, world) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
