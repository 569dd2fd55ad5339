"""Row-sharded training on 2 GPUs (one process per GPU, NCCL): the trees must equal the single-GPU trees bit for
bit -- cut points come from the union of the ranks' values, the gradient dither is keyed by the global row id and
all histogram sums are integers.  Skipped on a box with one GPU."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, q):
    for p in (ROOT, os.path.join(ROOT, 'tests', 'golden')):
        sys.path.insert(0, p)
    import torch
    import torch.distributed as dist
    from make_inputs import CASES
    from thundergbm_b200.booster import Booster, Comm
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    uid = [Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = Comm(uid[0], rank, world)
    make, params = CASES[case]
    d = make()
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw['n_trees'] = min(kw['n_trees'], 4)
    lo, hi = d.n_rows * rank // world, d.n_rows * (rank + 1) // world
    if d.group.size:  # cut at query-group boundaries
        ends = np.cumsum(d.group)
        gi = np.searchsorted(ends, [lo, hi], side='left')
        lo = 0 if rank == 0 else int(ends[gi[0] - 1]) if gi[0] > 0 else 0
        hi = d.n_rows if rank == world - 1 else (int(ends[gi[1] - 1]) if gi[1] > 0 else 0)
    shard = d.rows(lo, hi)
    if d.group.size:
        ends = np.cumsum(d.group)
        starts = ends - d.group
        sel = (starts >= lo) & (ends <= hi)
        shard.group = d.group[sel]
    b = Booster(shard, comm=comm, **kw)
    b.boost(kw['n_trees'])
    trees = b.trees()
    metrics = b.metrics()
    b.close()
    comm.close()
    dist.barrier()
    q.put((rank, lo, hi, trees.tobytes(), metrics.tolist()))
    dist.destroy_process_group()


@pytest.mark.parametrize('case', ['c2_higgs_small', 'c3_covtype_small', 'fixture_bin'])
def test_two_gpus_equal_one_gpu(gpu, cases, case):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    from thundergbm_b200.booster import Booster
    d, params = cases(case)
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw['n_trees'] = min(kw['n_trees'], 4)
    b = Booster(d, **kw)
    b.boost(kw['n_trees'])
    want, want_m = b.trees().tobytes(), b.metrics().tolist()
    b.close()
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=120)
    for rank, lo, hi, trees, metrics in res:
        assert trees == want, f'rank {rank} rows [{lo},{hi}) trees differ from the single-GPU run'
        assert np.allclose(metrics, want_m, rtol=0, atol=1e-6)
