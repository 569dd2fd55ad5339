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
    case, _, extra = case.partition('@')
    make, params = CASES[case]
    d = make()
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw['n_trees'] = min(kw['n_trees'], 4)
    if extra.startswith('column_shards='):
        kw['column_shards'] = int(extra.split('=')[1])
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


@pytest.mark.parametrize('case', ['c2_higgs_small', 'c3_covtype_small', 'fixture_bin', 'fixture_rank', 'c5_mslr_small',
                                  'c2_higgs_small@column_shards=3'])
def test_two_gpus_equal_one_gpu(gpu, cases, case):
    """(`@column_shards=3`: the reference's column-sharded builder as it would run on three devices, computed on two
    row-sharded GPUs: its cut points need the multiplicity of every value over all ranks.)"""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    from thundergbm_b200.booster import Booster
    name, _, extra = case.partition('@')
    d, params = cases(name)
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw['n_trees'] = min(kw['n_trees'], 4)
    if extra.startswith('column_shards='):
        kw['column_shards'] = int(extra.split('=')[1])
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
        if d.group.size:  # NDCG is a mean over ALL query groups, whichever rank holds them
            assert all(0.0 < v <= 1.0 for v in metrics)


def _scikit_train(d, n_device, depth, n_trees, objective, lr, tree_method=b'hist'):
    import ctypes as C
    from thundergbm_b200 import _lib
    from thundergbm_b200.booster import NODE_DTYPE
    lib = _lib.lib()
    val = np.ascontiguousarray(d.val, np.float32); rp = np.ascontiguousarray(d.row_ptr, np.int32)
    col = np.ascontiguousarray(d.col, np.int32); y = np.ascontiguousarray(d.y, np.float32)
    grp = np.ascontiguousarray(d.group, np.int32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    model = C.c_void_p(None)
    num_class = C.c_int(1); per_iter = C.c_int(0)
    group_label = (C.c_float * 64)()
    lib.sparse_train_scikit(d.n_rows, vp(val), vp(rp), vp(col), vp(y), depth, n_trees, n_device, 1.0, 1.0, 1.0, 255, 0, 1.0, 0, 1, lr,
                            objective.encode(), C.byref(num_class), tree_method, C.byref(model), C.byref(per_iter), group_label,
                            vp(grp) if grp.size else None, int(grp.size))
    if not model.value:
        return None, lib.tgbm_last_error().decode()
    n_nodes = (1 << (depth + 1)) - 1
    out = []
    for t in range(n_trees * per_iter.value):
        arrs = [np.zeros(n_nodes, np.int32) for _ in range(4)] + [np.zeros(n_nodes, np.float32) for _ in range(3)]
        lib.get_a_tree(C.byref(model), t, n_nodes, *[vp(a) for a in arrs])
        out.append(np.concatenate([a.view(np.uint8) for a in arrs]).tobytes())
    lib.model_free(C.byref(model))
    return out, ''


@pytest.mark.parametrize('case', ['c2_higgs_small', 'fixture_rank'])
def test_n_device_two_through_the_reference_entry_point(gpu, cases, case):
    """sparse_train_scikit(n_device=2): one process, one host thread per GPU, rows sharded inside the call
    (include/thundergbm/booster.h:39-64 does the same with OpenMP threads).  In the deterministic mode the trees equal
    those of n_device=1 bit for bit."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    d, params = cases(case)
    one, err1 = _scikit_train(d, 1, params['depth'], 3, params['objective'], params['learning_rate'])
    two, err2 = _scikit_train(d, 2, params['depth'], 3, params['objective'], params['learning_rate'])
    assert one is not None and two is not None, (err1, err2)
    assert one == two


def test_fp32_mode_on_two_devices(gpu, cases, monkeypatch):
    """The float arithmetic on two GPUs (spread histogram cells gathered into the all-reduced buffer, float sums of the
    ranks' partial histograms): not bit-identical to one GPU -- the order of the additions differs -- but the same
    trees wherever the split is decisive: root split identical, thresholds of the first tree equal on at least 90 % of
    the nodes, hessian sums of the root's children within 1e-5."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    monkeypatch.setenv('TGBM_HIST_MODE', 'fp32')
    d, params = cases('c2_higgs_small')
    one, err1 = _scikit_train(d, 1, params['depth'], 2, params['objective'], params['learning_rate'])
    two, err2 = _scikit_train(d, 2, params['depth'], 2, params['objective'], params['learning_rate'])
    assert one is not None and two is not None, (err1, err2)
    n = (1 << (params['depth'] + 1)) - 1

    def fields(blob):
        a = np.frombuffer(blob, np.uint8)
        return (a[3 * 4 * n:4 * 4 * n].view(np.int32), a[4 * 4 * n:5 * 4 * n].view(np.float32), a[6 * 4 * n:7 * 4 * n].view(np.float32))
    f1, t1, h1 = fields(one[0])
    f2, t2, h2 = fields(two[0])
    assert f1[0] == f2[0] and t1[0] == t2[0]
    assert np.mean((f1 == f2) & (t1 == t2)) >= 0.9
    assert np.allclose(h1[1:3], h2[1:3], rtol=1e-5)


def test_column_builder_through_the_reference_entry_point(gpu, cases, monkeypatch):
    """TGBM_COLUMN_BUILDER=1: sparse_train_scikit(n_device=2) gives what the reference's two-device builder computes
    (cut points shifted and re-rounded per device, bins counting down, ...), i.e. the trees of column_shards=2 on one GPU."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    from thundergbm_b200.booster import Booster
    d, params = cases('c2_higgs_small')
    monkeypatch.setenv('TGBM_COLUMN_BUILDER', '1')
    two, err = _scikit_train(d, 2, params['depth'], 3, params['objective'], params['learning_rate'])
    assert two is not None, err
    monkeypatch.delenv('TGBM_COLUMN_BUILDER')
    plain, err = _scikit_train(d, 2, params['depth'], 3, params['objective'], params['learning_rate'])
    assert plain is not None and plain != two
    b = Booster(d, objective=params['objective'], depth=params['depth'], n_trees=3, learning_rate=params['learning_rate'], column_shards=2)
    b.boost(3)
    t = b.trees()
    b.close()
    # get_a_tree's view of the first tree: children, default child, feature, threshold, value, hessian sum
    first = np.frombuffer(two[0], np.uint8)
    n = t.shape[2]
    feature = first[3 * 4 * n:4 * 4 * n].view(np.int32)
    threshold = first[4 * 4 * n:5 * 4 * n].view(np.float32)
    assert np.array_equal(feature, t[0, 0]['split_feature_id'])
    assert threshold.tobytes() == t[0, 0]['split_value'].tobytes()


def test_exact_builder_ignores_n_device(gpu, cases, monkeypatch):
    """tree_method=exact trains on one GPU: a call with n_device=2 returns what n_device=1 returns (the reference's
    column-sharded exact builder has the same candidates on any number of devices)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    monkeypatch.setenv('TGBM_HIST_MODE', 'exact')   # integer sums: two runs give the same bits
    d, params = cases('fixture_reg')
    two, err = _scikit_train(d, 2, 3, 2, 'reg:linear', 1.0, tree_method=b'exact')
    assert two is not None, err
    one, err = _scikit_train(d, 1, 3, 2, 'reg:linear', 1.0, tree_method=b'exact')
    assert one is not None, err
    assert one == two
    hist, err = _scikit_train(d, 2, 3, 2, 'reg:linear', 1.0)
    assert hist is not None and hist != two   # and it was the exact builder that ran


def test_n_device_beyond_the_visible_gpus_is_refused(gpu, cases):
    d, params = cases('fixture_reg')
    out, err = _scikit_train(d, 64, 3, 1, 'reg:linear', 1.0)
    assert out is None and 'GPU(s) are visible' in err


def test_bad_query_groups_on_one_rank_stop_every_rank(gpu, cases):
    """A rank-local validation failure (group sizes that do not add up) is agreed on before the first collective: the
    call returns an error instead of leaving the other GPU inside a collective.  The failure is made on the host."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    d, params = cases('fixture_rank')
    bad = d.rows(0, d.n_rows)
    bad.group = d.group.copy()
    bad.group[-1] += 5   # the last rank's groups no longer add up to its rows
    out, err = _scikit_train(bad, 2, 4, 2, 'rank:ndcg', 0.3)
    assert out is None and 'group sizes' in err
    # and the next call on the same devices works (the failed call's communicators were dropped)
    out, err = _scikit_train(d, 2, 4, 2, 'rank:ndcg', 0.3)
    assert out is not None, err
