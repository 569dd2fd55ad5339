"""tree_method = exact: the reference's ExactTreeBuilder (every distinct stored value of a node is a split candidate,
src/thundergbm/builder/exact_tree_builder.cu) on the GPU, through the C ABI

* in the fixed-point arithmetic bit for bit against the CPU oracle's restatement of that builder (all 48 bytes of every
  node, the row -> node table of every tree, raw scores, metrics);
* in the float arithmetic against what the reference itself produced with tree_method=exact
  (tests/golden/ref_exact_*.npz, three runs each): per-round metric and logloss to 1e-4 (plus twice the reference's
  own spread), gains and weights of the first tree along identically split paths to 1e-5 plus summation noise.
"""
import numpy as np
import pytest

from common import compare_with_noise, load_golden, sum_noise, within_noise

pytestmark = pytest.mark.gpu

CASES = ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small']


def _booster(d, params, **extra):
    from thundergbm_b200.booster import Booster
    kw = dict(params)
    kw.update(extra)
    kw['tree_method'] = 'exact'
    return Booster(d, **kw)


@pytest.mark.parametrize('name', CASES)
def test_bit_exact_with_oracle(gpu, orc, cases, name):
    d, params = cases(name)
    p = {**params, 'n_trees': min(params['n_trees'], 6), 'tree_method': 'exact'}
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = _booster(d, p, keep_nid=1, hist_mode='exact')
    assert b.info.n_bins == 0
    b.boost(p['n_trees'])
    trees = b.trees()
    assert trees.shape == o.trees.shape
    for r in range(trees.shape[0]):
        for k in range(trees.shape[1]):
            assert trees[r, k].tobytes() == o.trees[r, k].tobytes(), f'tree {r}/{k} differs'
    assert np.array_equal(b.nid(), o.nid)
    assert np.array_equal(b.ypred(), o.ypred)
    assert np.array_equal(b.metrics(), o.metric)
    b.close()


def test_column_sampling_and_bagging(gpu, orc, cases):
    d, params = cases('c2_higgs_small')
    p = {**params, 'n_trees': 4, 'depth': 5, 'tree_method': 'exact'}
    o = orc.train(d, hist_mode=1, keep_nid=1, bagging=1, column_sampling_rate=0.4, sample_seed=9, **p)
    b = _booster(d, p, keep_nid=1, hist_mode='exact', bagging=1, column_sampling_rate=0.4, sample_seed=9)
    b.boost(4)
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid)
    b.close()


def test_auto_resolves_to_exact_above_20000_features(gpu, orc, cases):
    """src/thundergbm/trainer.cu:19-23 through the reference's own entry point: 25000 columns and tree_method=auto train
    with the exact builder.  Thresholds of the first tree as get_a_tree reports them (scikit_tgbm.cpp:199-248)."""
    import ctypes as C
    from thundergbm_b200 import _lib, synth
    _, params = cases('c4_sparse_small')
    d = synth.sparse_binary(20_000, 25_000, seed=11)
    assert d.n_cols > 20000
    lib = _lib.lib()
    val = np.ascontiguousarray(d.val, np.float32); rp = np.ascontiguousarray(d.row_ptr, np.int32)
    col = np.ascontiguousarray(d.col, np.int32); y = np.ascontiguousarray(d.y, np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    model = C.c_void_p(None)
    num_class = C.c_int(2); per_iter = C.c_int(0)
    group_label = (C.c_float * 64)()
    depth, n_trees = params['depth'], 2
    lib.sparse_train_scikit(d.n_rows, vp(val), vp(rp), vp(col), vp(y), depth, n_trees, 1, C.c_float(params['min_child_weight']),
                            C.c_float(params['lambda']), C.c_float(params['gamma']), params['max_num_bin'], 0, C.c_float(1.0), 0, 1,
                            C.c_float(params['learning_rate']), params['objective'].encode(), C.byref(num_class), b'auto',
                            C.byref(model), C.byref(per_iter), group_label, None, 0)
    assert model.value, lib.tgbm_last_error().decode()
    n_nodes = C.c_int(0)
    lib.get_n_nodes(C.byref(model), C.byref(n_nodes), 1, 1)
    nn = n_nodes.value
    arrs = [np.zeros(nn, np.int32) for _ in range(4)] + [np.zeros(nn, np.float32) for _ in range(3)]
    lib.get_a_tree(C.byref(model), 0, nn, *[vp(a) for a in arrs])
    lib.model_free(C.byref(model))
    o = orc.train(d, hist_mode=0, portable_exp=1, n_threads=1, **{**params, 'n_trees': 2, 'tree_method': 'exact'})
    root = o.trees[0, 0][0]
    assert arrs[3][0] == root['split_feature_id']
    # a midpoint between two stored values (or below the smallest one), not one of 64 cut points
    assert arrs[4][0].tobytes() == root['split_value'].tobytes()


@pytest.mark.parametrize('name', CASES)
def test_fp32_follows_the_reference(gpu, orc, cases, name):
    from pack_golden import logloss
    g = load_golden('exact_' + name)
    d, params = cases(name)
    b = _booster(d, params, hist_mode='fp32')
    assert abs(b.info.base_score - float(g['base_score'])) <= 1e-6 * max(1.0, abs(float(g['base_score'])))
    b.boost(params['n_trees'])
    m = b.metrics()
    tol_m = max(1e-4, 2 * float(g['spread_metric']))
    assert np.max(np.abs(m - g['metric'])) <= tol_m, (np.max(np.abs(m - g['metric'])), tol_m)
    ll = logloss(params['objective'], b.ypred(), d.y, g['label'])
    if ll is not None:
        assert abs(ll - float(g['logloss'])) <= max(1e-4, 2 * float(g['spread_logloss']))
    labels = g['label']
    classes = max(1, labels.size)
    k = classes if classes > 2 else 1
    y = np.searchsorted(labels, d.y).astype(np.float32) if labels.size else d.y
    yp = np.full(k * d.n_rows, float(g['base_score']) if k == 1 else 0.0, np.float32)
    gh = orc.gradient(y, yp, params['objective'], K=k)
    # the largest run of equal values of a column bounds the length of any single float sum
    n_max = int(max(np.unique(d.val[d.col == f], return_counts=True)[1].max() for f in np.unique(d.col)[:64]))
    dG, dH = sum_noise(gh[:d.n_rows], n_max)
    ref, mine = g['trees'][0, 0].copy(), b.trees()[0, 0].copy()
    r = compare_with_noise(ref, mine, dG, dH, lam=params['lambda'])
    r.pop('parted')
    assert r['compared'] >= 1 and within_noise(r, hard=8.0), (name, r['worst_gain'], r['worst_weight'], r['bad_gain'], r['bad_weight'])
    b.close()


@pytest.mark.parametrize('n,f,density', [(1, 3, 1.0), (2, 1, 1.0), (33, 5, 0.5), (1000, 40, 0.3), (1025, 31, 1.0)])
def test_ragged_shapes(gpu, orc, n, f, density):
    """One row, one feature, rows without any stored value, features nobody stores."""
    from thundergbm_b200 import synth
    rng = np.random.default_rng(n + f)
    x = np.round(rng.standard_normal((n, f)) * 3).astype(np.float32) / 2      # few distinct values: long runs of equal values
    x[rng.random((n, f)) > density] = 0
    if not x.any():
        x[0, 0] = 1.0
    y = (x[:, 0] - x[:, 1 % f] + 0.3 * rng.standard_normal(n)).astype(np.float32)
    d = synth.dense_to_csr(x, y)
    p = dict(objective='reg:linear', depth=4, n_trees=3, max_num_bin=255, learning_rate=0.5, tree_method='exact')
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = _booster(d, p, keep_nid=1, hist_mode='exact')
    b.boost(3)
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid) and np.array_equal(b.ypred(), o.ypred)
    b.close()


@pytest.mark.parametrize('depth', [1, 10])
def test_depth_extremes(gpu, orc, cases, depth):
    d, params = cases('fixture_bin')
    p = {**params, 'depth': depth, 'n_trees': 2, 'tree_method': 'exact'}
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = _booster(d, p, keep_nid=1, hist_mode='exact')
    b.boost(2)
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid)
    b.close()


def test_cli_with_tree_method_exact(gpu, tmp_path):
    """thundergbm-train with tree_method=exact in the conf: split values are midpoints of stored values."""
    import os
    import subprocess
    from thundergbm_b200 import synth
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = synth.dense_regression(1500, 6, seed=9)
    data = tmp_path / 'train.txt'
    with open(data, 'w') as fh:
        for i in range(d.n_rows):
            a, b = d.row_ptr[i], d.row_ptr[i + 1]
            fh.write(f'{d.y[i]:.9g} ' + ' '.join(f'{c + 1}:{v:.9g}' for c, v in zip(d.col[a:b], d.val[a:b])) + '\n')
    conf = tmp_path / 'run.conf'
    conf.write_text(f'data={data}\ndepth=3\nn_trees=4\nlearning_rate=0.5\nobjective=reg:linear\ntree_method=exact\n')
    out = subprocess.run([os.path.join(root, 'thundergbm_b200', 'bin', 'thundergbm-train'), str(conf)], cwd=tmp_path,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert '[4/4] RMSE = ' in out.stdout and os.path.exists(tmp_path / 'tgbm.model')
    from pack_golden import read_model, tree_view
    t = tree_view(read_model(str(tmp_path / 'tgbm.model'))['trees'])
    root_node = t[0, 0][0]
    col = np.sort(d.val[d.col == root_node['split_feature_id']])
    mids = ((col[1:] + col[:-1]) * np.float32(0.5)).astype(np.float32)
    assert root_node['split_bid'] == 0 and np.any(mids == root_node['split_value'])
