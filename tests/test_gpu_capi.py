"""The reference's own extern "C" surface (what its Python wrapper binds), through ctypes."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


def _train(lib, d, objective, depth=5, n_trees=4, lr=0.3, max_bin=64, num_class=1):
    val = np.ascontiguousarray(d.val, np.float32); rp = np.ascontiguousarray(d.row_ptr, np.int32)
    col = np.ascontiguousarray(d.col, np.int32); y = np.ascontiguousarray(d.y, np.float32)
    grp = np.ascontiguousarray(d.group, np.int32)
    model = C.c_void_p(None)
    nc = C.c_int(num_class); per = C.c_int(0)
    gl = (C.c_float * 64)()
    lib.sparse_train_scikit(d.n_rows, _vp(val), _vp(rp), _vp(col), _vp(y), depth, n_trees, 1, 1.0, 1.0, 1.0, max_bin, 0,
                            1.0, 0, 1, lr, objective.encode(), C.byref(nc), b'hist', C.byref(model), C.byref(per), gl,
                            _vp(grp) if grp.size else None, int(grp.size))
    assert model.value, lib.tgbm_last_error().decode()
    return model, nc.value, per.value, np.array(gl[:max(nc.value, 1)], np.float32)


def _predict(lib, d, model, n_trees, per, objective, nc, lr, gl, n_out):
    val = np.ascontiguousarray(d.val, np.float32); rp = np.ascontiguousarray(d.row_ptr, np.int32)
    col = np.ascontiguousarray(d.col, np.int32)
    out = np.zeros(n_out, np.float32)
    glc = (C.c_float * len(gl))(*gl)
    lib.sparse_predict_scikit(d.n_rows, _vp(val), _vp(rp), _vp(col), _vp(out), C.byref(model), n_trees, per,
                              objective.encode(), nc, lr, glc, None, 0, 0)
    return out


def test_train_predict_save_load_roundtrip(gpu, orc, cases, tmp_path):
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    d, _ = cases('fixture_bin')
    model, nc, per, gl = _train(lib, d, 'binary:logistic')
    assert nc == 2 and per == 1 and gl.tolist() == [-1.0, 1.0]
    n_nodes = np.zeros(4, np.int32)
    lib.get_n_nodes(C.byref(model), _vp(n_nodes), 4, 1)
    assert (n_nodes == 63).all()
    arrs = [np.zeros(63, np.int32) for _ in range(4)] + [np.zeros(63, np.float32) for _ in range(3)]
    lib.get_a_tree(C.byref(model), 0, 63, *[_vp(a) for a in arrs])
    left, right, default, feat, thr, val, w = arrs
    o = orc.train(d, objective='binary:logistic', depth=5, n_trees=4, learning_rate=0.3, max_num_bin=64, hist_mode=1)
    t0 = o.trees[0, 0]
    leaf = t0['is_leaf'] == 1
    assert np.array_equal(feat, t0['split_feature_id']) and np.array_equal(thr, t0['split_value'])
    assert np.array_equal(left[~leaf], t0['lch_index'][~leaf]) and (left[leaf] == -1).all()
    assert np.array_equal(val[leaf], t0['base_weight'][leaf]) and np.array_equal(w, t0['sum_h'])
    pred = _predict(lib, d, model, 4, per, 'binary:logistic', nc, 0.3, gl, d.n_rows)
    assert set(np.unique(pred)) <= {-1.0, 1.0}
    # the scikit predict path does not apply the base score (src/thundergbm/scikit_tgbm.cpp:87-90)
    raw = orc.predict_raw(d, o.trees, 0.3, 0.0, n_features=d.n_cols)[0]
    assert np.array_equal(pred, np.where(raw > 0, 1.0, -1.0).astype(np.float32))
    # save -> load -> identical predictions, and the file has the reference's layout
    path = str(tmp_path / 'm.model').encode()
    glc = (C.c_float * 2)(*gl)
    lib.save(path, b'binary:logistic', 0.3, nc, 4, per, C.byref(model), glc)
    lr2 = C.c_float(0); nc2 = C.c_int(0); nt2 = C.c_int(0); per2 = C.c_int(0); model2 = C.c_void_p(None)
    lib.load_model(path, C.byref(lr2), C.byref(nc2), C.byref(nt2), C.byref(per2), C.byref(model2))
    assert model2.value and (round(lr2.value, 6), nc2.value, nt2.value, per2.value) == (0.3, 2, 4, 1)
    gl2 = (C.c_float * 2)()
    lib.load_config(path, gl2)
    assert list(gl2) == [-1.0, 1.0]
    pred2 = _predict(lib, d, model2, 4, 1, 'binary:logistic', 2, 0.3, gl, d.n_rows)
    assert np.array_equal(pred, pred2)
    raw_file = open(path.decode(), 'rb').read()
    assert raw_file[:4] == (15).to_bytes(4, 'little') and raw_file[4:19] == b'binary:logistic'
    assert len(raw_file) == 4 + 15 + 16 + 4 + 8 + 4 + 4 * (4 + 8 + 63 * 48)
    lib.model_free(C.byref(model)); lib.model_free(C.byref(model2))
    assert model.value is None


def test_multiclass_and_softprob(gpu, orc, cases):
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    d, _ = cases('c3_covtype_small')
    d = d.rows(0, 5000)
    for obj in ('multi:softmax', 'multi:softprob'):
        model, nc, per, gl = _train(lib, d, obj, depth=4, n_trees=2, lr=0.5)
        assert nc == 7 and per == 7
        n_out = d.n_rows * (7 if obj == 'multi:softprob' else 1)
        pred = _predict(lib, d, model, 2, per, obj, nc, 0.5, gl, n_out)
        if obj == 'multi:softprob':
            p = pred.reshape(7, d.n_rows)  # class-major, as the reference lays it out
            assert np.allclose(p.sum(axis=0), 1.0, atol=1e-5)
        else:
            assert set(np.unique(pred)) <= set(gl.tolist())
            assert (pred == d.y).mean() > 0.3
        lib.model_free(C.byref(model))


def test_errors_leave_model_null(gpu, cases):
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    d, _ = cases('fixture_reg')
    val = np.ascontiguousarray(d.val, np.float32); rp = np.ascontiguousarray(d.row_ptr, np.int32)
    col = np.ascontiguousarray(d.col, np.int32); y = np.ascontiguousarray(d.y, np.float32)
    model = C.c_void_p(123)
    nc = C.c_int(1); per = C.c_int(0); gl = (C.c_float * 4)()
    lib.sparse_train_scikit(d.n_rows, _vp(val), _vp(rp), _vp(col), _vp(y), 5, 2, 1, 1.0, 1.0, 1.0, 64, 0, 1.0, 0, 1, 0.3,
                            b'reg:linear', C.byref(nc), b'approx', C.byref(model), C.byref(per), gl, None, 0)
    assert model.value is None and b'tree_method' in lib.tgbm_last_error()
    # an objective the library does not know
    model = C.c_void_p(123)
    lib.sparse_train_scikit(d.n_rows, _vp(val), _vp(rp), _vp(col), _vp(y), 5, 2, 1, 1.0, 1.0, 1.0, 64, 0, 1.0, 0, 1, 0.3,
                            b'reg:nonsense', C.byref(nc), b'exact', C.byref(model), C.byref(per), gl, None, 0)
    assert model.value is None and b'objective' in lib.tgbm_last_error()


def test_python_mirror_classes(gpu, cases):
    from thundergbm_b200.thundergbm import TGBMClassifier, TGBMRegressor
    import scipy.sparse as sp
    d, _ = cases('c1_dense_reg')
    X = sp.csr_matrix((d.val, d.col, d.row_ptr), shape=(d.n_rows, d.n_cols))
    reg = TGBMRegressor(depth=5, n_trees=10, learning_rate=0.5, verbose=0)
    reg.fit(X, d.y)
    p = reg.predict(X)
    # the scikit predict path drops the base score, exactly like the reference's wrapper
    assert np.sqrt(np.mean((p + reg_base(d) - d.y) ** 2)) < np.std(d.y) * 0.6
    d2, _ = cases('fixture_bin')
    X2 = sp.csr_matrix((d2.val, d2.col, d2.row_ptr), shape=(d2.n_rows, d2.n_cols))
    clf = TGBMClassifier(depth=5, n_trees=6, learning_rate=0.5, verbose=0, objective='binary:logistic')
    clf.fit(X2, d2.y)
    assert (clf.predict(X2) == d2.y).mean() > 0.8
    with pytest.raises(RuntimeError, match='binary:logistic'):
        TGBMClassifier(depth=3, n_trees=1, verbose=0).fit(X2, d2.y)  # multi:softmax with two labels


def reg_base(d):
    return float(np.mean(d.y))


def test_python_mirror_cv_and_tree_arrays(gpu, cases):
    """cv() and the tree arrays behind get_shap_trees() of the reference's wrapper (python/thundergbm/thundergbm.py:223-351)."""
    from thundergbm_b200.thundergbm import TGBMClassifier, TGBMRanker, TGBMRegressor
    import scipy.sparse as sp
    d, _ = cases('fixture_bin')
    X = sp.csr_matrix((d.val, d.col, d.row_ptr), shape=(d.n_rows, d.n_cols))
    clf = TGBMClassifier(depth=4, n_trees=5, learning_rate=0.5, verbose=0, objective='binary:logistic')
    res = clf.cv(X, d.y, nfold=3, seed=1)
    assert set(res) == {'train-accuracy-mean', 'train-accuracy-std', 'test-accuracy-mean', 'test-accuracy-std'}
    assert 0.7 < res['test-accuracy-mean'] <= res['train-accuracy-mean'] + 0.05 <= 1.05
    trees = clf.get_trees()
    assert len(trees) == 5 and all(t['children_left'].shape == (31,) for t in trees)
    root = trees[0]
    assert root['children_left'][0] == 1 and root['children_right'][0] == 2 and root['children_default'][0] in (1, 2)
    leaves = root['children_left'] == -1
    assert leaves.any() and np.all(root['value'][~leaves] == 0)
    d1, _ = cases('c1_dense_reg')
    X1 = sp.csr_matrix((d1.val, d1.col, d1.row_ptr), shape=(d1.n_rows, d1.n_cols))
    reg = TGBMRegressor(depth=4, n_trees=5, learning_rate=0.5, verbose=0)
    # caller-made folds; predict() leaves the base score out, so the "RMSE" (a mean squared error) is large but finite
    folds = [(np.arange(0, 8000), np.arange(8000, 10000)), (np.arange(2000, 10000), np.arange(0, 2000))]
    res = reg.cv(X1, d1.y, folds=folds)
    assert np.isfinite(res['test-RMSE-mean']) and res['train-RMSE-std'] >= 0
    assert TGBMRanker(verbose=0).cv(X1, d1.y) is None


def test_cli_train_and_predict(gpu, tmp_path):
    """thundergbm-train <conf> writes ./tgbm.model; thundergbm-predict <conf> reads it and logs the metric."""
    import subprocess
    from thundergbm_b200 import synth
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = synth.dense_regression(2000, 8, seed=5)
    data = tmp_path / 'train.txt'
    with open(data, 'w') as fh:
        for i in range(d.n_rows):
            a, b = d.row_ptr[i], d.row_ptr[i + 1]
            fh.write(f'{d.y[i]:.9g} ' + ' '.join(f'{c + 1}:{v:.9g}' for c, v in zip(d.col[a:b], d.val[a:b])) + '\n')
    conf = tmp_path / 'run.conf'
    conf.write_text(f'data={data}\ndepth=4\nn_trees=5\nlearning_rate=0.5\nobjective=reg:linear\n')
    out = subprocess.run([os.path.join(root, 'thundergbm_b200', 'bin', 'thundergbm-train'), str(conf)], cwd=tmp_path,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert '[5/5] RMSE = ' in out.stdout and os.path.exists(tmp_path / 'tgbm.model')
    rmse_train = float(out.stdout.split('[5/5] RMSE = ')[1].split()[0])
    out2 = subprocess.run([os.path.join(root, 'thundergbm_b200', 'bin', 'thundergbm-predict'), str(conf)], cwd=tmp_path,
                          capture_output=True, text=True, timeout=300)
    assert out2.returncode == 0, out2.stderr
    rmse_pred = float(out2.stdout.split('RMSE = ')[1].split()[0])
    assert abs(rmse_pred - rmse_train) < 1e-4


def test_cli_text_loader_is_exact(gpu, tmp_path):
    """The LibSVM loader (threads + a fast path for short decimals) reads every spelling to the float atof gives:
    the trees trained from the text file equal the trees trained from the same values handed over as CSR."""
    import subprocess
    from thundergbm_b200 import synth
    from thundergbm_b200.booster import Booster
    from common import NODE_DTYPE
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = synth.dense_regression(60000, 8, seed=9)     # ~6 MB of text: parsed in several pieces
    spell = ['%.9g', '%.8e', '%+.9g', '%.17g', '%.9G']
    data = tmp_path / 'train.txt'
    with open(data, 'w') as fh:
        fh.write('# a comment line\n')
        for i in range(d.n_rows):
            a, b = d.row_ptr[i], d.row_ptr[i + 1]
            f = spell[i % len(spell)]
            fh.write((f % d.y[i]) + ' ' + ' '.join(f'{c + 1}:' + (f % v) for c, v in zip(d.col[a:b], d.val[a:b])))
            fh.write('  # trailing comment\n' if i % 97 == 0 else ('\r\n' if i % 89 == 0 else '\n'))
    conf = tmp_path / 'run.conf'
    conf.write_text(f'data={data}\ndepth=5\nn_trees=4\nlearning_rate=0.5\nobjective=reg:linear\n')
    out = subprocess.run([os.path.join(root, 'thundergbm_b200', 'bin', 'thundergbm-train'), str(conf)], cwd=tmp_path,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert f'#instances = {d.n_rows}' in out.stdout
    b = Booster(d, objective='reg:linear', depth=5, n_trees=4, learning_rate=0.5)
    b.boost(4)
    want = b.trees()
    b.close()
    # tail of the model file (src/thundergbm/parser.cpp:146-171): i32 rounds, then per round i32 trees and per tree
    # u64 nodes + the 48-byte node records
    raw = open(tmp_path / 'tgbm.model', 'rb').read()
    n_rounds, _, n_nodes = want.shape
    per_round = 4 + 8 + 48 * n_nodes
    tail = raw[len(raw) - (4 + n_rounds * per_round):]
    assert int.from_bytes(tail[:4], 'little') == n_rounds
    for r in range(n_rounds):
        rec = tail[4 + r * per_round: 4 + (r + 1) * per_round]
        assert int.from_bytes(rec[:4], 'little') == 1 and int.from_bytes(rec[4:12], 'little') == n_nodes
        assert rec[12:] == want[r, 0].tobytes(), f'tree {r} differs'



def test_metric_score_entry_point(gpu, orc, cases):
    """tgbm_metric_score on the raw training scores reproduces the per-round metric of training."""
    from thundergbm_b200 import _lib
    from thundergbm_b200.booster import Booster
    lib = _lib.lib()
    for name in ('c1_dense_reg', 'fixture_bin', 'c3_covtype_small', 'c5_mslr_small'):
        d, params = cases(name)
        kw = {k: v for k, v in params.items() if k != 'tree_method'}
        kw['n_trees'] = 2
        b = Booster(d, **kw)
        b.boost(2)
        raw = np.ascontiguousarray(b.ypred())
        o = orc.train(d, hist_mode=1, **kw)
        y = np.ascontiguousarray(d.y, np.float32)
        if o.labels.size:  # class index, as the library stores it
            y = np.searchsorted(o.labels, y).astype(np.float32)
        grp = np.ascontiguousarray(d.group, np.int32)
        out = C.c_float(0)
        rc = lib.tgbm_metric_score(params['objective'].encode(), d.n_rows, raw.shape[0], _vp(y), _vp(raw),
                                   _vp(grp) if grp.size else None, int(grp.size), C.byref(out))
        assert rc == 0, lib.tgbm_last_error()
        assert out.value == b.metrics()[-1], name
        b.close()


def test_released_buffers_are_kept_and_given_back_on_request(gpu, cases):
    """The library keeps the device buffers a call releases for the next call (a second training of the same shape
    allocates nothing) and tgbm_release_device_memory returns them to the driver; the trees do not depend on it."""
    import torch
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    d, _ = cases('c2_higgs_small')
    m0 = _train(lib, d, 'binary:logistic', depth=6, n_trees=3)[0]   # loads the kernels and whatever the driver keeps per context
    lib.model_free(C.byref(m0))
    lib.tgbm_release_device_memory()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    m1, _, per, _ = _train(lib, d, 'binary:logistic', depth=6, n_trees=3)
    free1, _ = torch.cuda.mem_get_info()
    m2, _, _, _ = _train(lib, d, 'binary:logistic', depth=6, n_trees=3)
    free2, _ = torch.cuda.mem_get_info()
    if not os.environ.get('TGBM_NO_POOL'):
        assert free1 < free0            # the first call's buffers stay with the library
        assert free2 == free1           # the second call found all of its buffers there
    lib.tgbm_release_device_memory()
    free3, _ = torch.cuda.mem_get_info()
    assert free3 > free1 or os.environ.get('TGBM_NO_POOL')
    assert free3 >= free0 - (8 << 20)   # everything is back
    n1, n2 = C.c_int(0), C.c_int(0)
    lib.get_n_nodes(C.byref(m1), C.byref(n1), 3, per)
    lib.get_n_nodes(C.byref(m2), C.byref(n2), 3, per)
    assert n1.value == n2.value
    lib.model_free(C.byref(m1)); lib.model_free(C.byref(m2))


def test_pageable_and_page_locked_arrays_give_the_same_model(gpu, monkeypatch):
    """Arrays of more than 32 MB in pageable memory travel through the library's own staging slots (several host threads,
    pieces of 8 MB, the last one ragged), page-locked ones through one cudaMemcpyAsync: same trees, same predictions."""
    import torch
    from thundergbm_b200 import _lib
    from thundergbm_b200.synth import CsrData
    lib = _lib.lib()
    monkeypatch.setenv('TGBM_HIST_MODE', 'exact')     # integer sums: the two runs must agree to the bit
    rng = np.random.default_rng(3)
    n, f = 1_250_003, 8                                # 40 MB of values, 40 MB of column indices, odd sizes
    x = rng.standard_normal((n, f)).astype(np.float32)
    y = (x[:, 0] * x[:, 1] + 0.1 * rng.standard_normal(n)).astype(np.float32)
    rp = (np.arange(n + 1, dtype=np.int64) * f).astype(np.int32)
    col = np.tile(np.arange(f, dtype=np.int32), n)
    d = CsrData(n, f, rp, col, x.reshape(-1), y, np.zeros(0, np.int32))

    def run(arrays):
        val, rp_, col_, y_ = arrays
        model = C.c_void_p(None); nc = C.c_int(1); per = C.c_int(0); gl = (C.c_float * 4)()
        lib.sparse_train_scikit(n, _vp(val), _vp(rp_), _vp(col_), _vp(y_), 5, 3, 1, 1.0, 1.0, 1.0, 64, 0, 1.0, 0, 1, 0.3,
                                b'reg:linear', C.byref(nc), b'hist', C.byref(model), C.byref(per), gl, None, 0)
        assert model.value, lib.tgbm_last_error().decode()
        out = np.zeros(n, np.float32)
        lib.sparse_predict_scikit(n, _vp(val), _vp(rp_), _vp(col_), _vp(out), C.byref(model), 3, 1, b'reg:linear', 1, 0.3,
                                  gl, None, 0, 0)
        lib.model_free(C.byref(model))
        return out

    pageable = (d.val, d.row_ptr, d.col, d.y)
    locked = tuple(torch.from_numpy(a).pin_memory().numpy() for a in pageable)
    a, b = run(pageable), run(locked)
    assert np.array_equal(a, b)
    assert np.std(a) > 0.1    # and the model learnt something from the data it was given
