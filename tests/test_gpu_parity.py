"""CUDA path against the CPU oracle on the same seeded inputs, through the C ABI.

Integer, byte and index results (cut points, bin matrix, histograms, row->node partition, tree topology) and, because
all histogram sums are exact integers on a fixed-point grid, also every float derived from them (gains, leaf values,
raw scores) are compared bit for bit with the oracle's exact mode."""
import numpy as np
import pytest

from common import load_golden

pytestmark = pytest.mark.gpu

ALL = ['fixture_reg', 'fixture_bin', 'fixture_rank', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small',
       'c4_sparse_small', 'c5_mslr_small']


def _booster(d, params, **extra):
    from thundergbm_b200.booster import Booster
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw.update(extra)
    return Booster(d, **kw)


@pytest.mark.parametrize('name', ALL)
def test_cuts_and_bins_bit_exact(gpu, orc, cases, name):
    d, params = cases(name)
    b = _booster(d, params)
    cut_val, cut_ptr, bins = orc.bin_only(d, params['max_num_bin'])
    cv, cp = b.cuts()
    assert np.array_equal(cp, cut_ptr)
    assert cv.tobytes() == cut_val.tobytes()
    if b.info.csr_layout:
        assert name == 'c4_sparse_small'
        assert np.array_equal(b.bins_csr(d.nnz), bins)
    else:
        assert np.array_equal(b.bins(), orc.bins_to_dense(d, bins, cut_ptr, b.info.fpad))
    # and against what the reference itself produced
    g = load_golden(name)
    assert cv.tobytes() == g['cut_val'].tobytes() and np.array_equal(cp, g['cut_ptr'])
    b.close()


@pytest.mark.parametrize('name', ALL)
def test_training_bit_exact_with_oracle(gpu, orc, cases, name):
    d, params = cases(name)
    o = orc.train(d, hist_mode=1, keep_nid=1, **params)
    b = _booster(d, params, keep_nid=1)
    assert b.info.base_score == o.base_score
    b.boost(params['n_trees'])
    b.sync()
    assert np.array_equal(b.quant_scale(), o.quant_scale)
    trees = b.trees()
    assert trees.shape == o.trees.shape
    for r in range(trees.shape[0]):
        for k in range(trees.shape[1]):
            assert trees[r, k].tobytes() == o.trees[r, k].tobytes(), f'tree {r}/{k} differs'
    assert np.array_equal(b.nid(), o.nid)            # ins2node partition of every tree
    assert np.array_equal(b.ypred(), o.ypred)        # raw training scores
    assert np.array_equal(b.metrics(), o.metric)
    b.close()


@pytest.mark.parametrize('name', ['fixture_reg', 'fixture_rank', 'c2_higgs_small', 'c3_covtype_small', 'c5_mslr_small'])
def test_csr_layout_forced_on_dense_data(gpu, orc, cases, name, monkeypatch):
    """The CSR-of-bin-ids layout (chosen by itself only for wide sparse data) gives the same bits as the dense one."""
    monkeypatch.setenv('TGBM_LAYOUT', 'sparse')
    d, params = cases(name)
    p = {**params, 'n_trees': min(params['n_trees'], 8)}
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = _booster(d, p, keep_nid=1)
    assert b.info.csr_layout == 1
    b.boost(p['n_trees'])
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid)
    assert np.array_equal(b.metrics(), o.metric)
    assert np.array_equal(b.bins_csr(d.nnz), orc.bin_only(d, p['max_num_bin'])[2])
    b.close()


def test_csr_layout_unordered_columns(gpu, orc, cases):
    """Rows whose columns arrive in arbitrary order train to the same trees (the bin ids are sorted per row at set-up)."""
    from thundergbm_b200.synth import CsrData
    d, params = cases('c4_sparse_small')
    p = {**params, 'n_trees': 4}
    rng = np.random.default_rng(5)
    rows = np.repeat(np.arange(d.n_rows), np.diff(d.row_ptr))
    order = np.lexsort((rng.random(d.nnz), rows))              # shuffle inside every row
    ds = CsrData(d.n_rows, d.n_cols, d.row_ptr.copy(), d.col[order].copy(), d.val[order].copy(), d.y)
    a = _booster(d, p); a.boost(4)
    b = _booster(ds, p); b.boost(4)
    assert b.info.csr_layout == 1
    assert a.trees().tobytes() == b.trees().tobytes()
    assert np.array_equal(a.bins_csr(d.nnz), b.bins_csr(d.nnz))
    a.close(); b.close()


@pytest.mark.parametrize('name', ['fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small'])
def test_metric_against_reference_run(gpu, cases, name):
    """Tolerance 5e-3 on the logged training metric: the reference's own float-atomic noise and exact gain ties let
    trees drift after the first rounds (two runs of the reference differ from tree 2 on)."""
    d, params = cases(name)
    g = load_golden(name)
    b = _booster(d, params)
    b.boost(params['n_trees'])
    m = b.metrics()
    assert abs(float(m[0]) - float(g['metric'][0])) <= 5e-3
    assert abs(float(m[-1]) - float(g['metric'][-1])) <= 5e-3
    b.close()


def test_root_histogram_against_oracle(gpu, orc, cases):
    d, params = cases('c2_higgs_small')
    p = {**params, 'n_trees': 1, 'depth': 1}
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = _booster(d, p)
    b.boost(1)
    h = b.root_hist().astype(np.float64)
    sg, sh = o.quant_scale[0]
    want = o.hist_dump.reshape(-1, 2)[:b.info.n_bins]
    assert np.array_equal((h[:, 0] / sg).astype(np.float32), want[:, 0])
    assert np.array_equal((h[:, 1] / sh).astype(np.float32), want[:, 1])
    # size-independent property: every feature's bins add up to the same total when no value is missing
    cp = b.cuts()[1]
    tot = np.add.reduceat(b.root_hist(), cp[:-1], axis=0)
    assert (tot == tot[0]).all()
    b.close()


@pytest.mark.parametrize('bits', [12, 16, 20])
def test_quant_bits_variants(gpu, orc, cases, bits):
    d, params = cases('c1_dense_reg')
    p = {**params, 'n_trees': 5}
    o = orc.train(d, hist_mode=1, quant_bits=bits, **p)
    b = _booster(d, p, quant_bits=bits)
    b.boost(5)
    assert b.trees().tobytes() == o.trees.tobytes()
    b.close()


def test_two_runs_identical(gpu, cases):
    d, params = cases('c2_higgs_small')
    outs = []
    for _ in range(2):
        b = _booster(d, {**params, 'n_trees': 6})
        b.boost(6)
        outs.append((b.trees().tobytes(), b.ypred().tobytes()))
        b.close()
    assert outs[0] == outs[1]


def test_boost_in_pieces_equals_one_call(gpu, cases):
    d, params = cases('c1_dense_reg')
    a = _booster(d, {**params, 'n_trees': 6}); a.boost(6)
    b = _booster(d, {**params, 'n_trees': 6}); b.boost(2); b.boost(3); b.boost(1)
    assert a.trees().tobytes() == b.trees().tobytes()
    a.close(); b.close()


def test_graph_replay_and_plain_launches_mix(gpu, cases, monkeypatch):
    """Rounds replayed as a CUDA graph, rounds launched kernel by kernel (profiling on, or TGBM_NO_GRAPH) and any mix of
    the two give the same trees and the same per-round metrics."""
    d, params = cases('c2_higgs_small')
    p = {**params, 'n_trees': 9}
    a = _booster(d, p); a.boost(9)
    b = _booster(d, p)
    b.boost(3); b.set_profile(True); b.boost(2); b.set_profile(False); b.boost(3); b.set_profile(True); b.boost(1)
    prof = b.profile()
    assert prof.hist_launches == 3 * p['depth'] and prof.hist_ms > 0
    monkeypatch.setenv('TGBM_NO_GRAPH', '1')
    c = _booster(d, p); c.boost(9)
    assert a.trees().tobytes() == b.trees().tobytes() == c.trees().tobytes()
    assert np.array_equal(a.metrics(), b.metrics()) and np.array_equal(a.metrics(), c.metrics())
    assert np.array_equal(a.quant_scale(), b.quant_scale())
    a.close(); b.close(); c.close()


def test_predict_raw_against_oracle(gpu, orc, cases):
    for name in ('c1_dense_reg', 'c3_covtype_small', 'c5_mslr_small', 'c4_sparse_small'):
        from thundergbm_b200.booster import predict_raw
        d, params = cases(name)
        o = orc.train(d, hist_mode=1, **{**params, 'n_trees': 3})
        got = predict_raw(d, o.trees, params['learning_rate'], o.base_score)
        want = orc.predict_raw(d, o.trees, params['learning_rate'], o.base_score, n_features=d.n_cols)
        assert np.array_equal(got, want), name
        # on the dense path the training scores are reproduced up to float rounding of the double accumulator
        assert np.allclose(got, o.ypred, rtol=1e-5, atol=1e-5)


def test_predict_raw_reference_model(gpu, cases):
    """Our predictor on the reference's own model file reproduces the reference's raw predictions."""
    from thundergbm_b200.booster import predict_raw
    for name in ('fixture_reg', 'fixture_bin', 'c1_dense_reg'):
        d, params = cases(name)
        g = load_golden(name)
        got = predict_raw(d, g['trees'], float(g['learning_rate']), float(g['base_score']))
        assert np.allclose(got.reshape(-1)[::37], g['raw_pred_sample'], rtol=2e-6, atol=2e-6)
