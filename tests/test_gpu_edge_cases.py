"""Edge cases of the inputs: ragged and empty rows, constant and absent features, tiny data, extreme parameters."""
import numpy as np
import pytest

from thundergbm_b200 import synth

pytestmark = pytest.mark.gpu


def _pair(orc, d, **p):
    from thundergbm_b200.booster import Booster
    o = orc.train(d, hist_mode=1, keep_nid=1, **p)
    b = Booster(d, keep_nid=1, **p)
    b.boost(p['n_trees'])
    return o, b


def _rand_csr(n, f, density, seed, n_values=None):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, f)).astype(np.float32)
    if n_values:
        x = np.round(x * n_values / 4).astype(np.float32)
    x[rng.random((n, f)) > density] = 0
    y = (x[:, 0] - x[:, 1 % f] + 0.3 * rng.standard_normal(n)).astype(np.float32)
    return synth.dense_to_csr(x, y)


@pytest.mark.parametrize('n,f,density', [(1, 3, 1.0), (2, 1, 1.0), (33, 5, 0.5), (1000, 40, 0.3), (5000, 70, 0.9),
                                         (1023, 33, 0.7), (1025, 31, 1.0)])
def test_ragged_shapes(gpu, orc, n, f, density):
    d = _rand_csr(n, f, density, seed=n + f)
    if d.nnz == 0:
        d = _rand_csr(n, f, 1.0, seed=n + f + 1)
    p = dict(objective='reg:linear', depth=4, n_trees=3, max_num_bin=255, learning_rate=0.5)
    o, b = _pair(orc, d, **p)
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid) and np.array_equal(b.ypred(), o.ypred)
    b.close()


def test_empty_rows_and_absent_features(gpu, orc):
    d = _rand_csr(3000, 12, 0.4, seed=7)
    # rows 10..19 empty, feature 5 never present, feature 11 constant
    x = np.zeros((3000, 12), np.float32)
    rows = np.repeat(np.arange(3000), np.diff(d.row_ptr))
    x[rows, d.col] = d.val
    x[10:20] = 0
    x[:, 5] = 0
    x[:, 11] = 3.5
    d2 = synth.dense_to_csr(x, d.y)
    p = dict(objective='reg:linear', depth=5, n_trees=4, max_num_bin=255, learning_rate=0.3)
    o, b = _pair(orc, d2, **p)
    assert b.trees().tobytes() == o.trees.tobytes() and np.array_equal(b.ypred(), o.ypred)
    cp = b.cuts()[1]
    assert cp[6] - cp[5] == 0 and cp[12] - cp[11] == 1
    b.close()


@pytest.mark.parametrize('max_bin', [2, 16, 64, 255])
def test_small_bin_budgets(gpu, orc, max_bin):
    d = _rand_csr(4000, 9, 1.0, seed=max_bin)
    p = dict(objective='reg:linear', depth=5, n_trees=3, max_num_bin=max_bin, learning_rate=0.5)
    o, b = _pair(orc, d, **p)
    assert b.info.n_bins == o.n_bins
    assert b.trees().tobytes() == o.trees.tobytes()
    b.close()


def test_low_cardinality_collisions(gpu, orc):
    """Few distinct values per feature: many rows hit the same bins (shared-memory atomics on one address)."""
    d = _rand_csr(20000, 8, 1.0, seed=3, n_values=3)
    p = dict(objective='binary:logistic', depth=6, n_trees=4, max_num_bin=255, learning_rate=0.3)
    d.y = (d.y > 0).astype(np.float32)
    o, b = _pair(orc, d, **p)
    assert b.trees().tobytes() == o.trees.tobytes() and np.array_equal(b.nid(), o.nid)
    b.close()


@pytest.mark.parametrize('depth', [1, 2, 10, 12, 14])
def test_depth_extremes(gpu, orc, depth):
    """Depth 14 is the limit; its node table no longer fits the shared memory of the kernel that applies a tree."""
    d = _rand_csr(6000, 6, 1.0, seed=depth)
    p = dict(objective='reg:linear', depth=depth, n_trees=2, max_num_bin=64, learning_rate=0.5, gamma=0.0)
    o, b = _pair(orc, d, **p)
    assert b.trees().tobytes() == o.trees.tobytes() and np.array_equal(b.ypred(), o.ypred)
    b.close()


@pytest.mark.parametrize('n,f,density', [(1, 3, 1.0), (33, 5, 0.5), (1025, 31, 1.0), (3000, 300, 0.05), (5000, 70, 0.9)])
def test_csr_layout_ragged_shapes(gpu, orc, n, f, density, monkeypatch):
    """The same ragged inputs through the CSR-of-bin-ids layout, with some rows emptied."""
    monkeypatch.setenv('TGBM_LAYOUT', 'sparse')
    d = _rand_csr(n, f, density, seed=n + f)
    if d.nnz == 0:
        d = _rand_csr(n, f, 1.0, seed=n + f + 1)
    p = dict(objective='reg:linear', depth=5, n_trees=3, max_num_bin=255, learning_rate=0.5)
    o, b = _pair(orc, d, **p)
    assert b.info.csr_layout == 1
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid) and np.array_equal(b.ypred(), o.ypred)
    b.close()


def test_csr_layout_many_bins_per_feature(gpu, orc, monkeypatch):
    """Features with 255 bins each: every evaluation chunk holds one feature; 60 features = 15k bins, more than the
    shared-memory part of the sparse histogram (12288 bins)."""
    monkeypatch.setenv('TGBM_LAYOUT', 'sparse')
    d = _rand_csr(20000, 60, 0.6, seed=11)
    p = dict(objective='reg:linear', depth=6, n_trees=3, max_num_bin=255, learning_rate=0.3)
    o, b = _pair(orc, d, **p)
    assert b.info.csr_layout == 1 and b.info.n_bins > 12288
    assert b.trees().tobytes() == o.trees.tobytes() and np.array_equal(b.ypred(), o.ypred)
    b.close()


def test_accumulator_window_flush(gpu, orc):
    """More rows per CTA than one int32 accumulation window holds (quant_bits 20 -> a window of one 1024-row tile)."""
    d = synth.higgs_like(300_000, seed=5)
    p = dict(objective='binary:logistic', depth=3, n_trees=2, max_num_bin=255, learning_rate=0.1, quant_bits=20)
    o, b = _pair(orc, d, **p)
    assert b.trees().tobytes() == o.trees.tobytes()
    b.close()


def test_rejects_what_is_out_of_scope(gpu):
    from thundergbm_b200.booster import Booster
    d = _rand_csr(100, 4, 1.0, seed=1)
    with pytest.raises(RuntimeError, match='max_num_bin'):
        Booster(d, objective='reg:linear', depth=3, n_trees=1, max_num_bin=300)
    with pytest.raises(RuntimeError, match='objective'):
        Booster(d, objective='reg:nope', depth=3, n_trees=1)
    with pytest.raises(RuntimeError, match='depth'):
        Booster(d, objective='reg:linear', depth=0, n_trees=1)


def test_full_size_properties(gpu):
    """Size-independent properties at a multi-million-row size: every feature's root histogram sums to the root
    total, every row ends in exactly one valid leaf, the error rate falls."""
    from thundergbm_b200.booster import Booster
    d = synth.higgs_like(2_000_000, seed=9)
    b = Booster(d, objective='binary:logistic', depth=8, n_trees=4, max_num_bin=255, learning_rate=0.1, keep_nid=1)
    b.boost(4)
    t = b.trees()
    nid = b.nid()
    for r in range(4):
        nodes = t[r, 0]
        leaf = nodes[nid[r]]
        assert (leaf['is_valid'] == 1).all() and (leaf['is_leaf'] == 1).all()
        # row counts per leaf add up
        assert np.bincount(nid[r], minlength=len(nodes)).sum() == d.n_rows
        # children sums add up to the parent within float rounding
        inner = np.nonzero((nodes['is_valid'] == 1) & (nodes['lch_index'] > 0) & (nodes['gain'] > 0) & (nodes['split_feature_id'] >= 0))[0]
        for i in inner[:50]:
            l, rr = nodes[nodes[i]['lch_index']], nodes[nodes[i]['rch_index']]
            if l['is_valid'] and rr['is_valid']:
                assert abs((l['sum_h'] + rr['sum_h']) - nodes[i]['sum_h']) <= 1e-5 * nodes[i]['sum_h'] + 1e-3
    m = b.metrics()
    assert m[-1] < m[0] + 1e-6
    b.close()


@pytest.mark.parametrize('n_features', [12, 40, 300])
def test_predict_raw_special_values(gpu, orc, n_features):
    """predict_raw on values that sit exactly on thresholds, on -0.0 / +0.0, on +-inf and NaN, on absent features and on
    features the model never saw -- for the reference's dense arithmetic (F * 128 * 4 <= 48 KB: double sums, +inf means
    absent) and its CSR arithmetic (float sums, fused multiply-add).  Bit-identical to the oracle."""
    from thundergbm_b200.booster import Booster, predict_raw
    from thundergbm_b200.synth import dense_to_csr
    rng = np.random.default_rng(n_features)
    n = 3000
    x = rng.standard_normal((n, n_features)).astype(np.float32)
    x[rng.random(x.shape) < 0.3] = 0.0                       # dropped by the CSR conversion: absent
    y = (x[:, 0] + 0.5 * x[:, 1] * x[:, 2] + 0.1 * rng.standard_normal(n)).astype(np.float32)
    d = dense_to_csr(x, y)
    b = Booster(d, objective='reg:linear', depth=5, n_trees=12, learning_rate=0.3, max_num_bin=32)
    b.boost(12)
    trees, base = b.trees(), b.info.base_score
    b.close()
    # test rows: every threshold of the model, its float neighbours, and the special values, in random columns
    thr = trees['split_value'][(trees['is_valid'] != 0) & (trees['is_leaf'] == 0)]
    pool = np.concatenate([thr, np.nextafter(thr, np.float32(np.inf)), np.nextafter(thr, np.float32(-np.inf)),
                           np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e30, -1e30], np.float32)]).astype(np.float32)
    m = 5000
    xt = pool[rng.integers(0, pool.size, (m, n_features + 3))]   # three more columns than the model was trained on
    keep = rng.random(xt.shape) < 0.7
    rows, cols = np.nonzero(keep)
    from thundergbm_b200.synth import CsrData
    rp = np.zeros(m + 1, np.int32)
    np.cumsum(keep.sum(1), out=rp[1:])
    dt = CsrData(m, n_features + 3, rp, cols.astype(np.int32), xt[rows, cols].astype(np.float32), np.zeros(m, np.float32))
    got = predict_raw(dt, trees, 0.3, base)
    want = orc.predict_raw(dt, trees, 0.3, base, n_features=n_features + 3)
    assert np.array_equal(got, want)


@pytest.mark.parametrize('shuffle', [False, True])
def test_predict_raw_dense_rows(gpu, orc, shuffle):
    """A dense matrix handed over as CSR (every row stores all 28 features) takes the one-thread-per-row conversion to
    threshold ranks; a row whose columns are not 0 .. F-1 in order sends the whole call back to the general kernel.
    Values on thresholds, their float neighbours, zeros of both signs, +-inf and NaN included.  Bit-identical to the
    oracle either way."""
    from thundergbm_b200.booster import Booster, predict_raw
    from thundergbm_b200.synth import CsrData, higgs_like
    d = higgs_like(20_000, seed=5)
    b = Booster(d, objective='binary:logistic', depth=8, n_trees=10, learning_rate=0.3, max_num_bin=255)
    b.boost(10)
    trees, base = b.trees(), b.info.base_score
    b.close()
    F = d.n_cols
    rng = np.random.default_rng(17)
    thr = trees['split_value'][(trees['is_valid'] != 0) & (trees['is_leaf'] == 0)]
    pool = np.concatenate([thr, np.nextafter(thr, np.float32(np.inf)), np.nextafter(thr, np.float32(-np.inf)),
                           np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e30, -1e30], np.float32)]).astype(np.float32)
    m = 6001
    x = d.val[:m * F].reshape(m, F).copy()
    special = rng.random(x.shape) < 0.2
    x[special] = pool[rng.integers(0, pool.size, int(special.sum()))]
    cols = np.tile(np.arange(F, dtype=np.int32), m).reshape(m, F)
    rp = (np.arange(m + 1) * F).astype(np.int32)
    ordered = CsrData(m, F, rp, cols.reshape(-1).copy(), x.reshape(-1).astype(np.float32), np.zeros(m, np.float32))
    want = orc.predict_raw(ordered, trees, 0.3, base, n_features=F)   # (the oracle looks columns up by binary search)
    if shuffle:                                   # the same data with two entries of one row stored the other way round
        cols[m // 2, [3, 11]] = cols[m // 2, [11, 3]]
        x[m // 2, [3, 11]] = x[m // 2, [11, 3]]
    dt = CsrData(m, F, rp, cols.reshape(-1), x.reshape(-1).astype(np.float32), np.zeros(m, np.float32))
    got = predict_raw(dt, trees, 0.3, base)
    assert np.array_equal(got, want)
