"""Pins the CPU oracle to the reference: outputs of the reference itself run on a B200
(tests/golden/ref_*.npz, made by tests/golden/run_reference.sh + pack_golden.py) and the
known-answer tests of the reference's own suite."""
import hashlib

import numpy as np
import pytest

from common import compare_tree_decisive, load_golden

ALL = ['fixture_reg', 'fixture_bin', 'fixture_rank', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small',
       'c4_sparse_small', 'c5_mslr_small']


@pytest.mark.parametrize('name', ALL)
def test_cut_points_and_bin_ids_bit_exact(orc, cases, name):
    d, params = cases(name)
    g = load_golden(name)
    cut_val, cut_ptr, bins = orc.bin_only(d, params['max_num_bin'])
    assert np.array_equal(cut_ptr, g['cut_ptr'])
    assert cut_val.tobytes() == g['cut_val'].tobytes()          # bit-exact floats
    assert bins.size == int(g['n_bin_ids'])
    assert np.array_equal(bins[:4096], g['bins_head'])
    assert hashlib.sha256(bins.tobytes()).digest() == g['bins_sha256'].tobytes()


@pytest.mark.parametrize('name', ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small',
                                  'c4_sparse_small'])
@pytest.mark.parametrize('mode', [0, 1])
def test_training_matches_reference(orc, cases, name, mode):
    """mode 0: float accumulation in row order with libm expf (closest to the reference);
    mode 1: the exact fixed-point arithmetic of the CUDA path with the portable expf."""
    d, params = cases(name)
    g = load_golden(name)
    o = orc.train(d, hist_mode=mode, portable_exp=mode, n_threads=1, **params)
    assert o.trees.shape == g['trees'].shape
    assert o.num_class == int(g['num_class'])
    assert np.allclose(o.base_score, float(g['base_score']), rtol=1e-6, atol=1e-7)
    assert np.array_equal(o.labels, g['label'])
    # first tree: every decisive split identical; later trees inherit the reference's own run-to-run noise
    # (its histograms are unordered float atomics and exact gain ties are frequent in small nodes)
    same, bad = compare_tree_decisive(g['trees'][0, 0], o.trees[0, 0], o.gain2[0, 0])
    assert not bad, f'non-tie split differs at nodes {bad[:8]}'
    assert same >= 3
    root_r, root_o = g['trees'][0, 0][0], o.trees[0, 0][0]
    # The reference accumulates bins in float: 40k equal hessians summed one by one drift by ~3e-5 relative (every
    # addition rounds the same way).  Mode 0 reproduces that drift, the exact sums of mode 1 do not, so its gains sit
    # up to a few 1e-4 relative away from the reference's.
    assert np.allclose(root_o['gain'], root_r['gain'], rtol=1e-4 if mode == 0 else 1e-3)
    assert np.allclose(root_o['sum_h'], root_r['sum_h'], rtol=1e-5)
    # the reference's root sum is an unordered float reduction over all rows: compare against the summed magnitude
    assert abs(float(root_o['sum_g']) - float(root_r['sum_g'])) <= 1e-6 * d.n_rows + 1e-3
    # per-round training metric as logged by the reference (6 significant digits)
    ref_metric = g['metric']
    assert len(ref_metric) == params['n_trees']
    # mode 0 follows the reference to its printed digits until near-ties (see compare_tree_decisive) let the trees
    # drift; the fixed-point grid of mode 1 perturbs gains by ~1e-5 relative, which decides near-ties differently
    chaotic = mode == 1 or name in ('c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small')
    assert abs(float(o.metric[0]) - float(ref_metric[0])) <= (5e-3 if mode == 1 else 2e-4)
    if not (mode == 1 and name == 'fixture_reg'):
        # (fixture_reg at learning rate 1 stalls once a tree prunes back to its root; the round in which that
        # happens is decided by near-ties, so its final value is not comparable across arithmetics)
        assert abs(float(o.metric[-1]) - float(ref_metric[-1])) <= (5e-3 if chaotic else 5e-4)


def test_readme_rmse_of_current_revision(orc, cases):
    """thundergbm-train on dataset/machine.conf logs RMSE = 0.528422 for this revision of the reference
    (its README's 0.489562 predates the base-score initialisation); the oracle reproduces both."""
    d, params = cases('fixture_reg')
    o = orc.train(d, hist_mode=0, portable_exp=0, n_threads=1, **params)
    assert abs(float(o.metric[-1]) - 0.528422) < 2e-6


@pytest.mark.parametrize('name', ['fixture_reg', 'fixture_bin', 'c1_dense_reg'])
def test_predict_raw_matches_reference(orc, cases, name):
    """Predictor::predict_raw of the reference on the reference's own model file."""
    d, params = cases(name)
    g = load_golden(name)
    raw = orc.predict_raw(d, g['trees'], float(g['learning_rate']), float(g['base_score']))
    ref = g['raw_pred_sample']
    assert np.allclose(raw.reshape(-1)[::37], ref, rtol=2e-6, atol=2e-6)


def test_rank_objectives_run_and_score(orc, cases):
    """The reference's LambdaRank sampling is seeded from std::rand() per OpenMP thread, so only the level of its
    NDCG can be pinned."""
    for name in ('fixture_rank', 'c5_mslr_small'):
        d, params = cases(name)
        g = load_golden(name)
        o = orc.train(d, hist_mode=1, n_threads=1, **params)
        assert 0.0 < o.metric[-1] <= 1.0
        assert abs(float(o.metric[-1]) - float(g['metric'][-1])) < 0.05


# ---- known-answer tests of the reference's own suite -------------------------------------------------------------
def test_reference_dataset_known_answers(cases):
    d, _ = cases('fixture_reg')      # src/test/test_dataset.cpp:178-181
    assert d.n_rows == 1605 and d.n_cols == 119
    assert d.y[0] == -1 and d.val[1] == 1
    assert d.group.tolist() == [100, 300, 400, 200, 605]


def test_reference_tree_known_answer(orc, cases):
    d, params = cases('fixture_reg')  # src/test/test_tree.cpp:68 -- depth 6 -> 127 nodes
    o = orc.train(d, **{**params, 'n_trees': 1})
    assert o.n_nodes == 127 and o.trees.shape[-1] == 127


def test_reference_metric_known_answers(orc, cases):
    """src/test/test_metrics.cpp:70,84,96: zeros against the fixture's -1/+1 labels give RMSE 1."""
    d, _ = cases('fixture_reg')
    e = np.zeros(d.n_rows, np.float32) - d.y
    assert np.sqrt(np.float32((e * e).sum(dtype=np.float64)) / d.n_rows) == 1.0
    o = orc.train(d, objective='reg:linear', depth=1, n_trees=1, learning_rate=0.0, hist_mode=0, portable_exp=0)
    # with learning rate 0 the scores stay at the base score = mean(y)
    assert np.allclose(o.metric[0], np.sqrt(np.mean((d.y - d.y.mean()) ** 2)), rtol=1e-6)


def test_portable_expf_accuracy(orc):
    x = np.linspace(-87, 88, 200001).astype(np.float32)
    l = orc.lib()
    got = np.array([l.tgo_portable_expf(float(v)) for v in x[::97]], np.float32)
    want = np.exp(x[::97].astype(np.float64))
    rel = np.abs(got.astype(np.float64) - want) / want
    assert rel.max() < 2.5e-7


def test_exact_mode_is_thread_count_invariant(orc, cases):
    d, params = cases('c2_higgs_small')
    p = {**params, 'n_trees': 3}
    a = orc.train(d, hist_mode=1, n_threads=1, **p)
    b = orc.train(d, hist_mode=1, n_threads=4, **p)
    assert a.trees.tobytes() == b.trees.tobytes() and np.array_equal(a.ypred, b.ypred)


def test_oracle_sampling_restatement(orc, cases):
    """Bagging multiplies every gradient by its multiplicity in a bootstrap sample of the gradient array
    (src/thundergbm/row_sampler.cu:9-35); column sampling leaves max(1, int(F * rate)) features out of the split search
    for a round (src/thundergbm/builder/shard.cu:8-23).  Same seed, same trees; another seed, other trees."""
    d, params = cases('c1_dense_reg')
    p = {**params, 'n_trees': 3}
    plain = orc.train(d, **p)
    a = orc.train(d, bagging=1, column_sampling_rate=0.5, sample_seed=5, **p)
    b = orc.train(d, bagging=1, column_sampling_rate=0.5, sample_seed=5, **p)
    c = orc.train(d, bagging=1, column_sampling_rate=0.5, sample_seed=6, **p)
    assert a.trees.tobytes() == b.trees.tobytes() != c.trees.tobytes()
    assert a.trees.tobytes() != plain.trees.tobytes()
    for r in range(3):
        t = a.trees[r, 0]
        used = set(t['split_feature_id'][(t['is_valid'] != 0) & (t['split_feature_id'] >= 0)].tolist())
        assert 1 <= len(used) <= 16          # 32 features, half of them ignored in every round
    # the root of a bagged tree sums multiplicity-weighted hessians: reg:linear has h = 1, so sum_h = number of draws kept
    assert abs(float(a.trees[0, 0][0]['sum_h']) - d.n_rows) < 5 * np.sqrt(d.n_rows)


MULTI = ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small']


@pytest.mark.parametrize('name', MULTI)
def test_column_sharded_builder_cut_points_and_bins(orc, cases, name):
    """The restatement of the reference's column-sharded builder (n_device = 2) against the reference's own cut points
    (per device, descending inside a feature, shifted and re-rounded values) and bin ids: bit for bit."""
    d, params = cases(name)
    g = load_golden('multi_' + name)
    shards = int(g['n_device'])
    cut_val, cut_ptr, bins = orc.bin_only(d, params['max_num_bin'], multi_shards=shards)
    assert np.array_equal(cut_ptr, g['cut_ptr'])
    assert cut_val.tobytes() == g['cut_val'].tobytes()
    assert bins.size == int(g['n_bin_ids'])
    assert np.array_equal(bins[:4096], g['bins_head'])
    assert hashlib.sha256(bins.tobytes()).digest() == g['bins_sha256'].tobytes()


@pytest.mark.parametrize('name', MULTI)
def test_column_sharded_builder_training_matches_reference(orc, cases, name):
    """fp32 arithmetic of the oracle, column-sharded rules, against the reference's two-device run: the first tree
    splits identically wherever the split is decisive, the logged metric follows."""
    d, params = cases(name)
    g = load_golden('multi_' + name)
    o = orc.train(d, hist_mode=0, portable_exp=0, n_threads=1, multi_shards=int(g['n_device']), **params)
    assert o.trees.shape == g['trees'].shape
    assert np.allclose(o.base_score, float(g['base_score']), rtol=1e-6, atol=1e-7)
    same, bad = compare_tree_decisive(g['trees'][0, 0], o.trees[0, 0], o.gain2[0, 0])
    assert not bad, f'non-tie split differs at nodes {bad[:8]}'
    assert same >= 3
    root_r, root_o = g['trees'][0, 0][0], o.trees[0, 0][0]
    assert root_o['split_feature_id'] == root_r['split_feature_id'] and root_o['split_bid'] == root_r['split_bid']
    assert root_o['split_value'].tobytes() == root_r['split_value'].tobytes()      # the cut point itself
    # this builder of the reference adds up per-block partial histograms (hist_tree_builder.cu:129-168), the oracle's
    # float mode one running sum per bin: the drift of the two orders differs, and a gain is a small difference of
    # large terms (covtype's root: 44.8 out of terms near 2e4)
    assert np.allclose(root_o['gain'], root_r['gain'], rtol=1e-3)
    # two runs of the reference itself sit spread_metric apart
    tol = 2 * float(g['spread_metric'])
    assert abs(float(o.metric[0]) - float(g['metric'][0])) <= max(2e-4, tol)
    assert abs(float(o.metric[-1]) - float(g['metric'][-1])) <= max(5e-3, tol)


EXACT = ['fixture_reg', 'fixture_bin', 'c1_dense_reg', 'c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small']


@pytest.mark.parametrize('name', EXACT)
def test_exact_builder_training_matches_reference(orc, cases, name):
    """The restatement of ExactTreeBuilder (tree_method=exact) against the reference's own exact runs (which repeat bit for
    bit: three runs, no spread): first tree identical at every decisive split, split values bit for bit along the
    way, the logged metric follows."""
    d, params = cases(name)
    g = load_golden('exact_' + name)
    o = orc.train(d, hist_mode=0, portable_exp=0, n_threads=1, **{**params, 'tree_method': 'exact'})
    assert o.trees.shape == g['trees'].shape
    assert np.allclose(o.base_score, float(g['base_score']), rtol=1e-6, atol=1e-7)
    ref, mine = g['trees'][0, 0], o.trees[0, 0]
    # a gain is a small difference of large terms and the two sides add in different orders (covtype's root: 44.8 out of
    # terms near 2e4 moves by 2e-4 relative): splits whose runner-up is closer than 1e-3 count as ties
    same, bad = compare_tree_decisive(ref, mine, o.gain2[0, 0], rel_margin=1e-3, min_child_weight=params['min_child_weight'])
    assert not bad, f'non-tie split differs at nodes {bad[:8]}'
    assert same >= 3
    assert mine[0]['split_feature_id'] == ref[0]['split_feature_id']
    assert mine[0]['split_value'].tobytes() == ref[0]['split_value'].tobytes()
    assert np.allclose(mine[0]['gain'], ref[0]['gain'], rtol=1e-3)
    chaotic = name in ('c2_higgs_small', 'c3_covtype_small', 'c4_sparse_small')
    # (covtype: one node of the first tree sits on the min_child_weight threshold, 22 of 100000 rows end up elsewhere)
    assert abs(float(o.metric[0]) - float(g['metric'][0])) <= (5e-4 if chaotic else 2e-4)
    assert abs(float(o.metric[-1]) - float(g['metric'][-1])) <= (5e-3 if chaotic else 5e-4)
