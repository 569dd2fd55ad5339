"""Row sampling (bagging) and column sampling: the CUDA path against the CPU oracle on the same seeded inputs.

The reference's samplers draw from std::rand() and cannot be reproduced run to run (src/thundergbm/row_sampler.cu:17,
src/thundergbm/builder/shard.cu:13); both sides here draw from the same counter-based hash, so in the deterministic
mode the trees must be identical bit for bit, like everywhere else."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _booster(d, params, **extra):
    from thundergbm_b200.booster import Booster
    kw = {k: v for k, v in params.items() if k != 'tree_method'}
    kw.update(extra)
    return Booster(d, **kw)


@pytest.mark.parametrize('name', ['c1_dense_reg', 'fixture_bin', 'c3_covtype_small', 'c4_sparse_small', 'fixture_rank'])
@pytest.mark.parametrize('bagging,rate', [(1, 1.0), (0, 0.5), (1, 0.3)])
def test_sampling_bit_exact_with_oracle(gpu, orc, cases, name, bagging, rate):
    d, params = cases(name)
    p = {**params, 'n_trees': min(params['n_trees'], 5)}
    o = orc.train(d, hist_mode=1, keep_nid=1, bagging=bagging, column_sampling_rate=rate, sample_seed=7, **p)
    b = _booster(d, p, keep_nid=1, hist_mode='exact', bagging=bagging, column_sampling_rate=rate, sample_seed=7)
    b.boost(p['n_trees'])
    assert b.trees().tobytes() == o.trees.tobytes()
    assert np.array_equal(b.nid(), o.nid)
    assert np.array_equal(b.metrics(), o.metric)
    b.close()


def test_sampling_changes_the_trees_and_depends_on_the_seed(gpu, cases):
    d, params = cases('c1_dense_reg')
    p = {**params, 'n_trees': 3}
    out = {}
    for key, kw in {'plain': {}, 'bag7': dict(bagging=1, sample_seed=7), 'bag8': dict(bagging=1, sample_seed=8),
                    'col7': dict(column_sampling_rate=0.5, sample_seed=7)}.items():
        b = _booster(d, p, hist_mode='exact', **kw)
        b.boost(3)
        out[key] = b.trees()
        b.close()
    assert out['plain'].tobytes() != out['bag7'].tobytes() != out['bag8'].tobytes()
    assert out['plain'].tobytes() != out['col7'].tobytes()
    # Shard::column_sampling puts max(1, int(F * rate)) features into the IGNORED set: with 32 features and rate 0.5
    # a round's trees split on at most 16 different features
    for r in range(3):
        t = out['col7'][r, 0]
        used = set(t['split_feature_id'][(t['is_valid'] != 0) & (t['split_feature_id'] >= 0)].tolist())
        assert len(used) <= 16


def test_sampling_in_fp32_mode_trains(gpu, cases):
    d, params = cases('c2_higgs_small')
    b = _booster(d, {**params, 'n_trees': 8}, hist_mode='fp32', bagging=1, column_sampling_rate=0.25, sample_seed=3)
    b.boost(8)
    m = b.metrics()
    assert np.all(np.isfinite(m)) and m[-1] < m[0]
    b.close()
