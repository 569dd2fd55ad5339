"""tgbm_metric_score_noalloc -- the metric entry point for hosts that may not allocate device memory (their own
pool owns the GPU, or they run inside someone else's step loop where cudaMalloc's device-wide synchronisation is not
acceptable).  Inputs and output are device buffers of the caller; the reduction scratch is a fixed array inside the
library.  Checked through the C ABI against the allocating entry point tgbm_metric_score (same kernels, same grid, so
the two floats must be identical) AND against the metric computed with NumPy from the same arrays, on two calls in a
row (the second call finds the scratch dirty)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _existing(lib, objective, y, raw):
    out = C.c_float(0)
    rc = lib.tgbm_metric_score(objective.encode(), y.size, raw.shape[0], y.ctypes.data_as(C.c_void_p),
                               raw.ctypes.data_as(C.c_void_p), None, 0, C.byref(out))
    assert rc == 0, lib.tgbm_last_error()
    return out.value


def _numpy_metric(objective, y, raw):
    """RMSE, binary error or multi-class accuracy as the reference defines them (pointwise_metric.cu:8-22,
    multiclass_metric.cu:9-46), in float64."""
    if objective == 'reg:linear':
        return float(np.sqrt(np.mean((raw[0].astype(np.float64) - y) ** 2)))
    if objective == 'binary:logistic':
        return float(1.0 - np.mean((raw[0] > 0).astype(np.float32) == y))
    return float(np.mean(np.argmax(raw, axis=0).astype(np.float32) == y))


@pytest.mark.parametrize('objective,k', [('reg:linear', 1), ('binary:logistic', 1), ('multi:softmax', 5)])
def test_noalloc_matches_allocating_entry_point_twice(gpu, objective, k):
    import torch
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(7)
    results = []
    for n in (300_001, 4_097):            # two calls in a row, different sizes: the second sees the first's leftovers
        if objective == 'reg:linear':
            y = rng.standard_normal(n).astype(np.float32)
        else:
            y = rng.integers(0, max(2, k), n).astype(np.float32)
        raw = np.ascontiguousarray(rng.standard_normal((k, n)).astype(np.float32))
        want = _existing(lib, objective, y, raw)
        d_y, d_raw = torch.from_numpy(y).cuda(), torch.from_numpy(raw).cuda()
        d_out = torch.full((1,), -123.0, device='cuda')
        torch.cuda.synchronize()
        rc = lib.tgbm_metric_score_noalloc(objective.encode(), n, k, d_y.data_ptr(), d_raw.data_ptr(), d_out.data_ptr(), None)
        assert rc == 0, lib.tgbm_last_error()
        torch.cuda.synchronize()
        got = float(d_out.cpu()[0])
        assert got == want, (objective, n, got, want)
        assert abs(got - _numpy_metric(objective, y, raw)) <= 1e-6, (objective, n, got)   # float result of an fp64 sum
        results.append(got)
    assert all(np.isfinite(results))


def test_noalloc_takes_no_device_memory_and_honours_the_stream(gpu):
    """What the entry point exists for: after the first call on the device (which only looks the scratch address up)
    a call on a caller's stream leaves the amount of free device memory exactly as it found it."""
    import torch
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(11)
    n = 200_003
    y = rng.standard_normal(n).astype(np.float32)
    raw = rng.standard_normal((1, n)).astype(np.float32)
    d_y, d_raw = torch.from_numpy(y).cuda(), torch.from_numpy(raw).cuda()
    d_out = torch.zeros(2, device='cuda')
    stream = torch.cuda.Stream()
    assert lib.tgbm_metric_score_noalloc(b'reg:linear', n, 1, d_y.data_ptr(), d_raw.data_ptr(), d_out.data_ptr(), None) == 0   # warms the lookup
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert lib.tgbm_metric_score_noalloc(b'reg:linear', n, 1, d_y.data_ptr(), d_raw.data_ptr(), d_out.data_ptr() + 4,
                                         C.c_void_p(stream.cuda_stream)) == 0
    stream.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    got = d_out.cpu().numpy()
    assert got[0] == got[1] and abs(float(got[1]) - _numpy_metric('reg:linear', y, raw)) <= 1e-6


def test_noalloc_rejects_what_it_cannot_hold(gpu):
    import torch
    from thundergbm_b200 import _lib
    lib = _lib.lib()
    t = torch.zeros(8, device='cuda')
    p = t.data_ptr()
    assert lib.tgbm_metric_score_noalloc(b'reg:linear', (1 << 30) + 1, 1, p, p, p, None) == 1
    assert b'n_rows' in lib.tgbm_last_error()
    assert lib.tgbm_metric_score_noalloc(b'multi:softmax', 8, 2000, p, p, p, None) == 1
    assert b'trees_per_round' in lib.tgbm_last_error()
    assert lib.tgbm_metric_score_noalloc(b'rank:ndcg', 8, 1, p, p, p, None) == 1
    assert b'ranking' in lib.tgbm_last_error()
    assert lib.tgbm_metric_score_noalloc(b'reg:linear', 8, 1, None, p, p, None) == 1
