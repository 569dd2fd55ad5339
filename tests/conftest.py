import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'oracle'), os.path.join(ROOT, 'tests', 'golden'), os.path.join(ROOT, 'tests')):
    if p not in sys.path:
        sys.path.insert(0, p)


# The parity tests written against the oracle's exact mode (bit-for-bit comparisons) run the library in its
# deterministic mode; the tests of the fp32 mode (the library's default, tests/test_gpu_fp32.py) ask for it by name.
os.environ.setdefault('TGBM_HIST_MODE', 'exact')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope='session')
def orc():
    """The CPU oracle (checker).  Built on demand."""
    import tgbm_oracle
    tgbm_oracle.lib()
    return tgbm_oracle


@pytest.fixture(scope='session')
def gpu():
    if not _have_gpu():
        pytest.skip('no CUDA device')
    import torch
    torch.cuda.set_device(0)
    return True


@pytest.fixture(scope='session')
def cases():
    from make_inputs import CASES
    cache = {}

    def get(name):
        if name not in cache:
            make, params = CASES[name]
            cache[name] = (make(), dict(params))
        return cache[name]
    return get
