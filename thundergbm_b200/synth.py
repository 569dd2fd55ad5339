"""Seeded synthetic stand-ins for the benchmark data sets.

The public data sets the reference is benchmarked on (HIGGS, covtype, MSLR-WEB,
a news20-like sparse set) are not available offline.  These generators only
reproduce their *shapes and value distributions*; no record of any real data
set is reproduced.  Every generator returns CSR arrays with explicit zeros
removed and column indices ascending inside a row, which is what the
reference's Python wrapper hands to ``sparse_train_scikit``
(python/thundergbm/thundergbm.py:87-129).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np


@dataclass
class CsrData:
    n_rows: int
    n_cols: int
    row_ptr: np.ndarray  # int32 [n_rows+1]
    col: np.ndarray  # int32 [nnz]
    val: np.ndarray  # float32 [nnz]
    y: np.ndarray  # float32 [n_rows]
    group: np.ndarray = field(default_factory=lambda: np.zeros(0, np.int32))  # rows per query

    @property
    def nnz(self) -> int:
        return int(self.row_ptr[-1])

    def rows(self, lo: int, hi: int) -> "CsrData":
        """Contiguous row block [lo, hi) as its own CSR (used for row sharding)."""
        a, b = int(self.row_ptr[lo]), int(self.row_ptr[hi])
        return CsrData(hi - lo, self.n_cols, (self.row_ptr[lo:hi + 1] - a).astype(np.int32),
                       self.col[a:b], self.val[a:b], self.y[lo:hi])


def dense_to_csr(x: np.ndarray, y: np.ndarray, group=None) -> CsrData:
    """Row-major dense matrix -> CSR with explicit zeros dropped (they become 'missing')."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, f = x.shape
    mask = x != 0
    counts = mask.sum(axis=1, dtype=np.int64)
    row_ptr = np.zeros(n + 1, np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    assert row_ptr[-1] < 2 ** 31, "nnz must fit int32 like the reference"
    col = np.nonzero(mask)[1].astype(np.int32)
    val = x[mask]
    g = np.zeros(0, np.int32) if group is None else np.asarray(group, np.int32)
    return CsrData(n, f, row_ptr.astype(np.int32), col, val, np.asarray(y, np.float32), g)


def dense_regression(n=10_000, f=32, seed=0) -> CsrData:
    """Config 1: x~U(0,1), y = sum w_i x_i + 0.5 x_0 x_1 + 0.1 N(0,1), w~N(0,1)."""
    rng = np.random.default_rng(seed)
    x = rng.random((n, f), dtype=np.float32)
    w = rng.standard_normal(f).astype(np.float32)
    y = x @ w + 0.5 * x[:, 0] * x[:, 1] + 0.1 * rng.standard_normal(n).astype(np.float32)
    return dense_to_csr(x, y.astype(np.float32))


def higgs_like(n=10_500_000, seed=1, rows=None, chunk=262_144) -> CsrData:
    """Config 2: 28 dense float32 features; 0-20 N(0,1) or |N(0,1)|, 21-27 LogNormal(0,0.5);
    y ~ Bernoulli(sigmoid(s)), s = sparse linear term over 8 features + 4 pairwise products,
    shifted to give ~53 % positives.

    Rows are generated in fixed chunks with one random stream per chunk, so `rows=(lo, hi)` yields
    exactly the rows [lo, hi) of the full data set without generating the rest (row sharding)."""
    f = 28
    lo, hi = (0, n) if rows is None else rows
    head = np.random.default_rng([seed, 0xC0FFEE])
    absf = head.random(21) < 0.5
    lin_idx = head.choice(f, 8, replace=False)
    lin_w = head.standard_normal(8).astype(np.float32)
    pairs = head.choice(f, (4, 2))
    pair_w = head.standard_normal(4).astype(np.float32) * 0.5

    def gen(c):  # chunk c -> (x, raw score, uniform draws)
        rng = np.random.default_rng([seed, c])
        m = min(chunk, n - c * chunk)
        a = rng.standard_normal((m, 21), dtype=np.float32)
        a[:, absf] = np.abs(a[:, absf])
        b = np.exp(0.5 * rng.standard_normal((m, 7), dtype=np.float32))
        xb = np.concatenate([a, b], axis=1)
        s = xb[:, lin_idx] @ lin_w
        for (i, j), w in zip(pairs, pair_w):
            s += w * xb[:, i] * xb[:, j]
        return xb, s, rng.random(m, dtype=np.float32)

    shift = np.quantile(gen(0)[1], 0.47)  # from chunk 0, the same on every shard
    m = hi - lo
    x = np.empty((m, f), np.float32)
    y = np.empty(m, np.float32)
    for c in range(lo // chunk, (hi + chunk - 1) // chunk):
        xb, s, u = gen(c)
        a, b = max(lo, c * chunk), min(hi, c * chunk + xb.shape[0])
        sl = slice(a - c * chunk, b - c * chunk)
        x[a - lo:b - lo] = xb[sl]
        y[a - lo:b - lo] = u[sl] < 1.0 / (1.0 + np.exp(-(s[sl] - shift)))
    # continuous features contain no exact zeros, so the CSR is fully dense
    row_ptr = (np.arange(m + 1, dtype=np.int64) * f)
    assert row_ptr[-1] < 2 ** 31
    x[x == 0] = np.float32(1e-30)
    col = np.tile(np.arange(f, dtype=np.int32), m)
    return CsrData(m, f, row_ptr.astype(np.int32), col, x.reshape(-1), y)


def covtype_like(n=581_012, seed=2) -> CsrData:
    """Config 3: 54 features; 0-9 integer U(0,cap_j) with cap_j<=4000, 10-13 one-hot(4),
    14-53 one-hot(40) drawn Zipf(1.3); 7 classes = argmax of random linear scores + Gumbel."""
    rng = np.random.default_rng(seed)
    caps = rng.integers(200, 4001, 10)
    x = np.zeros((n, 54), np.float32)
    for j in range(10):
        x[:, j] = rng.integers(0, caps[j] + 1, n)
    x[np.arange(n), 10 + rng.integers(0, 4, n)] = 1
    z = np.minimum(rng.zipf(1.3, n), 40) - 1
    x[np.arange(n), 14 + z] = 1
    w = rng.standard_normal((54, 7)).astype(np.float32)
    xs = x.copy()
    xs[:, :10] /= caps
    score = xs @ w + rng.gumbel(size=(n, 7)).astype(np.float32)
    y = score.argmax(axis=1).astype(np.float32)
    return dense_to_csr(x, y)


def sparse_binary(n=1_000_000, f=100_000, seed=3) -> CsrData:
    """Config 4: CSR, nnz/row Poisson(40) (min 1), columns Zipf(1.1), all values 1.0;
    y ~ Bernoulli(sigmoid(sum_j w_j x_j)), w~N(0,1) on 2,000 random columns."""
    rng = np.random.default_rng(seed)
    k = np.maximum(rng.poisson(40, n), 1)
    total = int(k.sum())
    cols = (rng.zipf(1.1, total) - 1) % f
    rows = np.repeat(np.arange(n, dtype=np.int64), k)
    key = np.unique(rows * f + cols)  # sorted by (row, col), duplicates dropped
    rows = (key // f).astype(np.int64)
    col = (key % f).astype(np.int32)
    row_ptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=row_ptr[1:])
    w = np.zeros(f, np.float32)
    w[rng.choice(f, min(2000, f), replace=False)] = rng.standard_normal(min(2000, f)).astype(np.float32)
    s = np.bincount(rows, weights=w[col], minlength=n)
    y = (rng.random(n) < 1.0 / (1.0 + np.exp(-s))).astype(np.float32)
    return CsrData(n, f, row_ptr.astype(np.int32), col, np.ones(col.size, np.float32), y)


def mslr_like(n=2_270_000, f=136, seed=4) -> CsrData:
    """Config 5: query groups Poisson(120) (min 1); half the features Poisson(5) counts, half
    LogNormal(0,1); relevance 0-4 from a hidden linear score + noise at 52/32/13/2/1 %."""
    rng = np.random.default_rng(seed)
    group = []
    left = n
    while left > 0:
        g = min(left, max(1, int(rng.poisson(120))))
        group.append(g)
        left -= g
    h = f // 2
    x = np.empty((n, f), np.float32)
    x[:, :h] = rng.poisson(5, (n, h))
    x[:, h:] = np.exp(rng.standard_normal((n, f - h), dtype=np.float32))
    w = rng.standard_normal(f).astype(np.float32)
    xs = x.copy()
    xs[:, :h] = (xs[:, :h] - 5) / np.sqrt(5.0)
    xs[:, h:] = np.log(xs[:, h:])
    s = xs @ w / np.sqrt(f) + 0.5 * rng.standard_normal(n).astype(np.float32)
    q = np.quantile(s, [0.52, 0.84, 0.97, 0.99])
    y = np.searchsorted(q, s).astype(np.float32)
    return dense_to_csr(x, y, group)


def read_libsvm(path: str, group_path: str | None = None) -> CsrData:
    """LibSVM text ``label idx:val ...`` (1-based idx) -> CSR; optional one-integer-per-line group file."""
    row_ptr, col, val, y = [0], [], [], []
    with open(path) as fh:
        for line in fh:
            line = line.split('#', 1)[0].split()
            if not line:
                continue
            y.append(float(line[0]))
            for tok in line[1:]:
                i, v = tok.split(':')
                col.append(int(i) - 1)
                val.append(float(v))
            row_ptr.append(len(col))
    group = np.zeros(0, np.int32)
    if group_path:
        group = np.loadtxt(group_path, dtype=np.int32, ndmin=1)
    col = np.asarray(col, np.int32)
    return CsrData(len(y), int(col.max()) + 1 if col.size else 0, np.asarray(row_ptr, np.int32), col,
                   np.asarray(val, np.float32), np.asarray(y, np.float32), group)


def write_tgbin(d: CsrData, path: str) -> None:
    """Binary CSR container read by the golden-vector harness and the CPU oracle's CLI:
    i32 n_rows, i32 n_group, i64 nnz, row_ptr, col, val, y, group."""
    with open(path, 'wb') as fh:
        fh.write(struct.pack('<iiq', d.n_rows, int(d.group.size), d.nnz))
        fh.write(np.ascontiguousarray(d.row_ptr, np.int32).tobytes())
        fh.write(np.ascontiguousarray(d.col, np.int32).tobytes())
        fh.write(np.ascontiguousarray(d.val, np.float32).tobytes())
        fh.write(np.ascontiguousarray(d.y, np.float32).tobytes())
        fh.write(np.ascontiguousarray(d.group, np.int32).tobytes())
