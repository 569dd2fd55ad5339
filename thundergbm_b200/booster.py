"""Explicit-state interface to the histogram tree builder: create / boost / read back.

Thin ctypes wrapper over part 2 of include/thundergbm.h.  Used by the benchmark, the parity tests
and multi-GPU launches (one process per GPU, a `Comm` per process).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import TgbmInfo, TgbmParam, TgbmProfile

NODE_DTYPE = np.dtype([('final_id', '<i4'), ('lch_index', '<i4'), ('rch_index', '<i4'), ('parent_index', '<i4'),
                       ('gain', '<f4'), ('base_weight', '<f4'), ('split_feature_id', '<i4'), ('split_value', '<f4'),
                       ('split_bid', 'u1'), ('default_right', 'u1'), ('is_leaf', 'u1'), ('is_valid', 'u1'),
                       ('is_pruned', 'u1'), ('pad', 'u1', (3,)), ('sum_g', '<f4'), ('sum_h', '<f4')])
assert NODE_DTYPE.itemsize == 48


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Comm:
    """NCCL communicator of one rank.  `unique_id()` on rank 0, then every rank constructs Comm(id, rank, world)."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _lib.check(_lib.lib().tgbm_comm_unique_id(buf))
        return buf.raw

    def __init__(self, uid: bytes, rank: int, world: int):
        self.rank, self.world = rank, world
        self.handle = _lib.lib().tgbm_comm_create(uid, rank, world)
        if not self.handle:
            raise RuntimeError(_lib.lib().tgbm_last_error().decode())

    def close(self):
        if self.handle:
            _lib.lib().tgbm_comm_destroy(self.handle)
            self.handle = None


def make_param(**kw) -> TgbmParam:
    p = TgbmParam()
    _lib.lib().tgbm_default_param(C.byref(p))
    for k, v in kw.items():
        if k == 'lambda':
            k = 'lambda_'
        if k == 'objective':
            v = v.encode()
        if k == 'tree_method':
            p.exact_builder = 1 if v == 'exact' else 0
            continue
        if k == 'hist_mode' and isinstance(v, str):
            v = {'fp32': 0, 'exact': 1}[v]
        if not hasattr(p, k):
            raise KeyError(k)
        setattr(p, k, v)
    return p


class Booster:
    def __init__(self, data, comm: Comm | None = None, **params):
        self._lib = _lib.lib()
        self._keep = [np.ascontiguousarray(data.val, np.float32), np.ascontiguousarray(data.row_ptr, np.int32),
                      np.ascontiguousarray(data.col, np.int32), np.ascontiguousarray(data.y, np.float32),
                      np.ascontiguousarray(data.group, np.int32)]
        val, rp, col, y, grp = self._keep
        self.param = make_param(**params)
        self.handle = self._lib.tgbm_booster_create(data.n_rows, _ptr(val), _ptr(rp), _ptr(col), _ptr(y),
                                                    _ptr(grp) if grp.size else None, int(grp.size),
                                                    C.byref(self.param), comm.handle if comm else None)
        if not self.handle:
            raise RuntimeError(self._lib.tgbm_last_error().decode())
        self._keep = None  # the library copied everything it needs

    def boost(self, n_rounds: int):
        _lib.check(self._lib.tgbm_booster_boost(self.handle, n_rounds))

    def boost_timed(self, n_rounds: int) -> float:
        """boost(n_rounds) + sync; returns the device time in milliseconds (CUDA events on the booster's stream)."""
        ms = C.c_float(0)
        _lib.check(self._lib.tgbm_booster_boost_timed(self.handle, n_rounds, C.byref(ms)))
        return ms.value

    def set_profile(self, on: bool):
        _lib.check(self._lib.tgbm_booster_set_profile(self.handle, int(on)))

    def sync(self):
        _lib.check(self._lib.tgbm_booster_sync(self.handle))

    @property
    def info(self) -> TgbmInfo:
        o = TgbmInfo()
        _lib.check(self._lib.tgbm_booster_info(self.handle, C.byref(o)))
        return o

    def profile(self) -> TgbmProfile:
        o = TgbmProfile()
        _lib.check(self._lib.tgbm_booster_profile(self.handle, C.byref(o)))
        return o

    def _get(self, name, shape, dtype):
        out = np.empty(shape, dtype)
        _lib.check(getattr(self._lib, 'tgbm_booster_' + name)(self.handle, _ptr(out)))
        return out

    def trees(self) -> np.ndarray:
        i = self.info
        return self._get('get_trees', (i.rounds_done, i.trees_per_round, i.n_nodes), NODE_DTYPE)

    def metrics(self) -> np.ndarray:
        return self._get('get_metrics', (self.info.rounds_done,), np.float32)

    def ypred(self) -> np.ndarray:
        i = self.info
        return self._get('get_ypred', (i.trees_per_round, i.n_rows), np.float32)

    def cuts(self):
        i = self.info
        cv, cp = np.empty(i.n_bins, np.float32), np.empty(i.n_features + 1, np.int32)
        _lib.check(self._lib.tgbm_booster_get_cuts(self.handle, _ptr(cv), _ptr(cp)))
        return cv, cp

    def bins(self) -> np.ndarray:
        i = self.info
        return self._get('get_bins', (i.n_rows, i.fpad), np.uint8)

    def bins_csr(self, nnz: int) -> np.ndarray:
        """CSR layout (info.csr_layout == 1): global bin id of every stored value, in input order."""
        return self._get('get_bins_csr', (nnz,), np.int32)

    def nid(self) -> np.ndarray:
        i = self.info
        return self._get('get_nid', (i.rounds_done * i.trees_per_round, i.n_rows), np.int32)

    def root_hist(self) -> np.ndarray:
        """Level-0 histogram of the last tree: int64 sums on the round's grid (exact mode) or float sums (fp32 mode)."""
        if self.param.hist_mode == 0:
            return self._get('get_root_hist_f32', (self.info.n_bins, 2), np.float32)
        return self._get('get_root_hist', (self.info.n_bins, 2), np.int64)

    def quant_scale(self) -> np.ndarray:
        return self._get('get_quant_scale', (self.info.rounds_done, 2), np.float64)

    def labels(self) -> np.ndarray:
        return self._get('get_labels', (self.info.n_labels,), np.float32)

    def close(self):
        if self.handle:
            self._lib.tgbm_booster_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def predict_raw(data, trees: np.ndarray, learning_rate: float, base_score: float, timing: bool = False):
    """Predictor::predict_raw on CSR rows; `trees` as returned by Booster.trees(); result [K][N].
    timing=True returns (result, device milliseconds of the traversal kernel)."""
    lib = _lib.lib()
    val = np.ascontiguousarray(data.val, np.float32)
    rp = np.ascontiguousarray(data.row_ptr, np.int32)
    col = np.ascontiguousarray(data.col, np.int32)
    trees = np.ascontiguousarray(trees)
    r, k, n = trees.shape
    out = np.empty((k, data.n_rows), np.float32)
    ms = C.c_float(0)
    _lib.check(lib.tgbm_predict_raw_timed(data.n_rows, _ptr(val), _ptr(rp), _ptr(col), _ptr(trees), r, k, n,
                                          learning_rate, base_score, _ptr(out), C.byref(ms) if timing else None))
    return (out, float(ms.value)) if timing else out
