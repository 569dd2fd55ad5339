"""ctypes wrapper of the CPU oracle (oracle/tgbm_oracle.cpp).

Test infrastructure: imported by tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline /
reference arm only.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'libtgbm_oracle.so')

OBJECTIVES = {'reg:linear': 0, 'reg:logistic': 1, 'binary:logistic': 2, 'multi:softmax': 3, 'multi:softprob': 4,
              'rank:pairwise': 5, 'rank:ndcg': 6}

NODE_DTYPE = np.dtype([('final_id', '<i4'), ('lch_index', '<i4'), ('rch_index', '<i4'), ('parent_index', '<i4'),
                       ('gain', '<f4'), ('base_weight', '<f4'), ('split_feature_id', '<i4'), ('split_value', '<f4'),
                       ('split_bid', 'u1'), ('default_right', 'u1'), ('is_leaf', 'u1'), ('is_valid', 'u1'),
                       ('is_pruned', 'u1'), ('pad', 'u1', (3,)), ('sum_g', '<f4'), ('sum_h', '<f4')])


class TgoParam(C.Structure):
    _fields_ = [('depth', C.c_int), ('n_trees', C.c_int), ('max_num_bin', C.c_int), ('objective', C.c_int),
                ('num_class', C.c_int), ('lambda_', C.c_float), ('gamma', C.c_float), ('min_child_weight', C.c_float),
                ('rt_eps', C.c_float), ('learning_rate', C.c_float), ('hist_mode', C.c_int), ('quant_bits', C.c_int),
                ('n_threads', C.c_int), ('keep_nid', C.c_int), ('portable_exp', C.c_int), ('rank_seed', C.c_uint),
                ('bagging', C.c_int), ('column_sampling_rate', C.c_float), ('sample_seed', C.c_uint),
                ('multi_shards', C.c_int), ('exact_builder', C.c_int)]


def build() -> str:
    subprocess.check_call(['make', '-s', '-C', HERE])
    return LIB_PATH


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            build()
        l = C.CDLL(LIB_PATH)
        vp = C.c_void_p
        l.tgo_train.restype = vp
        l.tgo_train.argtypes = [C.c_int, vp, vp, vp, vp, vp, C.c_int, C.POINTER(TgoParam)]
        l.tgo_bin_only.restype = vp
        l.tgo_bin_only.argtypes = [C.c_int, vp, vp, vp, C.c_int, C.c_int]
        l.tgo_free.argtypes = [vp]
        for n in ('n_features', 'n_bins', 'num_class', 'trees_per_round', 'n_nodes', 'n_labels'):
            getattr(l, 'tgo_' + n).argtypes = [vp]
            getattr(l, 'tgo_' + n).restype = C.c_int
        l.tgo_base_score.argtypes = [vp]; l.tgo_base_score.restype = C.c_float
        l.tgo_train_seconds.argtypes = [vp]; l.tgo_train_seconds.restype = C.c_double
        l.tgo_init_seconds.argtypes = [vp]; l.tgo_init_seconds.restype = C.c_double
        l.tgo_hist_dump_size.argtypes = [vp]; l.tgo_hist_dump_size.restype = C.c_long
        for n in ('cut_val', 'cut_ptr', 'bins', 'trees', 'metric', 'ypred', 'labels', 'nid', 'quant_scale', 'hist_dump', 'round_seconds', 'gain2'):
            getattr(l, 'tgo_' + n).argtypes = [vp]
            getattr(l, 'tgo_' + n).restype = vp
        l.tgo_predict_raw.argtypes = [C.c_int, vp, vp, vp, C.c_int, vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, vp]
        l.tgo_gradient.argtypes = [C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, vp]
        l.tgo_portable_expf.argtypes = [C.c_float]; l.tgo_portable_expf.restype = C.c_float
        _LIB = l
    return _LIB


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _view(addr, shape, dtype):
    n = int(np.prod(shape))
    if n == 0:
        return np.zeros(shape, dtype)
    buf = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(addr)
    return np.frombuffer(buf, dtype=dtype).reshape(shape).copy()


class Result:
    pass


def train(data, objective='reg:linear', depth=6, n_trees=40, max_num_bin=255, learning_rate=1.0, gamma=1.0,
          min_child_weight=1.0, hist_mode=1, quant_bits=18, n_threads=0, keep_nid=0, portable_exp=1, rank_seed=0,
          num_class=1, rt_eps=1e-6, tree_method='hist', bagging=0, column_sampling_rate=1.0, sample_seed=0,
          multi_shards=0, **kw):
    lam = kw.pop('lambda', kw.pop('lambda_', 1.0))
    assert not kw, kw
    l = lib()
    p = TgoParam(depth, n_trees, max_num_bin, OBJECTIVES[objective], num_class, lam, gamma, min_child_weight, rt_eps,
                 learning_rate, hist_mode, quant_bits, n_threads, keep_nid, portable_exp, rank_seed, int(bagging),
                 column_sampling_rate, sample_seed, multi_shards, 1 if tree_method == 'exact' else 0)
    rp = np.ascontiguousarray(data.row_ptr, np.int32); col = np.ascontiguousarray(data.col, np.int32)
    val = np.ascontiguousarray(data.val, np.float32); y = np.ascontiguousarray(data.y, np.float32)
    grp = np.ascontiguousarray(data.group, np.int32)
    h = l.tgo_train(data.n_rows, _ptr(rp), _ptr(col), _ptr(val), _ptr(y), _ptr(grp) if grp.size else None, int(grp.size), C.byref(p))
    r = Result()
    try:
        F, B, K, nn = l.tgo_n_features(h), l.tgo_n_bins(h), l.tgo_trees_per_round(h), l.tgo_n_nodes(h)
        r.n_features, r.n_bins, r.trees_per_round, r.n_nodes = F, B, K, nn
        r.num_class = l.tgo_num_class(h)
        r.base_score = l.tgo_base_score(h)
        r.train_seconds, r.init_seconds = l.tgo_train_seconds(h), l.tgo_init_seconds(h)
        r.cut_val = _view(l.tgo_cut_val(h), (B,), np.float32)
        r.cut_ptr = _view(l.tgo_cut_ptr(h), (F + 1,), np.int32)
        r.bins = _view(l.tgo_bins(h), (int(rp[-1]),), np.int32) if tree_method != 'exact' else np.zeros(0, np.int32)
        r.trees = _view(l.tgo_trees(h), (n_trees, K, nn), NODE_DTYPE)
        r.metric = _view(l.tgo_metric(h), (n_trees,), np.float32)
        r.ypred = _view(l.tgo_ypred(h), (K, data.n_rows), np.float32)
        r.labels = _view(l.tgo_labels(h), (l.tgo_n_labels(h),), np.float32)
        r.quant_scale = _view(l.tgo_quant_scale(h), (n_trees, 2), np.float64)
        r.gain2 = _view(l.tgo_gain2(h), (n_trees, K, nn), np.float32)
        r.round_seconds = _view(l.tgo_round_seconds(h), (n_trees,), np.float64)
        if keep_nid:
            r.nid = _view(l.tgo_nid(h), (n_trees * K, data.n_rows), np.int32)
            r.hist_dump = _view(l.tgo_hist_dump(h), (l.tgo_hist_dump_size(h),), np.float32)
    finally:
        l.tgo_free(h)
    return r


def bin_only(data, max_num_bin=255, multi_shards=0):
    l = lib()
    rp = np.ascontiguousarray(data.row_ptr, np.int32); col = np.ascontiguousarray(data.col, np.int32)
    val = np.ascontiguousarray(data.val, np.float32)
    h = l.tgo_bin_only(data.n_rows, _ptr(rp), _ptr(col), _ptr(val), max_num_bin, multi_shards)
    try:
        F, B = l.tgo_n_features(h), l.tgo_n_bins(h)
        return (_view(l.tgo_cut_val(h), (B,), np.float32), _view(l.tgo_cut_ptr(h), (F + 1,), np.int32),
                _view(l.tgo_bins(h), (int(rp[-1]),), np.int32))
    finally:
        l.tgo_free(h)


def predict_raw(data, trees, learning_rate, base_score, n_features=None):
    l = lib()
    rp = np.ascontiguousarray(data.row_ptr, np.int32); col = np.ascontiguousarray(data.col, np.int32)
    val = np.ascontiguousarray(data.val, np.float32)
    trees = np.ascontiguousarray(trees)
    r, k, n = trees.shape
    F = n_features if n_features is not None else (int(col.max()) + 1 if col.size else 0)
    out = np.empty((k, data.n_rows), np.float32)
    l.tgo_predict_raw(data.n_rows, _ptr(rp), _ptr(col), _ptr(val), F, _ptr(trees), r, k, n, learning_rate, base_score, _ptr(out))
    return out


def gradient(y, yp, objective, K=1, portable_exp=1):
    l = lib()
    y = np.ascontiguousarray(y, np.float32); yp = np.ascontiguousarray(yp, np.float32)
    out = np.empty((K * y.size, 2), np.float32)
    l.tgo_gradient(y.size, _ptr(y), _ptr(yp), OBJECTIVES[objective], K, portable_exp, _ptr(out))
    return out


def bins_to_dense(data, bins, cut_ptr, fpad):
    """global-bin-id CSR -> the dense local-bin matrix the CUDA path stores ([N][fpad] uint8, 255 = missing)."""
    out = np.full((data.n_rows, fpad), 255, np.uint8)
    rows = np.repeat(np.arange(data.n_rows), np.diff(data.row_ptr))
    out[rows, data.col] = (bins - cut_ptr[data.col]).astype(np.uint8)
    return out
