"""ctypes binding of libthundergbm.so (the CUDA library built by thundergbm_b200.build).

There is no fallback: if the library is missing or cannot be loaded this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'libthundergbm.so')


class TgbmParam(C.Structure):
    _fields_ = [('depth', C.c_int), ('n_trees', C.c_int), ('max_num_bin', C.c_int), ('num_class', C.c_int),
                ('min_child_weight', C.c_float), ('lambda_', C.c_float), ('gamma', C.c_float),
                ('learning_rate', C.c_float), ('objective', C.c_char_p), ('quant_bits', C.c_int),
                ('keep_nid', C.c_int), ('verbose', C.c_int), ('profile', C.c_int), ('rank_seed', C.c_uint),
                ('hist_mode', C.c_int), ('bagging', C.c_int), ('column_sampling_rate', C.c_float), ('sample_seed', C.c_uint), ('column_shards', C.c_int), ('exact_builder', C.c_int)]


class TgbmInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ('n_rows', 'n_features', 'fpad', 'n_bins', 'trees_per_round', 'n_nodes',
                                       'num_class', 'rounds_done', 'n_labels')] + [('base_score', C.c_float), ('csr_layout', C.c_int)]


class TgbmProfile(C.Structure):
    _fields_ = [(n, C.c_double) for n in ('hist_ms', 'hist_bytes', 'hist_root_ms', 'hist_root_bytes', 'partition_ms',
                                          'partition_bytes')] + \
               [(n, C.c_longlong) for n in ('hist_launches', 'hist_root_launches', 'partition_launches',
                                            'kernel_launches', 'hist_rows')]


def load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f'{LIB_PATH} not found: build it first (python -m thundergbm_b200.build)')
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    P = C.POINTER
    vp, ip, fp = C.c_void_p, P(C.c_int), P(C.c_float)
    lib.tgbm_last_error.restype = C.c_char_p
    lib.tgbm_default_param.argtypes = [P(TgbmParam)]
    lib.tgbm_comm_unique_id.argtypes = [C.c_char_p]
    lib.tgbm_comm_create.restype = vp
    lib.tgbm_comm_create.argtypes = [C.c_char_p, C.c_int, C.c_int]
    lib.tgbm_comm_destroy.argtypes = [vp]
    lib.tgbm_booster_create.restype = vp
    lib.tgbm_booster_create.argtypes = [C.c_int, vp, vp, vp, vp, vp, C.c_int, P(TgbmParam), vp]
    lib.tgbm_booster_boost.argtypes = [vp, C.c_int]
    lib.tgbm_booster_sync.argtypes = [vp]
    lib.tgbm_booster_set_profile.argtypes = [vp, C.c_int]
    lib.tgbm_booster_boost_timed.argtypes = [vp, C.c_int, fp]
    lib.tgbm_booster_info.argtypes = [vp, P(TgbmInfo)]
    lib.tgbm_booster_profile.argtypes = [vp, P(TgbmProfile)]
    for name in ('get_trees', 'get_metrics', 'get_ypred', 'get_bins', 'get_bins_csr', 'get_nid', 'get_root_hist', 'get_root_hist_f32', 'get_quant_scale',
                 'get_labels', 'to_model'):
        getattr(lib, 'tgbm_booster_' + name).argtypes = [vp, vp]
    lib.tgbm_booster_get_cuts.argtypes = [vp, vp, vp]
    lib.tgbm_booster_free.argtypes = [vp]
    lib.tgbm_release_device_memory.argtypes = []
    lib.tgbm_release_device_memory.restype = None
    lib.tgbm_predict_raw.argtypes = [C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, vp]
    lib.tgbm_predict_raw_timed.argtypes = [C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, vp, vp]
    lib.tgbm_metric_score.argtypes = [C.c_char_p, C.c_int, C.c_int, vp, vp, vp, C.c_int, fp]
    lib.tgbm_metric_score_noalloc.argtypes = [C.c_char_p, C.c_int, C.c_int, vp, vp, vp, vp]
    lib.sparse_train_scikit.argtypes = [C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                        C.c_float, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_float,
                                        C.c_char_p, ip, C.c_char_p, vp, ip, vp, vp, C.c_int]
    lib.sparse_predict_scikit.argtypes = [C.c_int, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_char_p, C.c_int,
                                          C.c_float, vp, vp, C.c_int, C.c_int]
    lib.save.argtypes = [C.c_char_p, C.c_char_p, C.c_float, C.c_int, C.c_int, C.c_int, vp, vp]
    lib.load_model.argtypes = [C.c_char_p, fp, ip, ip, ip, vp]
    lib.load_config.argtypes = [C.c_char_p, vp]
    lib.get_n_nodes.argtypes = [vp, vp, C.c_int, C.c_int]
    lib.get_a_tree.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, vp, vp, vp, vp]
    lib.model_free.argtypes = [vp]
    lib.set_logger.argtypes = [C.c_int]
    return lib


_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(lib().tgbm_last_error().decode())
