"""No GPU needed: the C-ABI library loads, exports every symbol include/thundergbm.h declares, and its host-only
entry points (model file I/O) behave like the reference's."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from thundergbm_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'thundergbm.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    text = '\n'.join(l for l in text.splitlines() if not l.lstrip().startswith('#'))
    return sorted(set(re.findall(r'\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;', text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert {'sparse_train_scikit', 'sparse_predict_scikit', 'save', 'load_model', 'load_config', 'get_n_nodes',
            'get_a_tree', 'model_free', 'set_logger', 'train_R', 'predict_R', 'tgbm_booster_create'} <= set(names)
    for n in names:
        assert hasattr(lib, n), f'{n} is declared in include/thundergbm.h but not exported'


def test_reference_symbol_list_matches_the_reference_library():
    """The 11 extern "C" names of the reference (src/thundergbm/scikit_tgbm.cpp, gbm_R_interface.cpp)."""
    ref = {'set_logger', 'sparse_train_scikit', 'sparse_predict_scikit', 'save', 'load_model', 'load_config',
           'get_n_nodes', 'get_a_tree', 'model_free', 'train_R', 'predict_R'}
    assert ref <= set(declared_symbols())


def test_model_file_layout_and_roundtrip(lib, tmp_path):
    """Model file written by hand in the reference's layout (src/thundergbm/parser.cpp:146-171) -> load_model ->
    save -> identical bytes (base_score excepted: the scikit save() writes its default 0)."""
    n_nodes, n_rounds, per = 7, 3, 2
    rng = np.random.default_rng(0)
    nodes = rng.integers(0, 255, (n_rounds, per, n_nodes, 48), dtype=np.uint8)
    obj = b'multi:softmax'
    blob = struct.pack('<i', len(obj)) + obj + struct.pack('<fiifi', 0.25, 2, n_rounds, 0.0, 2) + struct.pack('<ff', -1.0, 1.0)
    blob += struct.pack('<i', n_rounds)
    for r in range(n_rounds):
        blob += struct.pack('<i', per)
        for k in range(per):
            blob += struct.pack('<Q', n_nodes) + nodes[r, k].tobytes()
    path = tmp_path / 'in.model'
    path.write_bytes(blob)
    lr, nc, nt, pi = C.c_float(0), C.c_int(0), C.c_int(0), C.c_int(0)
    model = C.c_void_p(None)
    lib.load_model(str(path).encode(), C.byref(lr), C.byref(nc), C.byref(nt), C.byref(pi), C.byref(model))
    assert model.value, lib.tgbm_last_error()
    assert (lr.value, nc.value, nt.value, pi.value) == (0.25, 2, n_rounds, per)
    gl = (C.c_float * 2)()
    lib.load_config(str(path).encode(), gl)
    assert list(gl) == [-1.0, 1.0]
    cnt = np.zeros(n_rounds * per, np.int32)
    lib.get_n_nodes(C.byref(model), cnt.ctypes.data_as(C.c_void_p), n_rounds, per)
    assert (cnt == n_nodes).all()
    out = tmp_path / 'out.model'
    lib.save(str(out).encode(), obj, 0.25, 2, n_rounds, per, C.byref(model), gl)
    assert out.read_bytes() == blob
    lib.model_free(C.byref(model))
    assert model.value is None


def test_load_model_missing_file_reports_error(lib):
    lr, nc, nt, pi = C.c_float(0), C.c_int(0), C.c_int(0), C.c_int(0)
    model = C.c_void_p(7)
    lib.set_logger(0)
    lib.load_model(b'/nonexistent/none.model', C.byref(lr), C.byref(nc), C.byref(nt), C.byref(pi), C.byref(model))
    assert model.value is None and b'cannot read' in lib.tgbm_last_error()


def test_default_param_matches_reference_parser(lib):
    """src/thundergbm/parser.cpp:10-28"""
    from thundergbm_b200._lib import TgbmParam
    p = TgbmParam()
    lib.tgbm_default_param(C.byref(p))
    assert (p.depth, p.n_trees, p.max_num_bin, p.num_class) == (6, 40, 255, 1)
    assert (p.min_child_weight, p.lambda_, p.gamma, p.learning_rate) == (1.0, 1.0, 1.0, 1.0)
    assert p.objective == b'reg:linear'


def test_no_cpu_fallback_in_the_product():
    """The product never reaches for the oracle."""
    pkg = os.path.join(ROOT, 'thundergbm_b200')
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.cpp', '.h')):
                text = open(os.path.join(dirpath, f)).read()
                assert 'tgbm_oracle' not in text and 'oracle/' not in text, f
