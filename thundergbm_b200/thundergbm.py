"""scikit-learn style front end with the class names and constructor arguments of the reference's Python
package (python/thundergbm/thundergbm.py:46-395: TGBMModel, TGBMClassifier, TGBMRegressor, TGBMRanker).

Every method goes through the same extern "C" functions the reference's wrapper binds
(sparse_train_scikit, sparse_predict_scikit, save, load_model, load_config, get_n_nodes, get_a_tree,
model_free), so the reference's own wrapper file works against this library unchanged; this module only
spares users the dependency on it.  Behaviour kept on purpose: dense input is converted with
scipy.sparse.csr_matrix, which drops explicit zeros (they become missing values), and predict() does not add
the base score the training started from (src/thundergbm/scikit_tgbm.cpp:87-90).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import scipy.sparse as sp

from . import _lib


def _vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class TGBMModel:
    _impl = 'regressor'

    def __init__(self, depth=6, n_trees=40, n_gpus=1, min_child_weight=1.0, lambda_tgbm=1.0, gamma=1.0,
                 max_num_bin=255, verbose=1, column_sampling_rate=1.0, bagging=0, n_parallel_trees=1,
                 learning_rate=1.0, objective='reg:linear', num_class=1, tree_method='auto'):
        self.depth, self.n_trees, self.n_gpus = depth, n_trees, n_gpus
        self.min_child_weight, self.lambda_tgbm, self.gamma = min_child_weight, lambda_tgbm, gamma
        self.max_num_bin, self.verbose = max_num_bin, verbose
        self.column_sampling_rate, self.bagging, self.n_parallel_trees = column_sampling_rate, bagging, n_parallel_trees
        self.learning_rate, self.objective, self.num_class, self.tree_method = learning_rate, objective, num_class, tree_method
        self.model = None
        self.tree_per_iter = -1
        self.group_label = None
        self._lib = _lib.lib()

    # -- helpers -----------------------------------------------------------------------------------
    def _free(self):
        if self.model is not None and self.model.value:
            self._lib.model_free(C.byref(self.model))
        self.model = None

    def __del__(self):
        try:
            self._free()
        except Exception:
            pass

    @staticmethod
    def _csr(X):
        X = X if sp.issparse(X) else sp.csr_matrix(X)
        X = X.tocsr()
        X.sort_indices()
        return (np.ascontiguousarray(X.data, np.float32), np.ascontiguousarray(X.indptr, np.int32),
                np.ascontiguousarray(X.indices, np.int32), X.shape[0])

    # -- API ---------------------------------------------------------------------------------------
    def fit(self, X, y, groups=None):
        self._free()
        val, indptr, indices, n = self._csr(X)
        y = np.ascontiguousarray(y, np.float32)
        if y.shape[0] != n:
            raise ValueError('X and y have different numbers of rows')
        grp = None if groups is None else np.ascontiguousarray(groups, np.int32)
        n_labels = max(1, len(set(y.tolist())))
        group_label = (C.c_float * n_labels)()
        n_class = C.c_int(self.num_class)
        per_iter = C.c_int(0)
        model = C.c_void_p(None)
        self._lib.sparse_train_scikit(n, _vp(val), _vp(indptr), _vp(indices), _vp(y), self.depth, self.n_trees,
                                      self.n_gpus, self.min_child_weight, self.lambda_tgbm, self.gamma, self.max_num_bin,
                                      self.verbose, self.column_sampling_rate, int(self.bagging), self.n_parallel_trees,
                                      self.learning_rate, self.objective.encode(), C.byref(n_class),
                                      self.tree_method.encode(), C.byref(model), C.byref(per_iter), group_label,
                                      _vp(grp), 0 if grp is None else int(grp.size))
        if not model.value:
            raise RuntimeError('training failed: ' + self._lib.tgbm_last_error().decode())
        self.model, self.num_class, self.tree_per_iter = model, n_class.value, per_iter.value
        self.group_label = [group_label[i] for i in range(n_labels)]
        return self

    def predict(self, X, groups=None):
        if self.model is None:
            raise ValueError('Please train the model first or load model from file!')
        val, indptr, indices, n = self._csr(X)
        n_out = n * self.num_class if self.objective == 'multi:softprob' else n
        out = np.zeros(n_out, np.float32)
        gl = None
        if self.group_label is not None:
            gl = (C.c_float * max(len(self.group_label), self.num_class))(*self.group_label)
        grp = None if groups is None else np.ascontiguousarray(groups, np.int32)
        self._lib.sparse_predict_scikit(n, _vp(val), _vp(indptr), _vp(indices), _vp(out), C.byref(self.model),
                                        self.n_trees, self.tree_per_iter, self.objective.encode(), self.num_class,
                                        self.learning_rate, gl, _vp(grp), 0 if grp is None else int(grp.size), self.verbose)
        err = self._lib.tgbm_last_error()
        if err:
            raise RuntimeError(err.decode())
        if self.objective == 'multi:softprob':
            return out.reshape([-1, self.num_class])  # the reference reshapes its class-major buffer this way too
        return out

    def save_model(self, model_path):
        if self.model is None:
            raise ValueError('Please train the model first or load model from file!')
        gl = None
        if self.group_label is not None:
            gl = (C.c_float * max(len(self.group_label), self.num_class))(*self.group_label)
        self._lib.save(str(model_path).encode(), self.objective.encode(), self.learning_rate, self.num_class,
                       self.n_trees, self.tree_per_iter, C.byref(self.model), gl)

    def load_model(self, model_path):
        self._free()
        lr, nc, nt, per = C.c_float(0), C.c_int(0), C.c_int(0), C.c_int(0)
        model = C.c_void_p(None)
        self._lib.load_model(str(model_path).encode(), C.byref(lr), C.byref(nc), C.byref(nt), C.byref(per), C.byref(model))
        if not model.value:
            raise ValueError('Model is None: ' + self._lib.tgbm_last_error().decode())
        self.model, self.learning_rate, self.num_class, self.n_trees, self.tree_per_iter = model, lr.value, nc.value, nt.value, per.value
        gl = (C.c_float * max(1, self.num_class))()
        self._lib.load_config(str(model_path).encode(), gl)
        self.group_label = [gl[i] for i in range(self.num_class)]

    def get_trees(self):
        """Per tree the arrays get_a_tree exposes (children, default child, feature, threshold, leaf value,
        hessian sum) -- the input of the reference's get_shap_trees()."""
        total = self.n_trees * self.tree_per_iter
        n_nodes = np.zeros(total, np.int32)
        self._lib.get_n_nodes(C.byref(self.model), _vp(n_nodes), self.n_trees, self.tree_per_iter)
        trees = []
        for t in range(total):
            n = int(n_nodes[t])
            a = {k: np.empty(n, np.int32) for k in ('children_left', 'children_right', 'children_default', 'feature')}
            a.update({k: np.empty(n, np.float32) for k in ('threshold', 'value', 'node_sample_weight')})
            self._lib.get_a_tree(C.byref(self.model), t, n, _vp(a['children_left']), _vp(a['children_right']),
                                 _vp(a['children_default']), _vp(a['feature']), _vp(a['threshold']), _vp(a['value']),
                                 _vp(a['node_sample_weight']))
            trees.append(a)
        return trees


    def cv(self, X, y, folds=None, nfold=5, shuffle=True, seed=0):
        """k-fold cross validation as the reference's wrapper does it (python/thundergbm/thundergbm.py:223-282): rows
        permuted with RandomState(seed), folds of int(n / nfold) consecutive entries of the permutation (or the
        caller's (train_ids, test_ids) pairs), fit + predict per fold; accuracy for classifiers, mean squared error for
        regressors (which the reference reports under the key 'RMSE'); not for rankers.  Returns, and keeps in
        `eval_res`, mean and sample standard deviation of the train and test scores."""
        if self._impl == 'ranker':
            print('Cross-validation for ## Ranker ## have not been supported yep..')
            return None
        import statistics
        X = X.tocsr() if sp.issparse(X) else sp.csr_matrix(X)
        y = np.asarray(y, np.float32)
        n = X.shape[0]
        if folds is not None:
            train_ids, test_ids = [f[0] for f in folds], [f[1] for f in folds]
            nfold = len(train_ids)
        else:
            order = np.random.RandomState(seed).permutation(n) if shuffle else np.arange(n)
            step = int(n / nfold)
            test_ids = [order[i:i + step] for i in range(0, n, step)]
            train_ids = [np.concatenate([test_ids[i] for i in range(nfold) if i != k]) for k in range(nfold)]
        train_scores, test_scores = [], []
        for k in range(nfold):
            self.fit(X[train_ids[k], :], y[train_ids[k]])
            pairs = ((self.predict(X[train_ids[k], :]), y[train_ids[k]]), (self.predict(X[test_ids[k], :]), y[test_ids[k]]))
            for (pred, truth), scores in zip(pairs, (train_scores, test_scores)):
                if self._impl == 'classifier':
                    scores.append(float(np.mean(np.asarray(pred) == truth)))
                else:
                    scores.append(float(np.mean((np.asarray(pred, np.float64) - truth) ** 2)))
        name = 'accuracy' if self._impl == 'classifier' else 'RMSE'
        self.eval_res = {f'train-{name}-mean': statistics.mean(train_scores), f'train-{name}-std': statistics.stdev(train_scores),
                         f'test-{name}-mean': statistics.mean(test_scores), f'test-{name}-std': statistics.stdev(test_scores)}
        print('mean train %s:%.6f+%.6f' % (name, self.eval_res[f'train-{name}-mean'], self.eval_res[f'train-{name}-std']))
        print('mean test %s:%.6f+%.6f' % (name, self.eval_res[f'test-{name}-mean'], self.eval_res[f'test-{name}-std']))
        return self.eval_res

    def get_shap_trees(self):
        """The trees as `shap.explainers.tree.Tree` objects (python/thundergbm/thundergbm.py:284-351): one tree per
        round, leaf values as a column.  Needs the `shap` package; `get_trees()` gives the same arrays without it."""
        if self.objective != 'binary:logistic' and self.tree_per_iter != 1:
            raise RuntimeError('not supported yet!')
        import shap.explainers.tree as shap_tree
        out = []
        for t in self.get_trees()[::self.tree_per_iter]:
            t = dict(t)
            t['value'] = t['value'].reshape(-1, 1)
            out.append(shap_tree.Tree(t))
        return out


class TGBMClassifier(TGBMModel):
    _impl = 'classifier'

    def __init__(self, depth=6, n_trees=40, n_gpus=1, min_child_weight=1.0, lambda_tgbm=1.0, gamma=1.0,
                 max_num_bin=255, verbose=1, column_sampling_rate=1.0, bagging=0, n_parallel_trees=1,
                 learning_rate=1.0, objective='multi:softmax', num_class=2, tree_method='auto'):
        super().__init__(depth, n_trees, n_gpus, min_child_weight, lambda_tgbm, gamma, max_num_bin, verbose,
                         column_sampling_rate, bagging, n_parallel_trees, learning_rate, objective, num_class, tree_method)


class TGBMRegressor(TGBMModel):
    _impl = 'regressor'


class TGBMRanker(TGBMModel):
    _impl = 'ranker'
