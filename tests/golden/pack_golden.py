"""Packs what the reference produced on a B200 (tests/golden/run_reference.sh, outputs under
<run_dir>/<case>/) into small committed fixtures tests/golden/ref_<case>.npz:

  cut_val, cut_ptr     cut points of HistCut::get_cut_points_single, complete
  bins_sha256, bins_head   global bin ids of get_bin_ids: digest of the int32 array + its first 4096 entries
  trees                the model file's node tables (uint8 view of 48-byte records) [rounds, K, n_nodes*48]
  base_score, label, num_class
  metric               the per-round training metric the reference logged
  raw_pred_sample      every 37th raw prediction on the training rows + digest of the whole array
  logloss              mean negative log-likelihood of the training labels under the reference's raw scores
                       (classification objectives; the reference itself logs only error / accuracy)
  spread_*             how far further runs of the reference on the same input sit from the packed one
                       (its histograms are unordered float atomics): per-round metric, raw predictions,
                       logloss, gains and node weights of the first tree along identically split paths

    python tests/golden/pack_golden.py <run_dir> [--rerun <run_dir2> ...] [--out <dir>] [--shrink]

--prefix exact packs runs made with tree_method=exact dump_bins=0 (no cut points exist there) as ref_exact_<case>.npz.

A run made with n_device=D > 1 (the reference's column-sharded builder; run_reference.sh <out> n_device=2) is packed
as ref_multi_<case>.npz with the same keys plus n_device: cut points of all features in feature order (they descend
inside a feature there) and the global bin ids rebuilt from the devices' dense matrices.

--shrink replaces <case>/csr_bin_id.i32 by its digest (bins_digest.npz) so that a large case can be
carried off the GPU box; packing accepts either form.
"""
from __future__ import annotations

import hashlib
import os
import re
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, '..'))

NODE_DTYPE = np.dtype([('final_id', '<i4'), ('lch_index', '<i4'), ('rch_index', '<i4'), ('parent_index', '<i4'),
                       ('gain', '<f4'), ('base_weight', '<f4'), ('split_feature_id', '<i4'), ('split_value', '<f4'),
                       ('split_bid', 'u1'), ('default_right', 'u1'), ('is_leaf', 'u1'), ('is_valid', 'u1'),
                       ('is_pruned', 'u1'), ('pad', 'u1', (3,)), ('sum_g', '<f4'), ('sum_h', '<f4')])


def read_model(path):
    b = open(path, 'rb').read()
    o = 0
    (ln,) = struct.unpack_from('<i', b, o); o += 4
    obj = b[o:o + ln].decode(); o += ln
    lr, nc, nt, bs, nl = struct.unpack_from('<fiifi', b, o); o += 20
    label = np.frombuffer(b, '<f4', nl, o).copy(); o += 4 * nl
    (nr,) = struct.unpack_from('<i', b, o); o += 4
    rounds = []
    for _ in range(nr):
        (nk,) = struct.unpack_from('<i', b, o); o += 4
        ts = []
        for _ in range(nk):
            (nn,) = struct.unpack_from('<Q', b, o); o += 8
            ts.append(np.frombuffer(b, np.uint8, nn * 48, o).copy()); o += 48 * nn
        rounds.append(np.stack(ts))
    assert o == len(b)
    return dict(objective=obj, learning_rate=lr, num_class=nc, n_trees=nt, base_score=bs, label=label,
                trees=np.stack(rounds))


def logloss(objective, raw, y, label):
    """Mean negative log-likelihood from raw scores, evaluated in float64.  `y` holds the caller's label values,
    `label` the sorted distinct ones (class index = position).  None for objectives without class probabilities."""
    if objective == 'binary:logistic':
        cls = np.searchsorted(label, y).astype(np.float64)
        z = raw.astype(np.float64).reshape(-1)
        # -[c log s(z) + (1-c) log(1-s(z))] = softplus(z) - c z
        return float(np.mean(np.logaddexp(0.0, z) - cls * z))
    if objective in ('multi:softmax', 'multi:softprob'):
        k = label.size
        z = raw.astype(np.float64).reshape(k, -1)
        cls = np.searchsorted(label, y)
        lse = np.logaddexp.reduce(z, axis=0)
        return float(np.mean(lse - z[cls, np.arange(z.shape[1])]))
    return None


def metrics_of(log):
    return [float(x) for x in re.findall(r'\[\d+/\d+\] [^=]+ = ([-+0-9.eEnNaA]+)', log)]


def tree_view(trees_u8):
    r, k, nb = trees_u8.shape
    return trees_u8.reshape(r, k, nb // 48, 48).copy().view(NODE_DTYPE).reshape(r, k, nb // 48)


def spread(primary, others):
    """Largest distance of the further runs from the packed one.  Gains and node weights of the first tree are compared
    along the paths on which both runs split identically (common.walk_same_path); spread_parted_tree0 counts the nodes
    of the first tree at which some run chose another split (a near-tie decided by the order of the float atomics)."""
    from common import walk_same_path
    out = dict(spread_runs=len(others), spread_metric=0.0, spread_raw_max=0.0, spread_logloss=0.0,
               spread_gain_tree0=0.0, spread_root_gain=0.0, spread_weight_tree0=0.0, spread_parted_tree0=0,
               spread_first_diff_tree=-1)
    T = tree_view(primary['trees'])
    for o in others:
        n = min(len(primary['metric']), len(o['metric']))
        if n:
            out['spread_metric'] = max(out['spread_metric'], float(np.max(np.abs(np.asarray(primary['metric'][:n]) - np.asarray(o['metric'][:n])))))
        out['spread_raw_max'] = max(out['spread_raw_max'], float(np.max(np.abs(primary['raw'] - o['raw']))))
        if primary['logloss'] is not None:
            out['spread_logloss'] = max(out['spread_logloss'], abs(primary['logloss'] - o['logloss']))
        t = tree_view(o['trees'])
        w = walk_same_path(T[0, 0], t[0, 0])
        if w['gains'].size:
            out['spread_gain_tree0'] = max(out['spread_gain_tree0'], float(w['gains'].max()))
            out['spread_root_gain'] = max(out['spread_root_gain'], float(w['gains'][0]))
        if w['weights'].size:
            out['spread_weight_tree0'] = max(out['spread_weight_tree0'], float(w['weights'].max()))
        out['spread_parted_tree0'] = max(out['spread_parted_tree0'], len(w['parted']))
        for r in range(T.shape[0]):
            keys = ('is_valid', 'is_leaf', 'split_feature_id', 'split_bid', 'is_pruned')
            if any(not np.array_equal(T[r][f], t[r][f]) for f in keys):
                if out['spread_first_diff_tree'] < 0 or r < out['spread_first_diff_tree']:
                    out['spread_first_diff_tree'] = r
                break
    return out


def load_run(g, y):
    m = read_model(os.path.join(g, 'tgbm.model'))
    raw = np.fromfile(os.path.join(g, 'raw_pred.f32'), np.float32)
    log = open(os.path.join(g, 'log.txt')).read()
    return dict(model=m, trees=m['trees'], raw=raw, metric=metrics_of(log), logloss=logloss(m['objective'], raw, y, m['label']))


def bins_digest(g):
    d = os.path.join(g, 'bins_digest.npz')
    if os.path.exists(d):
        z = np.load(d)
        return z['sha256'], z['head'], int(z['n'])
    bins = np.fromfile(os.path.join(g, 'csr_bin_id.i32'), np.int32)
    return np.frombuffer(hashlib.sha256(bins.tobytes()).digest(), np.uint8), bins[:4096].copy(), bins.size


def multi_device_dumps(g, d):
    """Outputs of the reference's column-sharded builder (ref_harness with n_device = D > 1): per device its cut points
    and its dense matrix of local bin ids.  Returns the cut points of all features, their offsets, D and the global
    bin id of every stored value in CSR order -- the same form as the one-device dumps."""
    vals, ptrs, dense = [], [], []
    k = 0
    while os.path.exists(os.path.join(g, f'cut_val_d{k}.f32')):
        vals.append(np.fromfile(os.path.join(g, f'cut_val_d{k}.f32'), np.float32))
        ptrs.append(np.fromfile(os.path.join(g, f'cut_row_ptr_d{k}.i32'), np.int32))
        dense.append(np.fromfile(os.path.join(g, f'dense_bin_id_d{k}.u8'), np.uint8).reshape(d.n_rows, ptrs[-1].size - 1))
        k += 1
    cut_val = np.concatenate(vals)
    sizes = np.concatenate([np.diff(p) for p in ptrs])
    cut_ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    local = np.concatenate(dense, axis=1)
    rows = np.repeat(np.arange(d.n_rows), np.diff(d.row_ptr))
    lb = local[rows, d.col]
    assert lb.max() < 255 or (sizes.max() == 255 and (lb < 255).all()), 'a stored value without a bin'
    bins = (cut_ptr[d.col] + lb).astype(np.int32)
    return cut_val, cut_ptr, k, bins


def main(argv):
    src, reruns, out, shrink, prefix = None, [], HERE, False, None
    i = 0
    while i < len(argv):
        if argv[i] == '--rerun': reruns.append(argv[i + 1]); i += 2
        elif argv[i] == '--out': out = argv[i + 1]; i += 2
        elif argv[i] == '--shrink': shrink = True; i += 1
        elif argv[i] == '--prefix': prefix = argv[i + 1]; i += 2
        else: src = argv[i]; i += 1
    if src is None:
        raise SystemExit(__doc__)
    from make_inputs import CASES
    os.makedirs(out, exist_ok=True)
    for name in sorted(os.listdir(src)):
        g = os.path.join(src, name)
        if name not in CASES:
            continue
        if os.path.exists(os.path.join(g, 'cut_val_d0.f32')):  # a run of the column-sharded builder -> ref_multi_<case>.npz
            d = CASES[name][0]()
            cut_val, cut_ptr, n_dev, bins = multi_device_dumps(g, d)
            keys = dict(cut_val=cut_val, cut_ptr=cut_ptr, n_device=n_dev, n_bin_ids=bins.size, bins_head=bins[:4096].copy(),
                        bins_sha256=np.frombuffer(hashlib.sha256(bins.tobytes()).digest(), np.uint8))
            if os.path.exists(os.path.join(g, 'tgbm.model')):
                run = load_run(g, d.y)
                m = run['model']
                others = [load_run(os.path.join(r, name), d.y) for r in reruns if os.path.exists(os.path.join(r, name, 'tgbm.model'))]
                raw = run['raw']
                keys.update(spread(run, others) if others else dict(spread_runs=0))
                keys.update(trees=m['trees'], base_score=np.float32(m['base_score']), label=m['label'], num_class=m['num_class'],
                            learning_rate=np.float32(m['learning_rate']), metric=np.asarray(run['metric'], np.float32),
                            raw_pred_sample=raw[::37], raw_pred_sha256=np.frombuffer(hashlib.sha256(raw.tobytes()).digest(), np.uint8),
                            n_raw=raw.size, logloss=np.float64(run['logloss'] if run['logloss'] is not None else np.nan))
                print('multi', name, 'devices', n_dev, 'bins', bins.size, 'trees', m['trees'].shape, 'metric', run['metric'][-1],
                      {k: (float('%.3g' % v) if isinstance(v, float) else v) for k, v in keys.items() if k.startswith('spread')})
            else:  # the reference's training aborted on this case; its cut points and bin ids were dumped before
                print('multi', name, 'devices', n_dev, 'bins', bins.size, 'cut points and bin ids only')
            np.savez_compressed(os.path.join(out, f'ref_multi_{name}.npz'), **keys)
            continue
        if not os.path.exists(os.path.join(g, 'tgbm.model')):
            continue
        if not os.path.exists(os.path.join(g, 'cut_val.f32')):  # a run without cut points (tree_method=exact) -> ref_<prefix>_<case>.npz
            if not prefix:
                continue
            y = CASES[name][0]().y
            run = load_run(g, y)
            m = run['model']
            others = [load_run(os.path.join(r, name), y) for r in reruns if os.path.exists(os.path.join(r, name, 'tgbm.model'))]
            raw = run['raw']
            extra = spread(run, others) if others else dict(spread_runs=0)
            np.savez_compressed(
                os.path.join(out, f'ref_{prefix}_{name}.npz'), trees=m['trees'], base_score=np.float32(m['base_score']),
                label=m['label'], num_class=m['num_class'], learning_rate=np.float32(m['learning_rate']),
                metric=np.asarray(run['metric'], np.float32), raw_pred_sample=raw[::37],
                raw_pred_sha256=np.frombuffer(hashlib.sha256(raw.tobytes()).digest(), np.uint8), n_raw=raw.size,
                logloss=np.float64(run['logloss'] if run['logloss'] is not None else np.nan), **extra)
            print(prefix, name, 'trees', m['trees'].shape, 'metric', run['metric'][-1] if run['metric'] else None,
                  {k: (float('%.3g' % v) if isinstance(v, float) else v) for k, v in extra.items()})
            continue
        if not os.path.exists(os.path.join(g, 'cut_val.f32')):
            continue
        if shrink and os.path.exists(os.path.join(g, 'csr_bin_id.i32')):
            sha, head, n = bins_digest(g)
            np.savez(os.path.join(g, 'bins_digest.npz'), sha256=sha, head=head, n=n)
            os.remove(os.path.join(g, 'csr_bin_id.i32'))
        y = CASES[name][0]().y
        run = load_run(g, y)
        m = run['model']
        others = [load_run(os.path.join(r, name), y) for r in reruns if os.path.exists(os.path.join(r, name, 'tgbm.model'))]
        sha, head, n_bins = bins_digest(g)
        raw = run['raw']
        extra = spread(run, others) if others else dict(spread_runs=0)
        np.savez_compressed(
            os.path.join(out, f'ref_{name}.npz'),
            cut_val=np.fromfile(os.path.join(g, 'cut_val.f32'), np.float32),
            cut_ptr=np.fromfile(os.path.join(g, 'cut_row_ptr.i32'), np.int32),
            bins_sha256=sha, bins_head=head, n_bin_ids=n_bins, trees=m['trees'], base_score=np.float32(m['base_score']),
            label=m['label'], num_class=m['num_class'], learning_rate=np.float32(m['learning_rate']),
            metric=np.asarray(run['metric'], np.float32),
            raw_pred_sample=raw[::37], raw_pred_sha256=np.frombuffer(hashlib.sha256(raw.tobytes()).digest(), np.uint8),
            n_raw=raw.size, logloss=np.float64(run['logloss'] if run['logloss'] is not None else np.nan), **extra)
        print(name, 'bins', n_bins, 'trees', m['trees'].shape, 'metric', run['metric'][-1] if run['metric'] else None,
              'logloss', run['logloss'], {k: (float('%.3g' % v) if isinstance(v, float) else v) for k, v in extra.items()})


if __name__ == '__main__':
    main(sys.argv[1:])
