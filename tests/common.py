"""Helpers shared by the parity tests."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')

NODE_DTYPE = np.dtype([('final_id', '<i4'), ('lch_index', '<i4'), ('rch_index', '<i4'), ('parent_index', '<i4'),
                       ('gain', '<f4'), ('base_weight', '<f4'), ('split_feature_id', '<i4'), ('split_value', '<f4'),
                       ('split_bid', 'u1'), ('default_right', 'u1'), ('is_leaf', 'u1'), ('is_valid', 'u1'),
                       ('is_pruned', 'u1'), ('pad', 'u1', (3,)), ('sum_g', '<f4'), ('sum_h', '<f4')])


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, f'ref_{name}.npz'))
    g = {k: z[k] for k in z.files}
    r, k, nb = g['trees'].shape
    g['trees'] = g['trees'].reshape(r, k, nb // 48, 48).copy().view(NODE_DTYPE).reshape(r, k, nb // 48)
    return g


def compare_tree_decisive(ref, mine, gain2, rel_margin=1e-4):
    """Walks two trees of the same shape from the root.  Where both split on the same (feature, bin) the walk
    continues into both children; where they differ, the node must be a near-tie in `mine` (runner-up gain within
    rel_margin of the best), otherwise it is reported.  Returns (#nodes compared equal, list of real mismatches)."""
    bad, same = [], 0
    stack = [0]
    while stack:
        i = stack.pop()
        a, b = ref[i], mine[i]
        if not a['is_valid'] and not b['is_valid']:
            continue
        leaf_a = bool(a['is_leaf']) or a['lch_index'] < 0
        leaf_b = bool(b['is_leaf']) or b['lch_index'] < 0
        # a parent pruned back to a leaf keeps its split fields: compare the unpruned decision
        a_split = a['split_feature_id'] >= 0 and a['gain'] > 0
        b_split = b['split_feature_id'] >= 0 and b['gain'] > 0
        if a_split != b_split or (a_split and (a['split_feature_id'] != b['split_feature_id'] or a['split_bid'] != b['split_bid'])):
            g = max(float(b['gain']), float(a['gain']), 1e-30)
            tie = abs(float(b['gain']) - float(gain2[i])) <= rel_margin * g or g < 1e-3
            if not tie:
                bad.append(i)
            continue
        same += 1
        if a_split and a['lch_index'] > 0 and not (leaf_a and leaf_b and a['lch_index'] >= len(ref)):
            if a['lch_index'] < len(ref):
                stack.extend([int(a['lch_index']), int(a['rch_index'])])
    return same, bad


def walk_same_path(a, b):
    """Walks two trees from the root for as long as both split on the same (feature, bin).  Returns the relative gain
    differences of the identically split nodes, the weight differences of every node reached that way (relative to
    max(|weight|, 1 % of the tree's largest weight): a weight -G/(H+lambda) near zero is a cancellation and has no
    meaningful relative error) and the nodes where the two trees part."""
    gains, weights, parted = [], [], []
    wfloor = 0.01 * float(np.max(np.abs(a['base_weight'][a['is_valid'] != 0]))) if (a['is_valid'] != 0).any() else 0.0
    stack = [0]
    while stack:
        i = stack.pop()
        x, y = a[i], b[i]
        if not x['is_valid'] or not y['is_valid']:
            if bool(x['is_valid']) != bool(y['is_valid']):
                parted.append(i)
            continue
        weights.append(abs(float(x['base_weight']) - float(y['base_weight'])) / max(abs(float(x['base_weight'])), wfloor, 1e-30))
        xs = x['split_feature_id'] >= 0 and x['gain'] > 0 and x['lch_index'] > 0
        ys = y['split_feature_id'] >= 0 and y['gain'] > 0 and y['lch_index'] > 0
        if xs != ys or (xs and (x['split_feature_id'] != y['split_feature_id'] or x['split_bid'] != y['split_bid'])):
            parted.append(i)
            continue
        if xs:
            gains.append(abs(float(x['gain']) - float(y['gain'])) / abs(float(x['gain'])))
            # a split whose children were pruned back keeps its fields; children beyond the table do not exist
            if x['lch_index'] < len(a):
                stack.extend([int(x['lch_index']), int(x['rch_index'])])
    return dict(gains=np.asarray(gains), weights=np.asarray(weights), parted=parted)
