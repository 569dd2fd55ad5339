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


def compare_tree_decisive(ref, mine, gain2, rel_margin=1e-4, min_child_weight=None):
    """Walks two trees of the same shape from the root.  Where both split on the same (feature, bin) the walk
    continues into both children; where they differ, the node must be a near-tie in `mine` (runner-up gain within
    rel_margin of the best), otherwise it is reported.  With `min_child_weight`: also excused is a node where `ref` took
    `mine`'s runner-up while a child of `mine`'s own choice sits within 16 ulps of the node's sum of the hessian threshold -- the candidate
    passes `h >= min_child_weight` on one side and fails it on the other by the last bits of a float sum.
    Returns (#nodes compared equal, list of real mismatches)."""
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
        if a_split != b_split or (a_split and (a['split_feature_id'] != b['split_feature_id'] or a['split_bid'] != b['split_bid'] or
                                               a['split_value'] != b['split_value'])):   # (the exact builder has no bins)
            g = max(float(b['gain']), float(a['gain']), 1e-30)
            tie = abs(float(b['gain']) - float(gain2[i])) <= rel_margin * g or g < 1e-3
            if not tie and min_child_weight is not None and b_split and b['lch_index'] > 0:
                h_min = min(float(mine[b['lch_index']]['sum_h']), float(mine[b['rch_index']]['sum_h']))
                # a child's sum is the node's minus the sibling's: its error is a few ulps of the NODE's sum
                edge = max(2e-3 * min_child_weight, 16 * float(np.spacing(np.float32(abs(float(b['sum_h']))))))
                tie = abs(h_min - min_child_weight) <= edge and abs(float(a['gain']) - float(gain2[i])) <= rel_margin * g
            if not tie:
                bad.append(i)
            continue
        same += 1
        if a_split and a['lch_index'] > 0 and not (leaf_a and leaf_b and a['lch_index'] >= len(ref)):
            if a['lch_index'] < len(ref):
                stack.extend([int(a['lch_index']), int(a['rch_index'])])
    return same, bad


def gain_condition(n, lam=1.0):
    """How strongly rounding errors of the histogram sums are amplified in a node's split gain: the gain is the
    difference  lg^2/(lh+lam) + rg^2/(rh+lam) - pg^2/(ph+lam)  of terms that can be orders of magnitude larger than
    itself.  Computed from the node record alone; the children's sums are not needed because the two child terms add
    up to gain + parent term."""
    parent = float(n['sum_g']) ** 2 / (float(n['sum_h']) + lam)
    g = max(float(n['gain']), 1e-30)
    return (g + 2.0 * parent) / g


def walk_same_path(a, b, same_default=False, lam=1.0):
    """Walks two trees from the root for as long as both split on the same (feature, bin) -- with same_default also in
    the same default direction: on a feature without missing values the direction is decided by the float residue
    node.sum - sum of the bins, and it decides which child receives that residue.  Returns the relative gain differences
    of the identically split nodes with their gain condition numbers, the weight differences of every node reached
    that way (relative to max(|weight|, 1 % of the tree's largest weight): a weight -G/(H+lambda) near zero is a
    cancellation and has no meaningful relative error) and the nodes where the two trees part."""
    gains, conds, weights, parted = [], [], [], []
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
            conds.append(gain_condition(x, lam))
            if same_default and bool(x['default_right']) != bool(y['default_right']):
                parted.append(i)
                continue
            # a split whose children were pruned back keeps its fields; children beyond the table do not exist
            if x['lch_index'] < len(a):
                stack.extend([int(x['lch_index']), int(x['rch_index'])])
    return dict(gains=np.asarray(gains), conds=np.asarray(conds), weights=np.asarray(weights), parted=parted)


# ---- how exactly can two runs of the same float arithmetic agree? ----------------------------------------------------
# Below the root every histogram is a difference: the larger child of a pair is parent - smaller child
# (hist_tree_builder_single.cu:538-540), level after level.  The rounding noise of the root's sums -- a few ulps of the
# tree's whole gradient mass -- is therefore inherited as an ABSOLUTE error by every descendant, however small its own
# sums are.  Two runs that differ only in the order of their float additions (two runs of the reference, or of the fp32
# mode here) agree on a node's sums to about  SUM_NOISE_ULPS * 2^-24 * (sum over all rows of |g|, of h),  and on the
# quantities derived from them to that error times the derivative: d gain / d G = 2 G/(H+lambda) = -2 w for each of
# the three terms of the gain, d gain / d H = -w^2, d w / d G = -1/(H+lambda), d w / d H = -w/(H+lambda).
SUM_NOISE_ULPS = 8.0


def sum_noise(gh_rows, n_max=0):
    """(dG, dH): absolute uncertainty of a histogram sum of the tree grown on gradient pairs gh_rows[n][2];
    n_max = rows in the most populated bin."""
    u = max(SUM_NOISE_ULPS, 0.5 * float(np.sqrt(n_max))) * 2.0 ** -24
    return u * float(np.sum(np.abs(gh_rows[:, 0].astype(np.float64)))), u * float(np.sum(np.abs(gh_rows[:, 1].astype(np.float64))))


def gain_noise(tree, i, dG, dH):
    """Absolute uncertainty of node i's gain under sum errors (dG, dH)."""
    n = tree[i]
    ws = [abs(float(n['base_weight']))]
    for c in (int(n['lch_index']), int(n['rch_index'])):
        if 0 < c < len(tree):
            ws.append(abs(float(tree[c]['base_weight'])))
    return sum(2.0 * w * dG + w * w * dH for w in ws)


def weight_noise(tree, i, dG, dH, lam=1.0):
    n = tree[i]
    return (dG + abs(float(n['base_weight'])) * dH) / (float(n['sum_h']) + lam)


def compare_with_noise(ref, mine, dG, dH, rel=1e-5, lam=1.0, runner_up=None):
    """Walks two trees along identically split paths (same feature, bin and default direction) and checks every node:
    |gain difference| <= rel * gain + gain_noise, |weight difference| <= rel * |weight| + weight_noise.
    Where the trees part, the node must be a near-tie: with `runner_up` (the second-best |gain| of every node in `ref`'s
    run) the best and the second-best gain are within the gain noise of each other.  Returns a dict with the number of
    nodes compared, the worst ratios difference / tolerance and the nodes that broke a rule."""
    out = dict(compared=0, worst_gain=0.0, worst_weight=0.0, bad_gain=[], bad_weight=[], bad_split=[], parted=[],
               ratios_gain=[], ratios_weight=[])
    stack = [0]
    while stack:
        i = stack.pop()
        x, y = ref[i], mine[i]
        if not x['is_valid'] or not y['is_valid']:
            if bool(x['is_valid']) != bool(y['is_valid']):
                out['bad_split'].append(i)
            continue
        out['compared'] += 1
        tw = rel * abs(float(x['base_weight'])) + weight_noise(ref, i, dG, dH, lam)
        rw = abs(float(x['base_weight']) - float(y['base_weight'])) / max(tw, 1e-30)
        out['worst_weight'] = max(out['worst_weight'], rw)
        out['ratios_weight'].append(rw)
        if rw > 1.0:
            out['bad_weight'].append(i)
        xs = x['split_feature_id'] >= 0 and x['gain'] > 0 and x['lch_index'] > 0
        ys = y['split_feature_id'] >= 0 and y['gain'] > 0 and y['lch_index'] > 0
        noise = max(gain_noise(ref, i, dG, dH), gain_noise(mine, i, dG, dH))
        if xs != ys or (xs and (x['split_feature_id'] != y['split_feature_id'] or x['split_bid'] != y['split_bid'])):
            out['parted'].append(i)
            g = max(float(x['gain']), float(y['gain']))
            if runner_up is not None:
                second = float(runner_up[i])
                near_tie = abs(float(x['gain']) - second) <= rel * g + 2 * noise or g <= 1e-6 + 2 * noise
                if not near_tie:
                    out['bad_split'].append(i)
            continue
        if xs:
            tg = rel * abs(float(x['gain'])) + noise
            rg = abs(float(x['gain']) - float(y['gain'])) / tg
            out['worst_gain'] = max(out['worst_gain'], rg)
            out['ratios_gain'].append(rg)
            if rg > 1.0:
                out['bad_gain'].append(i)
            if bool(x['default_right']) != bool(y['default_right']) and x['lch_index'] < len(ref):
                # the residue went to the other child: the subtrees are comparable only if it is below the noise
                cx, cy = ref[int(x['lch_index'])], mine[int(y['lch_index'])]
                if abs(float(cx['sum_g']) - float(cy['sum_g'])) > dG or abs(float(cx['sum_h']) - float(cy['sum_h'])) > dH:
                    out['parted'].append(i)
                    continue
            if x['lch_index'] < len(ref):
                stack.extend([int(x['lch_index']), int(x['rch_index'])])
    return out


def within_noise(r, hard=4.0, share=0.9):
    """The noise is random: of the nodes compared by compare_with_noise, at least `share` must sit inside their tolerance
    and none further out than `hard` times it."""
    ok = True
    for key in ('ratios_gain', 'ratios_weight'):
        v = np.asarray(r[key])
        if v.size:
            ok = ok and float(v.max()) <= hard and float(np.mean(v <= 1.0)) >= share
    return ok
