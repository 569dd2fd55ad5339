"""Packs what the reference produced on a B200 (tests/golden/run_reference.sh, outputs under
<out_dir>/<case>/) into small committed fixtures tests/golden/ref_<case>.npz:

  cut_val, cut_ptr     cut points of HistCut::get_cut_points_single, complete
  bins_sha256, bins_head   global bin ids of get_bin_ids: digest of the int32 array + its first 4096 entries
  trees                the model file's node tables (uint8 view of 48-byte records) [rounds, K, n_nodes*48]
  base_score, label, num_class
  metric               the per-round training metric the reference logged
  raw_pred_sample      every 37th raw prediction on the training rows + digest of the whole array

    python tests/golden/pack_golden.py <out_dir>      (the folder run_reference.sh wrote to)
"""
from __future__ import annotations

import hashlib
import os
import re
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


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


def main(src):
    for name in sorted(os.listdir(src)):
        g = os.path.join(src, name)
        if not os.path.exists(os.path.join(g, 'tgbm.model')) or not os.path.exists(os.path.join(g, 'cut_val.f32')):
            continue
        m = read_model(os.path.join(g, 'tgbm.model'))
        bins = np.fromfile(os.path.join(g, 'csr_bin_id.i32'), np.int32)
        raw = np.fromfile(os.path.join(g, 'raw_pred.f32'), np.float32)
        log = open(os.path.join(g, 'log.txt')).read()
        metric = [float(x) for x in re.findall(r'\[\d+/\d+\] [^=]+ = ([-+0-9.eEnNaA]+)', log)]
        np.savez_compressed(
            os.path.join(HERE, f'ref_{name}.npz'),
            cut_val=np.fromfile(os.path.join(g, 'cut_val.f32'), np.float32),
            cut_ptr=np.fromfile(os.path.join(g, 'cut_row_ptr.i32'), np.int32),
            bins_sha256=np.frombuffer(hashlib.sha256(bins.tobytes()).digest(), np.uint8), bins_head=bins[:4096],
            n_bin_ids=bins.size, trees=m['trees'], base_score=np.float32(m['base_score']), label=m['label'],
            num_class=m['num_class'], learning_rate=np.float32(m['learning_rate']), metric=np.asarray(metric, np.float32),
            raw_pred_sample=raw[::37], raw_pred_sha256=np.frombuffer(hashlib.sha256(raw.tobytes()).digest(), np.uint8),
            n_raw=raw.size)
        print(name, 'bins', bins.size, 'trees', m['trees'].shape, 'metric', metric[-1] if metric else None)


if __name__ == '__main__':
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, '..', '..', 'gpurun_out', 'golden'))
