#!/usr/bin/env python
"""Benchmark of the histogram tree-building path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c1|c2|c3|c4|c5] [--hist-mode fp32|exact|both]

Default workload (config 2): the Higgs-shaped configuration, 10.5 M rows x 28 dense float32 features,
binary:logistic, depth 8, 255 bins, learning rate 0.1 -- seeded synthetic data with that shape and value
distribution.  A step is one boosting round.  With N > 1 the rows are sharded over the ranks (one process per GPU,
launched by torch.distributed.run) and the total work stays fixed ("strong" scaling).

Prints one JSON line on rank 0:
  value     seconds per 100 boosting rounds for the boosting loop with the bin matrix resident in HBM (the scope of
            the reference's own "training time" line, src/thundergbm/trainer.cu:42-50), in the library's default
            histogram arithmetic (fp32: the reference's own, one float accumulator per bin)
  deterministic_mode   the same loop in the exact fixed-point mode (bit-identical from run to run and for any number
            of GPUs), with the roofline of its histogram kernel
  e2e       the same unit through the reference's C entry point (sparse_train_scikit) with host CSR buffers: copies,
            cut points, binning, boosting and the model read-back inside the timed region; median of --e2e-repeats
            calls of K rounds each.  With N > 1 rank 0 makes the call with n_device = N (one host thread per GPU
            inside the call), the other ranks wait
  roofline  histogram-build kernels of either mode: algorithmic bytes / summed CUDA-event time, against the measured
            HBM copy bandwidth.  The per-kernel events are recorded in a second pass of up to 20 rounds on the same
            booster directly after the timed region (there a round is one CUDA graph launch and no event can be
            recorded between its kernels)
  predict   device time of predict_raw of the trained trees over the rank's rows
  cpu_baseline  the CPU oracle on this box's host cores, full row count, a few rounds
`--impl reference` times the reference's algorithm on the host cores instead (the reference itself has no CPU
implementation, so this is the CPU restatement under oracle/) and, beside it, the reference's own GPU build.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from thundergbm_b200 import synth  # noqa: E402

COMMON = dict(gamma=1.0, min_child_weight=1.0, **{'lambda': 1.0})
# name -> (rows, maker(rows, lo, hi), parameters, description); shapes and parameters of the five configurations
WORKLOADS = {
    'c1': (10_000, lambda n, lo, hi: synth.dense_regression(n, 32, seed=0).rows(lo, hi),
           dict(objective='reg:linear', depth=6, max_num_bin=255, learning_rate=1.0, **COMMON),
           'dense regression 10k x 32 f32, reg:linear, depth 6, 255 bins, lr 1.0, lambda 1'),
    'c2': (10_500_000, lambda n, lo, hi: synth.higgs_like(n, seed=1, rows=(lo, hi)),
           dict(objective='binary:logistic', depth=8, max_num_bin=255, learning_rate=0.1, **COMMON),
           'higgs-shape 10.5M x 28 f32, binary:logistic, depth 8, 255 bins, lr 0.1, lambda 1'),
    'c3': (581_012, lambda n, lo, hi: synth.covtype_like(n, seed=2).rows(lo, hi),
           dict(objective='multi:softmax', depth=8, max_num_bin=255, learning_rate=0.1, **COMMON),
           'covtype-shape 581012 x 54 f32, multi:softmax 7 classes (7 trees per round), depth 8, 255 bins, lr 0.1'),
    'c4': (1_000_000, lambda n, lo, hi: synth.sparse_binary(n, 100_000, seed=3).rows(lo, hi),
           dict(objective='binary:logistic', depth=6, max_num_bin=64, learning_rate=0.3, **COMMON),
           'sparse CSR 1M x 100k, nnz/row Poisson(40), binary:logistic, depth 6, 64 bins, lr 0.3'),
    'c5': (2_270_000, None,
           dict(objective='rank:ndcg', depth=8, max_num_bin=255, learning_rate=0.1, **COMMON),
           'mslr-shape 2.27M x 136 f32 in query groups of Poisson(120), rank:ndcg, depth 8, 255 bins, lr 0.1'),
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the histogram kernel of either mode on config 2, from the
# ncu captures summarised under profiles/ (None: no capture of that kernel yet)
NCU_TRAFFIC_BYTES_PER_LAUNCH = {'exact': 363.1e6, 'fp32': 443.8e6}


def make_shard(config, n_rows, rank, world):
    rows_default, maker, params, desc = WORKLOADS[config]
    if config == 'c5':  # shards are cut at query-group boundaries
        d = synth.mslr_like(n_rows, 136, seed=4)
        ends = np.cumsum(d.group)
        cut = [0] + [int(ends[np.searchsorted(ends, n_rows * r // world, side='left')]) if r < world else n_rows for r in range(1, world + 1)]
        cut[-1] = n_rows
        lo, hi = cut[rank], cut[rank + 1]
        s = d.rows(lo, hi)
        starts = ends - d.group
        s.group = d.group[(starts >= lo) & (ends <= hi)]
        return s, lo, hi
    lo, hi = n_rows * rank // world, n_rows * (rank + 1) // world
    return maker(n_rows, lo, hi), lo, hi


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


def logloss_terms(objective, raw, y, label):
    """Sum of the negative log-likelihoods of the rows under raw scores raw[K][n] (float64) and the row count;
    None for objectives without class probabilities.  The reference logs only error / accuracy, so this is computed
    by the harness from raw scores, the same way for both sides."""
    if objective == 'binary:logistic':
        cls = np.searchsorted(label, y).astype(np.float64)
        z = raw.astype(np.float64).reshape(-1)
        return float(np.sum(np.logaddexp(0.0, z) - cls * z)), z.size
    if objective in ('multi:softmax', 'multi:softprob'):
        z = raw.astype(np.float64).reshape(len(label), -1)
        cls = np.searchsorted(label, y)
        return float(np.sum(np.logaddexp.reduce(z, axis=0) - z[cls, np.arange(z.shape[1])])), z.shape[1]
    return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index
        self.first = 0
        self.last = None

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.gpu), '--query-gpu=' + self.Q,
                                          '--format=csv,noheader,nounits', '-lms', '20'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def mark(self):
        """Samples before this call (tool start-up, warm-up) are dropped."""
        self.first = len(self.rows)

    def mark_end(self):
        self.last = len(self.rows) + 2  # the tool prints every 20 ms: keep what was sampled up to now

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows[self.first:self.last]:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (('hw_slowdown', 5), ('hw_thermal_slowdown', 6), ('sw_thermal_slowdown', 7),
                              ('sw_power_cap', 8)):
                if len(r) > col and r[col].lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        return {'sm_mhz': float(np.median(sm)), 'sm_max_mhz': max(mx), 'reasons': sorted(reasons), 'samples': len(sm)}


def oracle_run(config, n_rows, n_trees: int, threads: int):
    """The CPU restatement on the FULL workload (all rows), exact mode (its histogram build is the multi-threaded one);
    per-round seconds."""
    sys.path.insert(0, os.path.join(ROOT, 'oracle'))
    import tgbm_oracle as orc
    d, _, _ = make_shard(config, n_rows, 0, 1)
    return orc.train(d, n_trees=n_trees, hist_mode=1, n_threads=threads, **WORKLOADS[config][2])


def reference_gpu_run(config, n_rows, n_trees: int, repeat: bool = True):
    """The reference itself (built by oracle/build_ref.sh into oracle/_ref/, GPU-only code) on the full workload on
    cuda:0 -- an extra figure beside the CPU arm: its own 'training time' (src/thundergbm/trainer.cu:42-50), the
    wall clock of TreeTrainer::train including its set-up, its final training metric and, for classification, the
    logloss of its raw scores.  A dict with 'unavailable' when the build is absent or the run fails."""
    import re
    import tempfile
    harness = os.path.join(ROOT, 'oracle', '_ref', 'bin', 'ref_harness')
    if not os.path.exists(harness):
        return {'unavailable': 'oracle/_ref/bin/ref_harness not built'}
    try:
        import torch
        if not torch.cuda.is_available():
            return {'unavailable': 'no GPU'}
        params = WORKLOADS[config][2]
        d, _, _ = make_shard(config, n_rows, 0, 1)
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, 'w.tgbin')
            synth.write_tgbin(d, path)
            env = dict(os.environ)
            env['LD_LIBRARY_PATH'] = os.path.join(ROOT, 'oracle', '_ref', 'lib') + ':' + env.get('LD_LIBRARY_PATH', '')
            cmd = [harness, path, tmp, 'objective=' + params['objective'], f"depth={params['depth']}", f'n_trees={n_trees}',
                   f"max_num_bin={params['max_num_bin']}", f"learning_rate={params['learning_rate']}", 'tree_method=hist', 'dump_bins=0']
            def one_run():
                out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200)
                if out.returncode != 0:
                    return None
                raw = np.fromfile(os.path.join(tmp, 'raw_pred.f32'), np.float32)
                t_train = float(re.search(r'training time = ([0-9.eE+-]+)', out.stdout).group(1))
                t_wall = float(re.search(r'train_wall_s ([0-9.eE+-]+)', out.stdout).group(1))
                vals = re.findall(r'\[(\d+)/\d+\] [^=]+ = ([0-9.eE+-]+)', out.stdout)
                ll = logloss_terms(params['objective'], raw, d.y, label)
                return t_train, t_wall, float(vals[-1][1]) if vals else None, ll[0] / ll[1] if ll else None
            label = np.unique(d.y.astype(np.int32)).astype(np.float32)
            runs = [one_run() for _ in range(2 if repeat else 1)]
        if any(r is None for r in runs):
            return {'unavailable': 'ref_harness failed'}
        t_train, t_wall, metric, ll = runs[0]
        res = {'value': t_train * 100.0 / n_trees, 'unit': 's/100 rounds', 'rounds': n_trees,
               # a 100-round job: its set-up once (wall clock of TreeTrainer::train minus its boosting loop) + 100 rounds
               'e2e_value': (t_wall - t_train) + t_train * 100.0 / n_trees, 'setup_s': t_wall - t_train,
               'final_train_metric': metric, 'final_train_logloss': ll,
               'kind': 'the reference built for sm_100a by oracle/build_ref.sh, same workload, 1 GPU'}
        if len(runs) > 1:  # how far two runs of the reference itself end up from each other (unordered float atomics)
            res['second_run'] = {'value': runs[1][0] * 100.0 / n_trees, 'final_train_metric': runs[1][2], 'final_train_logloss': runs[1][3]}
            if metric is not None and runs[1][2] is not None:
                res['spread_metric'] = abs(metric - runs[1][2])
            if ll is not None and runs[1][3] is not None:
                res['spread_logloss'] = abs(ll - runs[1][3])
        return res
    except Exception as e:  # noqa: BLE001 -- an extra figure must never break the arm
        return {'unavailable': f'{type(e).__name__}: {e}'[:200]}


def run_reference(args):
    """Reference arm: the reference's algorithm on the host cores (CPU restatement, all cores, all rows)."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    rows_default, _, params, desc = WORKLOADS[args.config]
    n_rows = args.rows or rows_default
    cores = os.cpu_count() or 1
    k, w = args.steps, args.warmup
    k_eff = min(k, 20)  # bounded: at most 20 timed rounds
    r = oracle_run(args.config, n_rows, w + k_eff, cores)
    per_round = np.asarray(r.round_seconds[w:w + k_eff])
    s_round = float(per_round.mean())
    sample = (f'all {n_rows} rows, {k_eff} timed rounds after {w} warm-up on {cores} threads; seconds/round x 100 '
              f'(set-up of {r.init_seconds:.1f} s -- cut points, bin ids -- not included, as in the reference\'s own timing scope)')
    line = {
        'impl': 'reference', 'metric': 'Higgs-shape train s/100 trees', 'value': s_round * 100.0, 'unit': 's/100 trees',
        'n_gpus': args.gpus, 'steps': k, 'warmup': w, 'ms_per_step': s_round * 1e3,
        'higher_is_better': False, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64', 'data': 'synthetic',
        'config': {'workload': desc if n_rows == rows_default else desc + f' [rows overridden: {n_rows}]',
                   'note': 'the reference is GPU-only; this arm is its CPU restatement (oracle/) on the host cores',
                   'final_train_metric': float(r.metric[-1])},
        'cpu_baseline': {'value': s_round * 100.0, 'unit': 's/100 trees', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': s_round * 100.0, 'unit': 's/100 trees', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
        # warm-up + timed rounds, so that its final metric and logloss describe the same number of rounds as the
        # `final_train_*` figures of the repo's own arm
        'reference_gpu': reference_gpu_run(args.config, n_rows, w + k),
    }
    print(json.dumps(line), flush=True)


def e2e_child(args):
    """The end-to-end leg, run by rank 0 in a process of its own (so that a fault in it cannot take the benchmark line with it
    and the parent can bound its time): K rounds through the reference's C entry point with host CSR buffers in pinned memory,
    n_device = the number of GPUs of the run.  Prints one JSON object."""
    import torch
    from thundergbm_b200 import _lib
    rows_default, _, PARAMS, desc = WORKLOADS[args.config]
    n_rows = args.rows or rows_default
    k, world = args.steps, args.gpus
    lib = _lib.lib()
    full = make_shard(args.config, n_rows, 0, 1)[0]

    def pin(a, dt):  # the caller's CSR sits in pinned host memory (page-locked once, outside the timed region)
        if args.e2e_pageable:  # ... or stays pageable, as the arrays of a NumPy caller are
            return np.ascontiguousarray(a, dt)
        return torch.from_numpy(np.ascontiguousarray(a, dt)).pin_memory().numpy()
    val = pin(full.val, np.float32); rp = pin(full.row_ptr, np.int32)
    col = pin(full.col, np.int32); y = pin(full.y, np.float32)
    grp = np.ascontiguousarray(full.group, np.int32)

    def scikit_call(n_trees):
        model = C.c_void_p(None)
        num_class = C.c_int(2); per_iter = C.c_int(0)
        group_label = (C.c_float * 64)()
        t_a = time.perf_counter()
        lib.sparse_train_scikit(full.n_rows, val.ctypes.data_as(C.c_void_p), rp.ctypes.data_as(C.c_void_p),
                                col.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), PARAMS['depth'], n_trees, world,
                                PARAMS['min_child_weight'], PARAMS['lambda'], PARAMS['gamma'], PARAMS['max_num_bin'], 0,
                                1.0, 0, 1, PARAMS['learning_rate'], PARAMS['objective'].encode(), C.byref(num_class),
                                b'hist', C.byref(model), C.byref(per_iter), group_label,
                                grp.ctypes.data_as(C.c_void_p) if grp.size else None, int(grp.size))
        dt = time.perf_counter() - t_a
        if not model.value:
            raise SystemExit('sparse_train_scikit failed: ' + lib.tgbm_last_error().decode())
        n_nodes = C.c_int(0)
        lib.get_n_nodes(C.byref(model), C.byref(n_nodes), 1, 1)
        lib.model_free(C.byref(model))
        return dt, per_iter.value, n_nodes.value
    scikit_call(3)  # untimed warm-up of the same entry point
    # The metric is the time of a 100-round job: a call trains at least 100 rounds, so that the once-per-call work (copies,
    # cut points, binning) weighs what it weighs in that job instead of being scaled up with a short run.
    n = max(k, 100)
    times = []
    for _ in range(max(1, args.e2e_repeats)):
        dt, per_iter, n_nodes = scikit_call(n)
        times.append(dt)
    h2d = val.nbytes + rp.nbytes + col.nbytes + y.nbytes
    d2h = n * per_iter * n_nodes * 48
    print(json.dumps({'value': float(np.median(times)) * 100.0 / n, 'unit': 's/100 trees', 'h2d_bytes_per_step': h2d / n,
                      'd2h_bytes_per_step': d2h / n, 'calls_s': times, 'rounds_per_call': n,
                      'hist_mode': 'fp32 (library default on this entry point)',
                      'note': f'median wall clock of {len(times)} calls of sparse_train_scikit(n_device={world}) with {n} rounds each, '
                              f'CSR in {"pageable" if args.e2e_pageable else "pinned"} host memory; the calls run in a child process of rank 0'}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=100)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours')
    ap.add_argument('--config', default='c2', choices=sorted(WORKLOADS))
    ap.add_argument('--hist-mode', default='both', choices=['fp32', 'exact', 'both'],
                    help='fp32 is the headline (library default); both adds the deterministic mode\'s figures')
    ap.add_argument('--rows', type=int, default=0, help='override the row count (debugging only)')
    ap.add_argument('--e2e-repeats', type=int, default=3)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-predict', action='store_true')
    ap.add_argument('--e2e-child', action='store_true', help=argparse.SUPPRESS)
    ap.add_argument('--e2e-pageable', action='store_true', help='end-to-end leg with the host CSR in pageable memory instead of pinned')
    ap.add_argument('--e2e-timeout', type=float, default=300.0, help='seconds the end-to-end leg may take before it is given up')
    args = ap.parse_args()
    if args.e2e_child:
        e2e_child(args)
        return
    if args.impl == 'reference':
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    from thundergbm_b200 import _lib
    from thundergbm_b200.booster import Booster, Comm

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the histogram path has no CPU fallback')
    torch.cuda.set_device(local_rank)
    comm = None
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
        uid = [Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = Comm(uid[0], rank, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_max(x):
        t = torch.tensor([x], dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_sum(x):
        t = torch.tensor([x], dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    rows_default, _, PARAMS, desc = WORKLOADS[args.config]
    n_rows = args.rows or rows_default
    t0 = time.time()
    data, lo, hi = make_shard(args.config, n_rows, rank, world)
    t_gen = time.time() - t0
    k, w = args.steps, args.warmup
    k_prof = min(k, 20)  # rounds of the second, profiled pass
    label = np.unique(data.y.astype(np.int32)).astype(np.float32)
    peak, peak_kind = measured_peaks()

    def run_mode(mode, sampler=None):
        """Boosting loop with the bin matrix resident in HBM, in one histogram arithmetic."""
        t_a = time.time()
        b = Booster(data, comm=comm, n_trees=w + k + k_prof, profile=0, hist_mode=mode, **PARAMS)
        b.sync()
        t_init = time.time() - t_a
        b.boost(w)
        b.sync()
        launches_before = int(b.profile().kernel_launches)
        barrier()
        if sampler:
            sampler.mark()
        ms = b.boost_timed(k)  # the timed region: K rounds, CUDA events around them on the booster's stream
        if sampler:
            sampler.mark_end()
        barrier()
        ms_max = all_max(ms)
        launches_timed = int(b.profile().kernel_launches) - launches_before
        metrics_timed = b.metrics()
        ll = logloss_terms(PARAMS['objective'], b.ypred(), data.y, label)
        if ll is not None:
            ll = all_sum(ll[0]) / all_sum(ll[1])
        # Second pass for the roofline: per-kernel CUDA events on the same booster, directly after the timed region
        # (the events cost ~5 % of a step, so they stay out of `value`).
        b.set_profile(True)
        barrier()
        ms_prof = b.boost_timed(k_prof)
        barrier()
        prof = b.profile()
        info = b.info
        trees = b.trees() if rank == 0 else None
        b.close()
        gbs = lambda by, ms_: by / (ms_ * 1e-3) / 1e9 if ms_ > 0 else 0.0
        hist_gbs = gbs(prof.hist_bytes, prof.hist_ms)
        root_gbs = gbs(prof.hist_root_bytes, prof.hist_root_ms)
        part_gbs = gbs(prof.partition_bytes, prof.partition_ms)
        kernel = {'fp32': 'k_hist_f32 (one float accumulator per bin, vector reductions in L2; all levels)',
                  'exact': 'k_hist (shared-memory integer histograms; all levels)'}[mode]
        if info.csr_layout:
            kernel = kernel.replace('k_hist', 'k_hist_sparse')
        roof = {'bound': 'hbm', 'kernel': kernel, 'achieved': hist_gbs, 'peak': peak, 'unit': 'GB/s', 'frac': hist_gbs / peak,
                'peak_kind': peak_kind, 'traffic': NCU_TRAFFIC_BYTES_PER_LAUNCH[mode] if args.config == 'c2' and n_rows == rows_default and world == 1 else None,
                'launches': int(prof.hist_launches), 'avg_launch_us': prof.hist_ms * 1e3 / max(1, prof.hist_launches),
                'root_level_gbs': root_gbs, 'root_level_frac': root_gbs / peak,
                'partition_gbs': part_gbs, 'partition_frac': part_gbs / peak,
                'hist_share_of_step': prof.hist_ms / ms_prof if ms_prof > 0 else None,
                'partition_share_of_step': prof.partition_ms / ms_prof if ms_prof > 0 else None,
                'measured_on': f'{k_prof} rounds directly after the timed region, per-kernel CUDA events (ms_per_step there {ms_prof / k_prof:.3f})'}
        if mode == 'fp32':
            # the kernel is bound by the rate at which the L2 performs float reductions, not by HBM: say so with numbers
            reds = float(prof.hist_rows) * data.nnz / max(1, data.n_rows)  # one reduction per stored value of a processed row
            roof['limiter'] = 'L2 float-reduction rate (one red.global.add.v2.f32 per stored value of a row)'
            roof['reductions_per_s'] = reds / (prof.hist_ms * 1e-3) if prof.hist_ms > 0 else None
            roof['reduction_peak_per_s'] = 191e9
            roof['limiter_frac'] = roof['reductions_per_s'] / 191e9 if roof['reductions_per_s'] else None
            roof['reduction_peak_kind'] = 'microbenchmark on this pool: 10.5 M rows x 28 bare reductions into cells 256 bytes apart (1, 8 or 64 nodes: 190-192 G/s)'
        return dict(ms_max=ms_max, launches=launches_timed, roofline=roof, t_init=t_init, info=info, trees=trees, logloss=ll,
                    final_metric=float(metrics_timed[w + k - 1]) if len(metrics_timed) >= w + k else None)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()      # started before the warm-up so that the tool is already printing when timing starts
        t_wait = time.time()
        while not sampler.rows and time.time() - t_wait < 3.0:
            time.sleep(0.01)
    head_mode = 'exact' if args.hist_mode == 'exact' else 'fp32'
    head = run_mode(head_mode, sampler if rank == 0 else None)
    clocks = sampler.stop() if rank == 0 else None
    other = run_mode('exact') if args.hist_mode == 'both' else None
    info = head['info']

    # batch predict_raw of the trained trees over this rank's rows (Predictor::predict_raw): device time of the
    # traversal kernel; algorithmic bytes = nnz * 8 + rows * (4 + 4)
    predict = None
    if rank == 0 and not args.no_predict:
        from thundergbm_b200.booster import predict_raw
        trees = head['trees'][:45]   # at most 45 rounds: the size the predict figures in the design notes are quoted on
        runs = []
        for i in range(4):            # one untimed call (the first launch of a kernel loads it), then three timed ones
            _, pms = predict_raw(data, trees, PARAMS['learning_rate'], float(info.base_score), timing=True)
            if i:
                runs.append(pms)
        pms = float(np.median(runs))
        pbytes = data.nnz * 8.0 + data.n_rows * 8.0
        predict = {'kernel_ms': pms, 'calls_ms': runs, 'rows': data.n_rows, 'rounds': int(trees.shape[0]),
                   'gbs': pbytes / (pms * 1e-3) / 1e9 if pms > 0 else None,
                   'frac_of_hbm_peak': pbytes / (pms * 1e-3) / 1e9 / peak if pms > 0 else None}

    # ---- end to end through the reference's C entry point with host buffers ----------------------
    e2e = None
    if not args.no_e2e:
        barrier()
        # With N > 1 rank 0 makes the call (n_device = N: one host thread per GPU inside it) and the other ranks wait on
        # the HOST (a key in the rendezvous store), not inside a collective: their GPUs must be idle for the call.
        store = dist.distributed_c10d._get_default_store() if world > 1 else None
        if rank != 0 and store is not None:
            import datetime
            store.wait(['tgbm_e2e_done'], datetime.timedelta(seconds=3600))
        if rank == 0:
            cmd = [sys.executable, os.path.abspath(__file__), '--e2e-child', '--config', args.config, '--rows', str(n_rows), '--gpus', str(world),
                   '--steps', str(k), '--e2e-repeats', str(args.e2e_repeats)] + (['--e2e-pageable'] if args.e2e_pageable else [])
            env = {key: v for key, v in os.environ.items() if key not in ('RANK', 'LOCAL_RANK', 'WORLD_SIZE', 'MASTER_ADDR', 'MASTER_PORT',
                                                                          'TORCHELASTIC_RUN_ID', 'GROUP_RANK', 'ROLE_RANK', 'LOCAL_WORLD_SIZE')}
            try:
                out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.e2e_timeout)
                lines = [l for l in out.stdout.splitlines() if l.startswith('{')]
                if out.returncode == 0 and lines:
                    e2e = json.loads(lines[-1])
                else:
                    e2e = {'value': None, 'unit': 's/100 trees', 'h2d_bytes_per_step': None, 'd2h_bytes_per_step': None,
                           'error': (out.stderr or out.stdout)[-400:]}
            except subprocess.TimeoutExpired:
                e2e = {'value': None, 'unit': 's/100 trees', 'h2d_bytes_per_step': None, 'd2h_bytes_per_step': None,
                       'error': f'the end-to-end call did not finish within {args.e2e_timeout:.0f} s'}
            if store is not None:
                store.set('tgbm_e2e_done', '1')
        barrier()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    wl = desc if n_rows == rows_default else desc + f' [rows overridden: {n_rows}]'
    line = {
        'metric': 'Higgs-shape train s/100 trees', 'value': head['ms_max'] / k * 100.0 / 1e3, 'unit': 's/100 trees',
        'n_gpus': world, 'steps': k, 'warmup': w, 'ms_per_step': head['ms_max'] / k, 'higher_is_better': False,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32' if head_mode == 'fp32' else 'i64', 'data': 'synthetic',
        'config': {'workload': wl, 'config': args.config, 'hist_mode': head_mode,
                   'hist_mode_note': 'fp32 = float (g,h) added value by value into one accumulator per bin, the reference\'s arithmetic; '
                                     'exact = integer sums on a fixed-point grid (deterministic)',
                   'rows_per_gpu': hi - lo, 'parallelism': f'rows sharded over {world} GPU(s), NCCL all-reduce of level histograms',
                   'l2': 'inputs larger than L2 (bin data %.0f MB per GPU)' % (max(data.nnz, (hi - lo) * info.fpad) / 1e6),
                   'trees_per_round': int(info.trees_per_round), 'rounds_trained': w + k, 'final_train_metric': head['final_metric'],
                   'final_train_logloss': head['logloss'], 'init_s': head['t_init'], 'datagen_s': t_gen},
        'roofline': head['roofline'],
        'e2e': e2e, 'gpu_launches': head['launches'], 'clocks': clocks, 'predict': predict,
    }
    if other is not None:
        line['deterministic_mode'] = {'hist_mode': 'exact', 'value': other['ms_max'] / k * 100.0 / 1e3, 'unit': 's/100 trees',
                                      'ms_per_step': other['ms_max'] / k, 'dtype': 'i64', 'quant_bits': 18, 'gpu_launches': other['launches'],
                                      'final_train_metric': other['final_metric'], 'final_train_logloss': other['logloss'],
                                      'roofline': other['roofline']}
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        nt = 4
        r = oracle_run(args.config, n_rows, nt, cores)
        s_round = float(np.mean(r.round_seconds[1:]))
        line['cpu_baseline'] = {'value': s_round * 100.0, 'unit': 's/100 trees', 'cores': cores, 'kind': 'port',
                                'sample': f'all {n_rows} rows, {nt - 1} timed rounds after 1 warm-up on {cores} threads; seconds/round x 100'}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
