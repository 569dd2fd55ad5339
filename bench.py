#!/usr/bin/env python
"""Benchmark of the histogram tree-building path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the Higgs-shaped configuration (10.5 M rows x 28 dense float32 features, binary:logistic,
depth 8, 255 bins, learning rate 0.1), seeded synthetic data with that shape and value distribution.
A step is one boosting round (one tree).  With N > 1 the rows are sharded over the ranks (one process
per GPU, launched by torch.distributed.run) and the total work stays fixed ("strong" scaling).

Prints one JSON line on rank 0:
  value     seconds per 100 trees for the boosting loop with the bin matrix resident in HBM
            (the scope of the reference's own "training time" line, src/thundergbm/trainer.cu:42-50)
  e2e       the same unit through the C ABI with host CSR buffers: copies, cut points, binning,
            boosting and the model read-back all inside the timed region
  roofline  histogram-build kernels: algorithmic bytes / summed CUDA-event time, against the measured
            HBM copy bandwidth.  The per-kernel events are recorded in a second pass of up to 20 trees on the
            same booster directly after the timed region: there a round is a single CUDA graph launch and no
            event can be recorded between its kernels
  predict   device time of predict_raw of the trained trees over the rank's rows
  cpu_baseline  the CPU oracle on a bounded row sample on this box's host cores
`--impl reference` times the reference's algorithm on the host cores instead (the reference itself has
no CPU implementation, so this is the CPU restatement under oracle/).
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

N_ROWS = 10_500_000
PARAMS = dict(objective='binary:logistic', depth=8, max_num_bin=255, learning_rate=0.1, gamma=1.0,
              min_child_weight=1.0, **{'lambda': 1.0})
WORKLOAD = 'higgs-shape 10.5M x 28 f32, binary:logistic, depth 8, 255 bins, lr 0.1, lambda 1'
SAMPLE_ROWS = 1_000_000
# dram__bytes_read.sum + dram__bytes_write.sum per k_hist launch, mean of the eight launches of one tree captured with
# ncu (root 425.0 MB, levels 1-7 331 to 397 MB; profiles/k_hist_higgs_10p5M_x28.md)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 363.1e6


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


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

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows[self.first:]:
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


def oracle_sample_run(n_trees: int, threads: int):
    """The CPU restatement on the first SAMPLE_ROWS rows of the workload; per-round seconds."""
    sys.path.insert(0, os.path.join(ROOT, 'oracle'))
    import tgbm_oracle as orc
    d = synth.higgs_like(N_ROWS, seed=1, rows=(0, SAMPLE_ROWS))
    r = orc.train(d, n_trees=n_trees, hist_mode=1, n_threads=threads, **PARAMS)
    return r


def reference_gpu_run(n_trees: int):
    """The reference itself (built by oracle/build_ref.sh into oracle/_ref/, GPU-only code) on the full workload on
    cuda:0 -- an extra figure beside the CPU arm: its own 'training time' (src/thundergbm/trainer.cu:42-50) and the
    wall clock of TreeTrainer::train including its set-up.  None when the build is absent or the run fails."""
    import re
    import tempfile
    harness = os.path.join(ROOT, 'oracle', '_ref', 'bin', 'ref_harness')
    if not os.path.exists(harness):
        return {'unavailable': 'oracle/_ref/bin/ref_harness not built'}
    try:
        import torch
        if not torch.cuda.is_available():
            return {'unavailable': 'no GPU'}
        d = synth.higgs_like(N_ROWS, seed=1)
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, 'c2.tgbin')
            synth.write_tgbin(d, path)
            del d
            env = dict(os.environ)
            env['LD_LIBRARY_PATH'] = os.path.join(ROOT, 'oracle', '_ref', 'lib') + ':' + env.get('LD_LIBRARY_PATH', '')
            cmd = [harness, path, tmp, 'objective=' + PARAMS['objective'], f"depth={PARAMS['depth']}", f'n_trees={n_trees}',
                   f"max_num_bin={PARAMS['max_num_bin']}", f"learning_rate={PARAMS['learning_rate']}", 'dump_bins=0']
            out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
        if out.returncode != 0:
            return {'unavailable': f'ref_harness exit {out.returncode}'}
        t_train = float(re.search(r'training time = ([0-9.eE+-]+)', out.stdout).group(1))
        t_wall = float(re.search(r'train_wall_s ([0-9.eE+-]+)', out.stdout).group(1))
        errs = re.findall(r'\[(\d+)/\d+\] test error = ([0-9.eE+-]+)', out.stdout)
        return {'value': t_train * 100.0 / n_trees, 'unit': 's/100 trees', 'trees': n_trees,
                'e2e_value': t_wall * 100.0 / n_trees, 'final_train_error': float(errs[-1][1]) if errs else None,
                'kind': 'the reference built for sm_100a by oracle/build_ref.sh, same workload, 1 GPU'}
    except Exception as e:  # noqa: BLE001 -- an extra figure must never break the arm
        return {'unavailable': f'{type(e).__name__}: {e}'[:200]}


def run_reference(args):
    """Reference arm: the reference's algorithm on the host cores (CPU restatement, all cores)."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    k, w = args.steps, args.warmup
    # bounded: at most 20 timed trees on the sample, scaled to rows and to 100 trees
    k_eff = min(k, 20)
    r = oracle_sample_run(w + k_eff, cores)
    per_round = np.asarray(r.round_seconds[w:w + k_eff])
    s_per_tree_sample = float(per_round.mean())
    s_per_100_full = s_per_tree_sample * 100.0 * (N_ROWS / SAMPLE_ROWS)
    sample = (f'{SAMPLE_ROWS} of {N_ROWS} rows, {k_eff} timed trees after {w} warm-up; seconds/tree scaled by '
              f'{N_ROWS / SAMPLE_ROWS:.1f} (rows) and to 100 trees')
    line = {
        'impl': 'reference', 'metric': 'Higgs-shape train s/100 trees', 'value': s_per_100_full, 'unit': 's/100 trees',
        'n_gpus': args.gpus, 'steps': k, 'warmup': w, 'ms_per_step': s_per_tree_sample * (N_ROWS / SAMPLE_ROWS) * 1e3,
        'higher_is_better': False, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64', 'data': 'synthetic',
        'config': {'workload': WORKLOAD, 'note': 'the reference is GPU-only; this arm is its CPU restatement on host cores'},
        'cpu_baseline': {'value': s_per_100_full, 'unit': 's/100 trees', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': s_per_100_full, 'unit': 's/100 trees', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
        'reference_gpu': reference_gpu_run(k),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=100)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours')
    ap.add_argument('--rows', type=int, default=N_ROWS, help='override the row count (debugging only)')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    args = ap.parse_args()
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

    n_rows = args.rows
    lo, hi = n_rows * rank // world, n_rows * (rank + 1) // world
    t0 = time.time()
    data = synth.higgs_like(n_rows, seed=1, rows=(lo, hi))
    t_gen = time.time() - t0
    k, w = args.steps, args.warmup

    # ---- boosting loop with the bin matrix resident in HBM --------------------------------------
    t0 = time.time()
    k_prof = min(k, 20)  # trees of the second, profiled pass
    b = Booster(data, comm=comm, n_trees=w + k + k_prof, profile=0, **PARAMS)
    b.sync()
    t_init = time.time() - t0
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()      # started before the warm-up so that the tool is already printing when timing starts
        t_wait = time.time()
        while not sampler.rows and time.time() - t_wait < 3.0:
            time.sleep(0.01)
    b.boost(w)
    b.sync()
    launches_before = int(b.profile().kernel_launches)
    barrier()
    sampler.mark()
    ms = b.boost_timed(k)  # the timed region: K trees, CUDA events around them on the booster's stream
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    launches_timed = int(b.profile().kernel_launches) - launches_before
    # Second pass for the roofline: per-kernel CUDA events on the same booster, directly after the timed region.
    # (In the timed region a round is one CUDA graph launch -- events cannot be recorded between its kernels -- and the
    # events themselves cost ~5 % of a step, so they stay out of `value`.)
    b.set_profile(True)
    barrier()
    ms_prof = b.boost_timed(k_prof)
    barrier()
    prof = b.profile()
    metrics = b.metrics()
    info = b.info
    # batch predict_raw of the trained trees over this rank's rows (Predictor::predict_raw): device time of the
    # traversal kernel; algorithmic bytes = nnz * 8 + rows * (4 + 4)
    predict = None
    if rank == 0 and not args.no_e2e:
        from thundergbm_b200.booster import predict_raw
        trees = b.trees()
        _, pms = predict_raw(data, trees, PARAMS['learning_rate'], float(info.base_score), timing=True)
        pbytes = data.nnz * 8.0 + data.n_rows * 8.0
        predict = {'kernel_ms': pms, 'rows': data.n_rows, 'trees': int(trees.shape[0]), 'gbs': pbytes / (pms * 1e-3) / 1e9 if pms > 0 else None}
    b.close()

    # ---- end to end through the C ABI with host buffers -----------------------------------------
    e2e = None
    if not args.no_e2e:
        lib = _lib.lib()
        # the caller's CSR sits in pinned host memory (page-locked once, outside the timed region)
        def pin(a, dt):
            return torch.from_numpy(np.ascontiguousarray(a, dt)).pin_memory().numpy()
        val = pin(data.val, np.float32); rp = pin(data.row_ptr, np.int32)
        col = pin(data.col, np.int32); y = pin(data.y, np.float32)
        def scikit_call(n_trees):
            model = C.c_void_p(None)
            num_class = C.c_int(2); per_iter = C.c_int(0)
            group_label = (C.c_float * 16)()
            lib.sparse_train_scikit(data.n_rows, val.ctypes.data_as(C.c_void_p), rp.ctypes.data_as(C.c_void_p),
                                    col.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), PARAMS['depth'], n_trees, 1,
                                    PARAMS['min_child_weight'], PARAMS['lambda'], PARAMS['gamma'], PARAMS['max_num_bin'], 0,
                                    1.0, 0, 1, PARAMS['learning_rate'], PARAMS['objective'].encode(), C.byref(num_class),
                                    b'hist', C.byref(model), C.byref(per_iter), group_label, None, 0)
            if not model.value:
                raise SystemExit('sparse_train_scikit failed: ' + lib.tgbm_last_error().decode())
            lib.model_free(C.byref(model))
        # untimed warm-up of the same entry point (allocator state after the first booster's frees)
        if world == 1:
            scikit_call(3)
        else:
            bw = Booster(synth.CsrData(data.n_rows, data.n_cols, rp, col, val, y), comm=comm, n_trees=3, **PARAMS)
            bw.boost(3)
            bw.close()
        barrier()
        t0 = time.perf_counter()
        if world == 1:
            model = C.c_void_p(None)
            num_class = C.c_int(2); per_iter = C.c_int(0)
            group_label = (C.c_float * 16)()
            lib.sparse_train_scikit(data.n_rows, val.ctypes.data_as(C.c_void_p), rp.ctypes.data_as(C.c_void_p),
                                    col.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), PARAMS['depth'], k, 1,
                                    PARAMS['min_child_weight'], PARAMS['lambda'], PARAMS['gamma'], PARAMS['max_num_bin'], 0,
                                    1.0, 0, 1, PARAMS['learning_rate'], PARAMS['objective'].encode(), C.byref(num_class),
                                    b'hist', C.byref(model), C.byref(per_iter), group_label, None, 0)
            if not model.value:
                raise SystemExit('sparse_train_scikit failed: ' + lib.tgbm_last_error().decode())
            d2h = k * info.n_nodes * 48
            lib.model_free(C.byref(model))
        else:
            ta = time.perf_counter()
            b2 = Booster(synth.CsrData(data.n_rows, data.n_cols, rp, col, val, y), comm=comm, n_trees=k, **PARAMS)
            tb = time.perf_counter()
            b2.boost(k)
            trees = b2.trees()
            tc = time.perf_counter()
            d2h = trees.nbytes
            b2.close()
            if os.environ.get('BENCH_DEBUG'):
                print(f'[rank {rank}] e2e: create {tb - ta:.3f} boost+trees {tc - tb:.3f} close {time.perf_counter() - tc:.3f}', file=sys.stderr)
        barrier()
        e2e_s = time.perf_counter() - t0
        t = torch.tensor([e2e_s], dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        h2d = val.nbytes + rp.nbytes + col.nbytes + y.nbytes
        e2e = {'value': float(t.item()) * 100.0 / k, 'unit': 's/100 trees', 'h2d_bytes_per_step': h2d / k,
               'd2h_bytes_per_step': d2h / k, 'note': f'wall clock of one C-ABI training call of {k} trees x 100/{k}, CSR in pinned host memory'}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    hist_gbs = prof.hist_bytes / (prof.hist_ms * 1e-3) / 1e9 if prof.hist_ms > 0 else 0.0
    root_gbs = prof.hist_root_bytes / (prof.hist_root_ms * 1e-3) / 1e9 if prof.hist_root_ms > 0 else 0.0
    part_gbs = prof.partition_bytes / (prof.partition_ms * 1e-3) / 1e9 if prof.partition_ms > 0 else 0.0
    line = {
        'metric': 'Higgs-shape train s/100 trees', 'value': ms_max / k * 100.0 / 1e3, 'unit': 's/100 trees',
        'n_gpus': world, 'steps': k, 'warmup': w, 'ms_per_step': ms_max / k, 'higher_is_better': False,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'i64', 'data': 'synthetic',
        'config': {'workload': WORKLOAD if n_rows == N_ROWS else WORKLOAD.replace('10.5M', str(n_rows)),
                   'rows_per_gpu': hi - lo, 'parallelism': f'rows sharded over {world} GPU(s), NCCL all-reduce of level histograms',
                   'l2': 'inputs larger than L2 (bin matrix %.0f MB per GPU)' % ((hi - lo) * 32 / 1e6),
                   'quant_bits': 18, 'final_train_error': float(metrics[w + k - 1]) if len(metrics) >= w + k else None,
                   'init_s': t_init, 'datagen_s': t_gen},
        'roofline': {'bound': 'hbm', 'kernel': 'k_hist (histogram build, all levels)', 'achieved': hist_gbs, 'peak': peak,
                     'unit': 'GB/s', 'frac': hist_gbs / peak, 'peak_kind': peak_kind, 'traffic': NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     'launches': int(prof.hist_launches), 'avg_launch_us': prof.hist_ms * 1e3 / max(1, prof.hist_launches),
                     'root_level_gbs': root_gbs, 'root_level_frac': root_gbs / peak,
                     'partition_gbs': part_gbs, 'partition_frac': part_gbs / peak,
                     'hist_share_of_step': prof.hist_ms / ms_prof if ms_prof > 0 else None,
                     'partition_share_of_step': prof.partition_ms / ms_prof if ms_prof > 0 else None,
                     'measured_on': f'{k_prof} trees directly after the timed region, per-kernel CUDA events (ms_per_step there {ms_prof / k_prof:.3f})'},
        'e2e': e2e, 'gpu_launches': launches_timed, 'clocks': clocks, 'predict': predict,
    }
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        nt = 5
        r = oracle_sample_run(nt, cores)
        s_tree = float(np.mean(r.round_seconds[1:]))
        line['cpu_baseline'] = {'value': s_tree * 100.0 * (N_ROWS / SAMPLE_ROWS), 'unit': 's/100 trees', 'cores': cores, 'kind': 'port',
                                'sample': f'{SAMPLE_ROWS} of {N_ROWS} rows, {nt - 1} timed trees after 1 warm-up; seconds/tree scaled by '
                                          f'{N_ROWS / SAMPLE_ROWS:.1f} (rows) and to 100 trees'}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
