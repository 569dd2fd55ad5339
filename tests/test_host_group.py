"""Failure handling of in-process rank groups, made on the host only: CPU threads stand in for the ranks, one of them
fails a local check, leaves the group or never arrives, and the others must learn of it before they would enqueue
their next collective (tgbm::HostGroup, thundergbm_b200/csrc/tgbm_hostgroup.h).  No GPU is involved."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_group_agreement(tmp_path):
    exe = tmp_path / 'hostgroup_check'
    subprocess.check_call(['g++', '-O1', '-std=c++17', '-pthread', os.path.join(ROOT, 'tests', 'cpp', 'hostgroup_check.cpp'),
                           '-o', str(exe)])
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, check=True).stdout
    got = {l.split()[0]: [int(v) for v in l.split()[1:]] for l in out.strip().splitlines()}
    assert got['all_ok'] == [1, 1, 1, 1]
    assert got['one_fails_round1'] == [1, 1, 1, 1]
    assert got['one_fails_round2'] == [0, 0, 0, 0]          # every rank stops in the round one of them failed
    assert got['one_fails_round3'] == [0, 0, 0, 0]          # and the group stays closed
    assert got['abandon'] == [0, -1, 0, 0]                   # rank 1 left; the others were released with a failure
    assert got['missing_rank'] == [0, 0, 0, -1]              # rank 3 never came; the time limit ended the wait
