#!/usr/bin/env bash
# Runs the reference (built by oracle/build_ref.sh) on golden inputs on a GPU box and leaves its
# outputs under <out_dir>/<case>/ : cut points, global bin ids, model file, raw predictions and
# the log with the per-round metric.  tests/golden/pack_golden.py turns those outputs (and those
# of further runs, for the reference's own run-to-run spread) into the committed fixtures.
# usage: run_reference.sh <out_dir> [harness key=value ...]
#   CASES="a b" restricts the cases; dump_bins=0 skips the cut-point / bin-id dumps (repeat runs).
#   n_device=2 runs the reference's column-sharded builder on two GPUs: call once with the default dump_bins=1 (writes
#   the devices' cut points and bin matrices, no training) and once with dump_bins=0 (trains) into the same <out_dir>.
set -u
ROOT=$(cd "$(dirname "$0")/../.." && pwd)
IN=$ROOT/oracle/_ref/inputs
BIN=$ROOT/oracle/_ref/bin
OUT=${1:?usage: run_reference.sh <out_dir> [key=value ...]}
shift
mkdir -p "$OUT"
for args in "$IN"/*.args; do
  name=$(basename "$args" .args)
  if [ -n "${CASES:-}" ] && ! echo " $CASES " | grep -q " $name "; then continue; fi
  mkdir -p "$OUT/$name"
  echo "== $name"
  timeout 600 "$BIN/ref_harness" "$IN/$name.tgbin" "$OUT/$name" $(cat "$args") "$@" > "$OUT/$name/log.txt" 2>&1
  echo "exit $?" >> "$OUT/$name/log.txt"
  tail -3 "$OUT/$name/log.txt"
done
# the README run through the reference's own CLI (writes ./tgbm.model)
if [ -z "${CASES:-}" ] && [ -f "$IN/test_dataset.txt" ]; then
  mkdir -p "$OUT/cli_machine_conf" && cd "$OUT/cli_machine_conf"
  echo "data=$IN/test_dataset.txt" > machine.conf
  timeout 300 "$BIN/thundergbm-train" machine.conf > log.txt 2>&1
  echo "exit $?" >> log.txt
  tail -3 log.txt
fi
