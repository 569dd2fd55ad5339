#!/usr/bin/env bash
# Runs the reference (built by oracle/build_ref.sh) on every golden input on a GPU
# box and leaves its outputs under <out_dir>/<case>/ : cut points, global bin ids,
# model file, raw predictions and the log with the per-round metric.
# tests/golden/pack_golden.py turns those outputs into the committed fixtures.
# usage: run_reference.sh [out_dir]
set -u
ROOT=$(cd "$(dirname "$0")/../.." && pwd)
IN=$ROOT/oracle/_ref/inputs
BIN=$ROOT/oracle/_ref/bin
OUT=${1:-$ROOT/gpurun_out/golden}
mkdir -p "$OUT"
for args in "$IN"/*.args; do
  name=$(basename "$args" .args)
  mkdir -p "$OUT/$name"
  echo "== $name"
  timeout 300 "$BIN/ref_harness" "$IN/$name.tgbin" "$OUT/$name" $(cat "$args") > "$OUT/$name/log.txt" 2>&1
  echo "exit $?" >> "$OUT/$name/log.txt"
  tail -3 "$OUT/$name/log.txt"
done
# second run of one case: how much do the reference's unordered fp32 atomics move its own result?
mkdir -p "$OUT/c2_higgs_small_rerun"
timeout 300 "$BIN/ref_harness" "$IN/c2_higgs_small.tgbin" "$OUT/c2_higgs_small_rerun" $(cat "$IN/c2_higgs_small.args") dump_bins=0 \
  > "$OUT/c2_higgs_small_rerun/log.txt" 2>&1
echo "exit $?" >> "$OUT/c2_higgs_small_rerun/log.txt"
# the README run through the reference's own CLI (writes ./tgbm.model)
if [ -f "$IN/test_dataset.txt" ]; then
  mkdir -p "$OUT/cli_machine_conf" && cd "$OUT/cli_machine_conf"
  echo "data=$IN/test_dataset.txt" > machine.conf
  timeout 300 "$BIN/thundergbm-train" machine.conf > log.txt 2>&1
  echo "exit $?" >> log.txt
  tail -3 log.txt
fi
