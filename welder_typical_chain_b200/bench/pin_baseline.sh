#!/usr/bin/env bash
# Copies the numbers of an A/B run into a baseline folder the perf guard compares against.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
SRC="${SRC_OUT_BASE:-/tmp/wtc_ab}"
NAME="${BASELINE_NAME:-default}"
DST="${BASELINE_DIR:-${BENCH_DIR}/baselines/${NAME}}"
for f in ab_summary.tsv ab_summary.csv speedup.tsv search/best.json; do
  [[ -f "${SRC}/${f}" ]] || die "missing ${SRC}/${f}: run run_ab.sh first"
done
mkdir -p "${DST}/search"
cp "${SRC}/ab_summary.tsv" "${SRC}/ab_summary.csv" "${SRC}/speedup.tsv" "${DST}/"
cp "${SRC}/search/best.json" "${DST}/search/best.json"
for v in baseline fused; do
  mkdir -p "${DST}/${v}"
  cp "${SRC}/${v}/05.out.nvvm.runnable.mlir" "${SRC}/${v}/04.after_workgroup_launch.mlir" "${DST}/${v}/"
done
{
  echo "pinned_at=$(date -u +%Y-%m-%dT%H:%M:%SZ)"
  echo "source=${SRC}"
  echo "gpu=$(nvidia-smi --query-gpu=name --format=csv,noheader 2>/dev/null | head -n 1 || echo unknown)"
} >"${DST}/manifest.txt"
echo "[wtc] pinned baseline: ${DST}"
