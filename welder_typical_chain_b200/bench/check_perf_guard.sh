#!/usr/bin/env bash
# Compares an A/B run with a pinned baseline: each avg_ms may regress by at most
# MAX_REGRESSION_PCT (default 3); the speedup may drop by at most the same share.
# SPEEDUP_CHECK_MODE: auto (default; skip the speedup floor when the unfused baseline itself
# got faster than the threshold), strict, off.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
BASELINE_DIR="${BASELINE_DIR:-${BENCH_DIR}/baselines/default}"
CURRENT_OUT_BASE="${CURRENT_OUT_BASE:-/tmp/wtc_ab}"
MAX_REGRESSION_PCT="${MAX_REGRESSION_PCT:-3}"
SPEEDUP_CHECK_MODE="${SPEEDUP_CHECK_MODE:-auto}"
case "${SPEEDUP_CHECK_MODE}" in auto|strict|off) ;; *) die "invalid SPEEDUP_CHECK_MODE=${SPEEDUP_CHECK_MODE} (expected auto|strict|off)";; esac
for p in "${BASELINE_DIR}/ab_summary.tsv" "${BASELINE_DIR}/speedup.tsv" "${CURRENT_OUT_BASE}/ab_summary.tsv" "${CURRENT_OUT_BASE}/speedup.tsv"; do
  [[ -f "${p}" ]] || die "missing required file: ${p}"
done
ms() { awk -F'\t' -v k="$2" '$1==k{print $2}' "$1"; }
bb="$(ms "${BASELINE_DIR}/ab_summary.tsv" baseline)"; bf="$(ms "${BASELINE_DIR}/ab_summary.tsv" fused)"
cb="$(ms "${CURRENT_OUT_BASE}/ab_summary.tsv" baseline)"; cf="$(ms "${CURRENT_OUT_BASE}/ab_summary.tsv" fused)"
bs="$(awk 'NR==1{print $2}' "${BASELINE_DIR}/speedup.tsv")"; cs="$(awk 'NR==1{print $2}' "${CURRENT_OUT_BASE}/speedup.tsv")"
for v in "${bb}" "${bf}" "${cb}" "${cf}" "${bs}" "${cs}"; do [[ -n "${v}" ]] || die "failed to parse performance metrics"; done
awk -v bb="${bb}" -v bf="${bf}" -v cb="${cb}" -v cf="${cf}" -v bs="${bs}" -v cs="${cs}" -v p="${MAX_REGRESSION_PCT}" -v mode="${SPEEDUP_CHECK_MODE}" '
function slower(name, base, cur,   lim) { lim = base * (1 + p / 100)
  if (cur > lim) { printf "FAIL %s: baseline=%s, current=%s, limit=%.9g (%s%% regression threshold)\n", name, base, cur, lim, p; bad = 1 }
  else printf "PASS %s: baseline=%s, current=%s, threshold=%s%%\n", name, base, cur, p }
BEGIN {
  slower("baseline.avg_ms", bb, cb); slower("fused.avg_ms", bf, cf)
  if (mode == "off") print "SKIP speedup: SPEEDUP_CHECK_MODE=off"
  else if (mode == "auto" && cb < bb * (1 - p / 100)) printf "SKIP speedup: baseline improved beyond %s%% (baseline=%s, current=%s)\n", p, bb, cb
  else { lim = bs * (1 - p / 100)
    if (cs < lim) { printf "FAIL speedup: baseline=%s, current=%s, min_allowed=%.9g (%s%% drop threshold)\n", bs, cs, lim, p; bad = 1 }
    else printf "PASS speedup: baseline=%s, current=%s, drop_threshold=%s%%\n", bs, cs, p }
  exit bad }' || { echo "[wtc] perf guard FAILED" >&2; exit 1; }
echo "[wtc] perf guard passed"
echo "  baseline_dir: ${BASELINE_DIR}"
echo "  current_out:  ${CURRENT_OUT_BASE}"
