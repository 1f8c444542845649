#!/usr/bin/env bash
# Host-side regression (no GPU needed): search through the C API, named-softmax
# decomposition, a full api run, and a pure-api repeat in one process.
# Writes PASS/FAIL rows to <OUT_BASE>/regression_summary.tsv; exits 1 on the first FAIL.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_f16_native.mlir}"
NAMED_SOFTMAX_INPUT_MLIR="${NAMED_SOFTMAX_INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_named_softmax.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_regression}"
PURE_API_REPEAT="${PURE_API_REPEAT:-10}"
mkdir -p "${OUT_BASE}"
SUMMARY="${OUT_BASE}/regression_summary.tsv"
printf 'check\tstatus\tdetail\n' >"${SUMMARY}"
pass() { printf '%s\tPASS\t%s\n' "$1" "$2" >>"${SUMMARY}"; }
fail() { printf '%s\tFAIL\t%s\n' "$1" "$2" >>"${SUMMARY}"; echo "FAIL $1: $2" >&2; exit 1; }
have_file() { [[ -s "$2" ]] && pass "$1" "exists: $2" || fail "$1" "missing or empty file: $2"; }
has() { grep -q -- "$3" "$2" && pass "$1" "found '$3' in $2" || fail "$1" "pattern '$3' not found in $2"; }
hasnt() { grep -q -- "$3" "$2" && fail "$1" "pattern '$3' still present in $2" || pass "$1" "'$3' absent from $2"; }

wtc_build; pass build "${WTC}"
out="${OUT_BASE}/search_api"
wtc --output-dir "${out}" --backend-mode api --search-only --max-connect-level "${MAX_CONNECT_LEVEL}" >/dev/null || fail search_api "wtc-compiler failed"
have_file search_api.best "${out}/search/best.json"
have_file search_api.candidates "${out}/search/candidates.tsv"
has search_api.tile_keys "${out}/search/best.json" '"tileM"'

out="${OUT_BASE}/search_named_softmax"
INPUT_MLIR="${NAMED_SOFTMAX_INPUT_MLIR}" wtc --output-dir "${out}" --backend-mode process_chain --search-only \
  --max-connect-level "${MAX_CONNECT_LEVEL}" >/dev/null || fail named_softmax "wtc-compiler failed"
have_file named_softmax.canonicalized "${out}/ir/01.canonicalized.mlir"
has named_softmax.exp "${out}/ir/01.canonicalized.mlir" 'math\.exp'
has named_softmax.div "${out}/ir/01.canonicalized.mlir" 'arith\.divf'
hasnt named_softmax.decompose "${out}/ir/01.canonicalized.mlir" 'linalg\.softmax'

out="${OUT_BASE}/full_api_default"
wtc --output-dir "${out}" --backend-mode api --max-connect-level "${MAX_CONNECT_LEVEL}" --fused >/dev/null || fail full_api_default "wtc-compiler failed"
have_file full_api_default.runnable "${out}/fused/05.out.nvvm.runnable.mlir"
has full_api_default.workgroup "${out}/fused/04.after_workgroup_launch.mlir" 'workgroup('
has full_api_default.launchfunc "${out}/fused/05.out.nvvm.runnable.mlir" 'gpu\.launch_func'
have_file full_api_default.report "${out}/fused/postbufferize_report.txt"

out="${OUT_BASE}/pure_api_repeat"
wtc --output-dir "${out}" --backend-mode api --pure-api-full --max-connect-level "${MAX_CONNECT_LEVEL}" --fused \
  --repeat "${PURE_API_REPEAT}" >/dev/null || fail pure_api_repeat "wtc-compiler failed"
last=$((PURE_API_REPEAT - 1))
have_file pure_api_repeat.runnable "${out}/iter_${last}/fused/05.out.nvvm.runnable.mlir"
has pure_api_repeat.launchfunc "${out}/iter_${last}/fused/05.out.nvvm.runnable.mlir" 'gpu\.launch_func'
echo "[wtc] regression passed"
echo "  summary: ${SUMMARY}"
