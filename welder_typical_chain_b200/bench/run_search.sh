#!/usr/bin/env bash
# Tile search only: <OUT_BASE>/search/{best.json,best_summary.json,candidates.tsv,solver.log}.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_f16_native.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_search}"
[[ -f "${INPUT_MLIR}" ]] || die "input not found: ${INPUT_MLIR}"
wtc_build
wtc --output-dir "${OUT_BASE}" --backend-mode "${BACKEND_MODE}" --search-only --max-connect-level "${MAX_CONNECT_LEVEL}" --verbose
echo "[wtc] best: ${OUT_BASE}/search/best.json"
cat "${OUT_BASE}/search/best.json"
