#!/usr/bin/env bash
# Search once, then compile the baseline (connect level 0) and the fused variant with the
# same tile choice: <OUT_BASE>/{search,baseline,fused}/...
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_f16_native.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_pair}"
[[ -f "${INPUT_MLIR}" ]] || die "input not found: ${INPUT_MLIR}"
wtc_build
mkdir -p "${OUT_BASE}"
BEST_JSON="${OUT_BASE}/search/best.json"
echo "[wtc] search"
wtc --output-dir "${OUT_BASE}" --backend-mode "${BACKEND_MODE}" --search-only --max-connect-level "${MAX_CONNECT_LEVEL}" --verbose
for variant in baseline fused; do
  echo "[wtc] compile ${variant}"
  level="${MAX_CONNECT_LEVEL}"; [[ "${variant}" == baseline ]] && level=0
  wtc --output-dir "${OUT_BASE}" --backend-mode "${BACKEND_MODE}" --compile-only --best-json "${BEST_JSON}" "--${variant}" \
      --max-connect-level "${level}" --verbose
done
echo "[wtc] done"
echo "  best:     ${BEST_JSON}"
echo "  baseline: ${OUT_BASE}/baseline/05.out.nvvm.runnable.mlir"
echo "  fused:    ${OUT_BASE}/fused/05.out.nvvm.runnable.mlir"
