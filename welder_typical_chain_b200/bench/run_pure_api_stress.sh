#!/usr/bin/env bash
# Re-entrancy stress: search(api) + compile(api) REPEAT times inside one wtc-compiler process.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_f16_native.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_pure_api_stress}"
REPEAT="${REPEAT:-100}"
[[ -f "${INPUT_MLIR}" ]] || die "input not found: ${INPUT_MLIR}"
wtc_build
rm -rf "${OUT_BASE}"; mkdir -p "${OUT_BASE}"
start="$(date +%s.%N)"
wtc --output-dir "${OUT_BASE}" --backend-mode api --pure-api-full --max-connect-level "${MAX_CONNECT_LEVEL}" --fused --repeat "${REPEAT}" \
  >"${OUT_BASE}/stress.log" 2>&1 || die "stress run failed, see ${OUT_BASE}/stress.log"
end="$(date +%s.%N)"
last=$((REPEAT - 1))
artifact="${OUT_BASE}/iter_${last}/fused/05.out.nvvm.runnable.mlir"
[[ -s "${artifact}" ]] || die "last iteration left no artifact: ${artifact}"
awk -v s="${start}" -v e="${end}" -v n="${REPEAT}" 'BEGIN{printf "[wtc] pure-api stress passed: %d iterations, %.3f s, %.2f ms/iter\n", n, e-s, (e-s)*1000/n}'
echo "  last artifact: ${artifact}"
