"""The harness end to end on a GPU: compile pair -> welder-profiler runs -> dump -> verify.py,
as bench/run_ab.sh does in the reference (VERIFY=1 path, bench/run_ab.sh:165-187)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "welder_typical_chain_b200")


@pytest.mark.parametrize("mlir,pattern,rows", [
    ("matmul_softmax_chain_f16_native.mlir", "linear", None),       # the reference's default input and pattern
    ("matmul_softmax_chain.mlir", "random", "512"),                 # f32 chain, xorshift inputs
    ("cfg2_f16_native_4096x1024x1024.mlir", "linear", None),        # tcgen05 cluster kernel
    ("cfg3_batched_attention_named.mlir", "linear", "2048"),        # named softmax, batched plan (first batch verified)
])
def test_run_ab_with_verification(tmp_path, wtc_lib, cuda_dev, mlir, pattern, rows):
    env = dict(os.environ, INPUT_MLIR=os.path.join(PKG, "mlir", mlir), OUT_BASE=str(tmp_path / "ab"), BACKEND_MODE="api",
               WARMUP="2", ITERS="5", VERIFY="1", PATTERN=pattern, VERIFY_RTOL="1e-2", VERIFY_ATOL="2e-3")
    if rows:
        env["M"] = rows
    r = subprocess.run(["bash", os.path.join(PKG, "bench", "run_ab.sh")], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "[warn" not in r.stdout, r.stdout[-3000:]
    for case in ("baseline", "fused"):
        v = open(tmp_path / "ab" / case / "verify.log").read()
        assert v.startswith("PASS"), (case, v)
        assert "avg_ms=" in open(tmp_path / "ab" / case / "profile.log").read()
    rows_ = open(tmp_path / "ab" / "ab_summary.tsv").read().splitlines()
    assert rows_[0].split("\t")[:3] == ["case", "avg_ms", "kernels"] and len(rows_) == 3
    assert rows_[1].split("\t")[2] == "5"                                  # the unfused pipeline is five launches
    assert float(open(tmp_path / "ab" / "speedup.tsv").read().split("\t")[1]) > 0
