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
    ("matmul_softmax_chain_f16_matmul.mlir", "random", "1024"),     # f32 buffers rounded to f16 on the device
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


def test_search_with_on_device_profiling(tmp_path, wtc_lib, cuda_dev):
    """welder-solver --enable-profiling on the GPU: both tile shapes the kernel library has are
    compiled, timed by welder-profiler and cached; a second run is answered by the cache."""
    env = dict(os.environ, OUT_BASE=str(tmp_path / "sp"), PROFILE_WARMUP="3", PROFILE_ITERS="20")
    script = os.path.join(PKG, "bench", "run_search_profile.sh")
    r = subprocess.run(["bash", script], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("[wtc.profile] measured") == 2, r.stdout[-3000:]
    rows = [l.split("\t") for l in open(tmp_path / "sp" / "search" / "candidates.tsv").read().splitlines()]
    col = rows[0].index("profiledMs")
    ms = [float(x[col]) for x in rows[1:3]]
    assert 0 < ms[0] <= ms[1] < 1.0, ms                     # config 2 runs in tens of microseconds
    assert len(open(tmp_path / "sp" / "profile_cache.tsv").read().splitlines()) == 2
    r = subprocess.run(["bash", script], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and r.stdout.count("[wtc.profile] cache hit") == 2, r.stdout[-3000:]


def test_native_multi_gpu_runner_on_one_gpu():
    """welder-multi (one native process, one thread per GPU, NCCL for the column split) on the
    GPUs this test has: every way of sharing the chain, reduced shapes, row sums checked by the
    tool itself.  With one GPU the all-gather runs on a communicator of one rank."""
    import json
    import torch
    tool = os.path.join(PKG, "backend", "welder", "compiler", "build", "welder-multi")
    n = min(2, torch.cuda.device_count())
    for wl, extra in (("rows", ["--m", "1024", "--n", "1024", "--k", "256"]), ("batch", ["--batch", "6", "--m", "512", "--n", "2048", "--k", "128"]),
                      ("cols", ["--m", "512", "--n", "4104", "--k", "512"])):
        r = subprocess.run([tool, "--workload", wl, "--gpus", str(n), "--steps", "5", "--warmup", "2", *extra], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert line["gpus"] == n and line["row_sums_ok"] and line["us_per_step"] > 0 and len(line["us_per_step_per_gpu"]) == n
