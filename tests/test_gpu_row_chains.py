"""The two chains without a matmul (row softmax of a given matrix; row variance broadcast
along the row), through the C ABI against the CPU checker, and through the backend tools
(welder-compiler -> welder-profiler -> verify.py) on the inputs the package ships."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "welder_typical_chain_b200")
BK = os.path.join(PKG, "backend", "welder", "compiler", "build")


@pytest.mark.parametrize("shape", [(32, 256), (1, 8), (7, 24), (300, 1000), (64, 1024), (5, 2048), (33, 2056), (3, 32000), (2, 4, 520)])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_row_softmax_matches_the_checker(wtc_lib, cuda_dev, shape, dtype):
    import torch
    w = wtc_lib
    rng = np.random.default_rng(sum(shape))
    X = (rng.standard_normal(shape) * 3).astype(np.float16 if dtype == "f16" else np.float32)
    X.reshape(-1, shape[-1])[0, 0] = 11.0                         # one dominant entry
    out = w.row_softmax(torch.from_numpy(X).to(cuda_dev))
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(-1, shape[-1])
    res = oracle.compare(got, oracle.row_softmax(X).reshape(-1, shape[-1]))
    assert res["ok"], res
    if dtype == "f32":
        assert np.abs(got.astype(np.float64) - oracle.row_softmax(X).reshape(-1, shape[-1])).max() < 2e-6


@pytest.mark.parametrize("shape", [(32, 256), (1, 8), (7, 24), (300, 1000), (5, 2048), (33, 2056), (3, 32000)])
def test_row_variance_matches_the_checker(wtc_lib, cuda_dev, shape):
    import torch
    w = wtc_lib
    rng = np.random.default_rng(sum(shape) + 1)
    A = (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32)
    out = w.row_variance(torch.from_numpy(A).to(cuda_dev))
    torch.cuda.synchronize()
    ref = oracle.row_variance(A)
    assert np.abs(out.cpu().numpy().astype(np.float64) - ref).max() <= 1e-4 * np.abs(ref).max()
    # other constants than 1/N, f16 elements
    out = w.row_variance(torch.from_numpy(A).to(cuda_dev), mean_factor=0.5 / shape[-1], var_factor=2.0)
    ref = oracle.row_variance(A, 0.5 / shape[-1], 2.0)
    assert np.abs(out.cpu().numpy().astype(np.float64) - ref).max() <= 1e-4 * np.abs(ref).max()
    A16 = A.astype(np.float16)
    out = w.row_variance(torch.from_numpy(A16).to(cuda_dev))
    torch.cuda.synchronize()
    ref = oracle.row_variance(A16)
    assert np.abs(out.cpu().numpy().astype(np.float64) - ref).max() <= 2e-3 * np.abs(ref).max()


def test_row_chain_descriptor_errors_and_empty(wtc_lib, cuda_dev):
    import ctypes as C
    w = wtc_lib
    L = w.lib()
    d = w.RowChainDesc()
    d.struct_size = C.sizeof(w.RowChainDesc)
    d.kind, d.rows, d.N, d.dtype = 7, 4, 4, w.F32
    one = C.c_void_p(256)
    assert L.wtc_row_chain_launch(C.byref(d), one, one, None) == -1 and b"kind" in L.wtc_last_error()
    d.kind, d.rows = w.ROW_SOFTMAX, 0
    assert L.wtc_row_chain_launch(C.byref(d), None, None, None) == 0        # nothing to do
    d.rows, d.ld_in = 4, 2
    assert L.wtc_row_chain_launch(C.byref(d), one, one, None) == -1 and b"stride" in L.wtc_last_error()


@pytest.mark.parametrize("name", ["softmax_row_chain.mlir", "layernorm_variance_chain.mlir"])
@pytest.mark.parametrize("init", ["linear", "random"])
def test_backend_tools_run_and_verify_the_row_chains(tmp_path, name, init):
    out = tmp_path / "c"
    tiles = ["--force-tile-m", "32", "--force-tile-n", "64", "--force-tile-k", "16", "--thread-tile-m", "2", "--thread-tile-n", "2"]
    r = subprocess.run([os.path.join(BK, "welder-compiler"), os.path.join(PKG, "mlir", name), *tiles, "--emit-all-stages", "--output",
                        str(out / "03.after_postbufferize.mlir")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    plan = str(out / "05.out.nvvm.runnable.mlir")
    dump = str(tmp_path / "out.bin")
    r = subprocess.run([os.path.join(BK, "welder-profiler"), plan, "--warmup", "2", "--iters", "5", f"--init={init}", "--seed", "3", "--dump-last-2d", dump],
                       capture_output=True, text=True)
    assert r.returncode == 0 and "avg_ms=" in r.stdout, r.stderr
    v = subprocess.run([sys.executable, os.path.join(PKG, "bench", "verify.py"), "--out", dump, "--plan", plan, "--pattern", init, "--seed", "3",
                        "--rows", "0,1,2,3,7,15,31", "--rtol", "1e-5", "--atol", "1e-7"], capture_output=True, text=True)
    assert v.returncode == 0 and v.stdout.startswith("PASS"), v.stdout + v.stderr
