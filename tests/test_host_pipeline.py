"""The native host side on the CPU: chain recogniser, tile contract, the three backend
modes of wtc-compiler, artifact tree, error behaviour, the dlopen C APIs and the harness
scripts that need no GPU.  Mirrors the reference's script-level regression
(bench/run_regression.sh:60-112, bench/run_pure_api_stress.sh:46-68)."""
import ctypes
import json
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "welder_typical_chain_b200")
WTC = os.path.join(PKG, "build", "wtc-compiler")
BK = os.path.join(PKG, "backend", "welder", "compiler", "build")
MLIR = os.path.join(PKG, "mlir")


@pytest.fixture(scope="module", autouse=True)
def built(wtc_lib):
    if not (os.path.exists(WTC) and os.path.exists(os.path.join(BK, "libwelder-compile-capi.so"))):
        subprocess.run(["make", "-C", os.path.join(PKG, "host"), "-j8"], check=True, capture_output=True)


def run(args, **kw):
    return subprocess.run([WTC] + args, capture_output=True, text=True, **kw)


def test_capi_headers_match_exports():
    for header, lib in (("welder_solver_capi.h", "libwelder-solver-capi.so"), ("welder_compile_capi.h", "libwelder-compile-capi.so")):
        text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", header)).read(), flags=re.S)
        L = ctypes.CDLL(os.path.join(BK, lib))
        for sym in re.findall(r"\b(welder_[a-z_]+)\s*\(", text):
            assert hasattr(L, sym), f"{sym} missing from {lib}"
    # the C++-linkage in-process entry is exported from the compile library too
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(BK, "libwelder-compile-capi.so")], capture_output=True, text=True).stdout
    assert "_Z18welderCompilerMainiPPc" in out


@pytest.mark.parametrize("mode", ["api", "process_chain", "shell", "inprocess"])
def test_full_pipeline_artifact_tree(tmp_path, mode):
    out = tmp_path / "o"
    r = run(["--input", os.path.join(MLIR, "cfg2_f16_native_4096x1024x1024.mlir"), "--out-dir", str(out), "--backend-mode", mode, "--verbose"])
    assert r.returncode == 0, r.stderr
    for rel in ("ir/01.canonicalized.mlir", "ir/01.canonicalize.log", "ir/02.tagged.mlir", "ir/02.tags.json", "ir/chain.json",
                "search/best.json", "search/best_summary.json", "search/candidates.tsv", "search/solver.log",
                "fused/03.after_postbufferize.mlir", "fused/04.after_workgroup_launch.mlir", "fused/04c.after_linalg_to_loops.mlir",
                "fused/05.out.nvvm.runnable.mlir", "fused/compile.log", "fused/postbufferize_report.txt"):
        assert (out / rel).stat().st_size > 0, rel
    best = json.load(open(out / "search/best.json"))
    assert best == dict(tileM=128, tileN=256, tileK=64, threadTileM=1, threadTileN=128)
    chain = json.load(open(out / "ir/chain.json"))
    assert (chain["M"], chain["N"], chain["K"], chain["scale"]) == (4096, 1024, 1024, 0.03125)
    assert (chain["in_dtype"], chain["acc_dtype"], chain["out_dtype"]) == ("f16", "f32", "f16")
    plan = open(out / "fused/05.out.nvvm.runnable.mlir").read()
    assert 'kernel = "tc_cluster"' in plan and "cluster_n = 4" in plan and "gpu.launch_func" in plan
    assert "workgroup(" in open(out / "fused/04.after_workgroup_launch.mlir").read()
    tags = json.load(open(out / "ir/02.tags.json"))
    assert tags["counts"]["matmul"] == 1 and tags["counts"]["exp"] == 1 and tags["counts"]["div"] == 1
    tagged = open(out / "ir/02.tagged.mlir").read()
    for t in ("welder.matmul_anchor", "welder.row_reduction", "welder.elementwise_exp", "welder.elementwise_div"):
        assert tagged.count("// wtc.tag: " + t) == 1
    if mode == "api":
        assert "search falls back to process_chain" in r.stdout


def test_named_softmax_is_decomposed(tmp_path):
    for name, batched in (("matmul_softmax_chain_named_softmax.mlir", False), ("cfg3_batched_attention_named.mlir", True)):
        out = tmp_path / name
        r = run(["--input", os.path.join(MLIR, name), "--out-dir", str(out), "--backend-mode", "process_chain", "--search-only"])
        assert r.returncode == 0, r.stderr
        text = open(out / "ir/01.canonicalized.mlir").read()
        assert "linalg.softmax" not in text and "math.exp" in text and "arith.divf" in text
        assert text.count('"reduction"') == 2
        assert ("linalg.batch_matmul" in text) == batched
        chain = json.load(open(out / "ir/chain.json"))
        assert chain["softmax_form"] == "named" and chain["batched"] == batched


def test_every_shipped_chain_compiles_to_the_expected_kernel(tmp_path):
    expect = {"cfg1_decomposed_f32_128": "simt_fused", "cfg2_f16_native_4096x1024x1024": "tc_cluster",
              "cfg3_batched_attention_named": "tc_cluster", "cfg4_vocab_logits": "tc_tiled", "cfg5_skinny_decode": "tc_tiled",
              "matmul_softmax_chain": "simt_fused", "matmul_softmax_chain_f16_native": "tc_cluster",
              "matmul_softmax_chain_named_softmax": "simt_fused", "matmul_softmax_chain_f16_matmul": "tc_cluster"}
    for stem, kernel in expect.items():
        out = tmp_path / stem
        r = run(["--input", os.path.join(MLIR, stem + ".mlir"), "--out-dir", str(out), "--backend-mode", "api", "--pure-api-full"])
        assert r.returncode == 0, (stem, r.stderr)
        assert f'kernel = "{kernel}"' in open(out / "fused/05.out.nvvm.runnable.mlir").read(), stem


def test_f32_arguments_rounded_to_f16_are_recognised(tmp_path):
    """f32 arguments may reach the matmul through arith.truncf generics (the reference's
    matmul_softmax_chain_f16_matmul.mlir); the plan then keeps f32 buffers and asks the launch
    layer to round them.  Any other indirection is still rejected."""
    out = tmp_path / "o"
    inp = os.path.join(MLIR, "matmul_softmax_chain_f16_matmul.mlir")
    r = run(["--input", inp, "--out-dir", str(out), "--backend-mode", "api", "--pure-api-full"])
    assert r.returncode == 0, r.stderr
    chain = json.load(open(out / "ir" / "chain.json"))
    assert (chain["arg_dtype"], chain["in_dtype"], chain["acc_dtype"], chain["out_dtype"]) == ("f32", "f16", "f16", "f32")
    plan = open(out / "fused" / "05.out.nvvm.runnable.mlir").read()
    assert 'arg_dtype = "f32", in_dtype = "f16"' in plan and "launches = 2" in plan     # one launch that rounds both operands + the fused kernel
    ws = int(re.search(r"workspace_bytes = (\d+)", plan).group(1))
    assert ws == 8192 * 64 * 2 + 64 * 128 * 2                                           # the two rounded copies
    bad = tmp_path / "bad.mlir"
    bad.write_text(open(inp).read().replace("arith.truncf %x : f32 to f16", "arith.negf %x : f32"))
    r = run(["--input", str(bad), "--out-dir", str(tmp_path / "b"), "--backend-mode", "api", "--pure-api-full"])
    assert r.returncode == 1 and "rounded to f16 by arith.truncf" in open(tmp_path / "b" / "ir" / "01.canonicalize.log").read()


def test_type_and_map_aliases_are_expanded(tmp_path):
    """MLIR printers name types and affine maps at the top of a module; the recogniser expands the
    names, and the canonical form it writes spells everything out."""
    out = tmp_path / "o"
    r = run(["--input", os.path.join(MLIR, "matmul_softmax_chain_named_softmax.mlir"), "--out-dir", str(out), "--search-only", "--backend-mode", "api"])
    assert r.returncode == 0, r.stderr
    canon = open(out / "ir" / "01.canonicalized.mlir").read()
    assert "!t0" not in canon and "#m0" not in canon and "tensor<8192x128xf32>" in canon and "affine_map<(d0, d1) -> (d0)>" in canon
    spelled = tmp_path / "spelled.mlir"
    spelled.write_text(canon)                                               # alias-free text parses to the same chain
    r = run(["--input", str(spelled), "--out-dir", str(tmp_path / "o2"), "--search-only", "--backend-mode", "api"])
    a, b = json.load(open(tmp_path / "o2" / "ir" / "chain.json")), json.load(open(out / "ir" / "chain.json"))
    assert r.returncode == 0 and a.pop("softmax_form") == "decomposed" and b.pop("softmax_form") == "named" and a == b
    nested = tmp_path / "nested.mlir"                                       # an alias may use an earlier alias; !t1 must not eat !t10
    nested.write_text("!e = f32\n!t1 = tensor<8x16x!e>\n!t10 = tensor<16x24x!e>\n!t2 = tensor<8x24x!e>\n" + """module {
  func.func @main(%A: !t1, %B: !t10) -> !t2 {
    %z = arith.constant 0.0 : f32
    %e = tensor.empty() : !t2
    %f = linalg.fill ins(%z : f32) outs(%e : !t2) -> !t2
    %C = linalg.matmul ins(%A, %B : !t1, !t10) outs(%f : !t2) -> !t2
    %s = tensor.empty() : !t2
    %P = linalg.softmax dimension(1) ins(%C : !t2) outs(%s : !t2) -> !t2
    return %P : !t2
  }
}
""")
    r = run(["--input", str(nested), "--out-dir", str(tmp_path / "o3"), "--search-only", "--backend-mode", "api"])
    assert r.returncode == 0, r.stderr
    c = json.load(open(tmp_path / "o3" / "ir" / "chain.json"))
    assert (c["M"], c["N"], c["K"], c["softmax_form"]) == (8, 24, 16, "named")


def test_tile_source_priority_and_overrides(tmp_path):
    inp = os.path.join(MLIR, "cfg2_f16_native_4096x1024x1024.mlir")
    bj = tmp_path / "best.json"
    # a nested summary loads too: the first occurrence of each key wins
    bj.write_text('{"problem": {"m": 1}, "best": {"tileM": 64, "tileN": 128, "tileK": 32, "threadTileM": 8, "threadTileN": 2}}')
    out = tmp_path / "o"
    r = run(["--input", inp, "--out-dir", str(out), "--backend-mode", "api", "--compile-only", "--best-json", str(bj), "--tile-k", "16"])
    assert r.returncode == 0, r.stderr
    assert not (out / "search/best_summary.json").exists()            # --best-json given: no search
    assert json.load(open(out / "search/best.json")) == dict(tileM=64, tileN=128, tileK=16, threadTileM=8, threadTileN=2)
    plan = open(out / "fused/05.out.nvvm.runnable.mlir").read()
    # 64-row tiles and the 128-column tile are honoured; a 16-deep stage has no kernel and is replaced
    assert "requested_m = 64" in plan and "tile_m = 64" in plan and "requested_k = 16" in plan and "tile_k = 64" in plan and "substituted = 1" in plan
    assert "substituted" in open(out / "fused/compile.log").read()
    # --no-search without tiles: built-in defaults 32x64x16, thread tile 2x2
    out2 = tmp_path / "o2"
    assert run(["--input", inp, "--out-dir", str(out2), "--backend-mode", "api", "--no-search"]).returncode == 0
    assert json.load(open(out2 / "search/best.json")) == dict(tileM=32, tileN=64, tileK=16, threadTileM=2, threadTileN=2)


def test_baseline_variant_and_repeat(tmp_path):
    inp = os.path.join(MLIR, "matmul_softmax_chain_f16_native.mlir")
    out = tmp_path / "o"
    assert run(["--input", inp, "--out-dir", str(out), "--backend-mode", "api", "--baseline"]).returncode == 0
    assert open(out / "baseline/04.after_workgroup_launch.mlir").read().count("gpu.launch") == 5
    assert "launch_kernel_count=5" in open(out / "baseline/postbufferize_report.txt").read()
    out = tmp_path / "rep"
    r = run(["--input", inp, "--out-dir", str(out), "--backend-mode", "api", "--pure-api-full", "--repeat", "25"])
    assert r.returncode == 0, r.stderr
    assert (out / "iter_24/fused/05.out.nvvm.runnable.mlir").exists()


def test_usage_and_stage_errors(tmp_path):
    assert run([]).returncode == 2
    assert run(["--bogus"]).returncode == 2
    assert run(["--input", "x.mlir", "--backend-mode", "nope"]).returncode == 2
    assert run(["--input", "x.mlir", "--repeat", "0"]).returncode == 2
    r = run(["--input", str(tmp_path / "missing.mlir"), "--out-dir", str(tmp_path / "o")])
    assert r.returncode == 1 and "canonicalize failed" in r.stderr
    bad = tmp_path / "bad.mlir"
    bad.write_text("module { func.func @main(%A: tensor<4x4xf32>, %B: tensor<4x4xf32>) -> tensor<4x4xf32> { return %A : tensor<4x4xf32> } }")
    r = run(["--input", str(bad), "--out-dir", str(tmp_path / "o")])
    assert r.returncode == 1 and "matmul" in r.stderr
    src = open(os.path.join(MLIR, "cfg1_decomposed_f32_128.mlir")).read()
    assert "%B: !t0" in src and "!t0 = tensor<128x128xf32>" in src          # the shipped inputs name their types once (aliases)
    mism = src.replace("%B: !t0", "%B: tensor<64x128xf32>")
    (tmp_path / "mism.mlir").write_text(mism)
    r = run(["--input", str(tmp_path / "mism.mlir"), "--out-dir", str(tmp_path / "o")])
    assert r.returncode == 1
    r = run(["--input", os.path.join(MLIR, "cfg1_decomposed_f32_128.mlir"), "--out-dir", str(tmp_path / "o3"), "--backend-root", str(tmp_path / "nowhere")])
    assert r.returncode == 1 and "backend root not found" in r.stderr
    # a non-positive override is ignored (only values > 0 apply); a non-positive tile in best.json is refused
    r = run(["--input", os.path.join(MLIR, "cfg1_decomposed_f32_128.mlir"), "--out-dir", str(tmp_path / "o4"), "--no-search", "--tile-m", "-4", "--backend-mode", "api"])
    assert r.returncode == 0
    zero = tmp_path / "zero.json"
    zero.write_text('{"tileM": 0, "tileN": 64, "tileK": 16, "threadTileM": 2, "threadTileN": 2}')
    for mode in ("api", "process_chain"):
        r = run(["--input", os.path.join(MLIR, "cfg1_decomposed_f32_128.mlir"), "--out-dir", str(tmp_path / "o5"), "--best-json", str(zero), "--backend-mode", mode])
        assert r.returncode == 1 and "tile" in r.stderr


def test_solver_and_compile_c_api_directly(tmp_path):
    inp = os.path.join(MLIR, "cfg4_vocab_logits.mlir").encode()
    S = ctypes.CDLL(os.path.join(BK, "libwelder-solver-capi.so"))
    tiles = [ctypes.c_int64(0) for _ in range(5)]
    err = ctypes.create_string_buffer(4096)
    rc = S.welder_solver_solve_typical_chain(inp, str(tmp_path / "bs.json").encode(), str(tmp_path / "c.tsv").encode(), ctypes.c_int64(1), 0,
                                             *[ctypes.byref(t) for t in tiles], err, ctypes.c_size_t(4096))
    assert rc == 0 and [t.value for t in tiles] == [128, 256, 64, 1, 128] and err.value == b""
    header = open(tmp_path / "c.tsv").readline().split("\t")
    assert len(header) == 13 and header[:6] == ["rank", "tileM", "tileN", "tileK", "threadTileM", "threadTileN"]
    summary = json.load(open(tmp_path / "bs.json"))
    assert summary["problem"] == dict(m=8192, n=32000, k=4096, batch=1) and summary["arch"]["numSM"] == 148
    assert summary["best"]["bytesCut"] > 0          # two-pass: the output crosses HBM again
    rc = S.welder_solver_solve_typical_chain(b"/nonexistent.mlir", None, None, ctypes.c_int64(1), 0, *[ctypes.byref(t) for t in tiles], err, ctypes.c_size_t(4096))
    assert rc == 2 and b"failed to read" in err.value
    assert S.welder_solver_solve_typical_chain(None, None, None, ctypes.c_int64(1), 0, *[ctypes.byref(t) for t in tiles], err, ctypes.c_size_t(4096)) == 1
    Cc = ctypes.CDLL(os.path.join(BK, "libwelder-compile-capi.so"))
    args = lambda tm: (inp, str(tmp_path / "cc").encode(), b"", b"", ctypes.c_int64(tm), ctypes.c_int64(256), ctypes.c_int64(64),
                       ctypes.c_int64(1), ctypes.c_int64(128), ctypes.c_int64(1), 1, 0, err, ctypes.c_size_t(4096))
    assert Cc.welder_compile_typical_chain_to_nvvm(*args(128)) == 0
    assert 'kernel = "tc_tiled"' in open(tmp_path / "cc" / "05.out.nvvm.runnable.mlir").read()
    assert Cc.welder_compile_typical_chain_to_nvvm(*args(0)) == 1 and err.value == b"invalid tile sizes"
    small = ctypes.create_string_buffer(8)            # the buffer is always NUL-terminated, however small
    a = list(args(0)); a[-2], a[-1] = small, ctypes.c_size_t(8)
    assert Cc.welder_compile_typical_chain_to_nvvm(*a) == 1 and small.value == b"invalid"


def test_harness_scripts_without_gpu(tmp_path):
    env = dict(os.environ, OUT_BASE=str(tmp_path / "reg"), PURE_API_REPEAT="5")
    r = subprocess.run(["bash", os.path.join(PKG, "bench", "run_regression.sh")], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    rows = open(tmp_path / "reg" / "regression_summary.tsv").read().splitlines()[1:]
    assert len(rows) >= 14 and all(x.split("\t")[1] == "PASS" for x in rows)
    env = dict(os.environ, OUT_BASE=str(tmp_path / "st"), REPEAT="30")
    r = subprocess.run(["bash", os.path.join(PKG, "bench", "run_pure_api_stress.sh")], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "stress passed" in r.stdout
    # perf guard arithmetic on synthetic summaries
    base, cur = tmp_path / "base", tmp_path / "cur"
    for d, (b, f) in ((base, (1.0, 0.5)), (cur, (1.02, 0.51))):
        d.mkdir()
        (d / "ab_summary.tsv").write_text(f"case\tavg_ms\nbaseline\t{b}\t5\nfused\t{f}\t1\n")
        (d / "speedup.tsv").write_text(f"speedup\t{b / f:.4f}\n")
    env = dict(os.environ, BASELINE_DIR=str(base), CURRENT_OUT_BASE=str(cur))
    r = subprocess.run(["bash", os.path.join(PKG, "bench", "check_perf_guard.sh")], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and r.stdout.count("PASS") == 3
    (cur / "ab_summary.tsv").write_text("case\tavg_ms\nbaseline\t1.0\t5\nfused\t0.6\t1\n")
    r = subprocess.run(["bash", os.path.join(PKG, "bench", "check_perf_guard.sh")], capture_output=True, text=True, env=env)
    assert r.returncode == 1 and "FAIL fused.avg_ms" in r.stdout


def test_trace_file(tmp_path):
    env = dict(os.environ, WTC_TRACE_FILE=str(tmp_path / "trace.jsonl"))
    r = run(["--input", os.path.join(MLIR, "cfg1_decomposed_f32_128.mlir"), "--out-dir", str(tmp_path / "o"), "--backend-mode", "api", "--pure-api-full"], env=env)
    assert r.returncode == 0
    spans = [json.loads(l) for l in open(tmp_path / "trace.jsonl")]
    assert {s["name"] for s in spans} >= {"canonicalize", "tagging", "search", "compile"} and all(s["ok"] for s in spans)


def test_solver_profiles_top_candidates_through_the_profiler_binary(tmp_path):
    """--enable-profiling: each implemented candidate is compiled to a plan and handed to the
    profiler binary (a stand-in here: no GPU), its avg_ms lands in candidates.tsv and in the
    append-only cache, the measured candidates are re-ranked by time, and a second run is served
    from the cache without starting the profiler (solver/WelderSolver.cpp:202-213,479-513)."""
    fake = tmp_path / "fake-profiler"
    calls = tmp_path / "calls.log"
    # 128-column tiles "run" faster than 256-column ones, the opposite of the model's order
    fake.write_text("#!/bin/bash\nplan=\"${@: -1}\"\necho \"$@\" >> %s\n"
                    "if grep -q ', tile_n = 128,' \"$plan\"; then echo 'avg_ms=0.2500 iters=3 warmup=1'; else echo 'avg_ms=0.7500 iters=3 warmup=1'; fi\n" % calls)
    fake.chmod(0o755)
    solver = os.path.join(BK, "welder-solver")
    cache = tmp_path / "profile_cache.tsv"
    args = [solver, os.path.join(MLIR, "cfg2_f16_native_4096x1024x1024.mlir"), "--enable-generic-problem", "--max-connect-level", "1",
            "--dump-best-summary-json", str(tmp_path / "bs.json"), "--dump-candidates-tsv", str(tmp_path / "c.tsv"),
            "--enable-profiling", "--schedule-topk", "3", "--profile-warmup", "1", "--profile-iters=3",
            "--profile-cache", str(cache), "--profile-profiler-bin", str(fake)]
    r = subprocess.run(args, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "tileN=128" in r.stdout                      # the faster measured tile wins over the model's first choice
    rows = [l.split("\t") for l in open(tmp_path / "c.tsv").read().splitlines()]
    col = rows[0].index("profiledMs")
    # (the model's first three: 128x256x64, its 32-deep sibling, then 128x128x64)
    assert [float(x[col]) for x in rows[1:4]] == [0.25, 0.75, 0.75] and all(float(x[col]) == -1 for x in rows[4:])
    assert json.load(open(tmp_path / "bs.json"))["best"]["profiledMs"] == 0.25
    lines = open(cache).read().splitlines()
    assert len(lines) == 3 and all(re.fullmatch(r"wtc_b200_chain\|.*\|tile=128x(128|256)x(32|64)\|level=1\|profile_key_rev=\S+\t0\.(25|75)", l) for l in lines)
    assert len(open(calls).read().splitlines()) == 3 and "--warmup=1 --iters=3" in open(calls).read()
    # second run: the cache answers, the profiler is not started (it would now fail)
    fake.write_text("#!/bin/bash\nexit 3\n")
    r = subprocess.run(args, capture_output=True, text=True)
    assert r.returncode == 0 and "tileN=128" in r.stdout
    assert len(open(cache).read().splitlines()) == 3
    # a profiler that fails leaves the candidates unmeasured and the model's order in place
    r = subprocess.run(args[:-4] + ["--profile-profiler-bin", str(fake)], capture_output=True, text=True)
    assert r.returncode == 0 and "tileN=256" in r.stdout


def _chain_gen():
    import importlib.util
    spec = importlib.util.spec_from_file_location("chain_gen", os.path.join(os.path.dirname(os.path.abspath(__file__)), "chain_gen.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    return gen


def test_chains_that_are_not_the_operator_are_rejected(tmp_path):
    """The recogniser follows the dataflow: anything that is not scale * A . B followed by a row
    softmax is refused at the canonicalize stage instead of being compiled as the fixed kernel."""
    gen = _chain_gen()
    ok = dict(batch=1, M=256, N=512, K=64, in_t="f16", out_t="f16", scale=0.125)
    cases = {
        "factor after the division": (gen.chain(**ok, post_scale=2.0), "division"),
        "non-zero matmul init": (gen.chain(**ok, fill="1.0"), "zero fill"),
        "constant added to the logits": (gen.chain(**ok, extra_add=0.5), "between the matmul and the softmax"),
        "factor after a named softmax": (gen.chain(**ok, named=True, post_scale=0.5), "division"),
    }
    # a sum that does not start from zero, a maximum that starts from zero, an exp of the wrong difference,
    # swapped matmul operands, a second (dead) generic
    good = gen.chain(**ok, aliases=False)
    cases["row sum from 1"] = (good.replace("%zero = arith.constant 0.0 : f32", "%zero = arith.constant 1.0 : f32"), "start from 0")
    cases["row max from 0"] = (good.replace("%neg_inf = arith.constant -3.4028235e+38 : f32", "%neg_inf = arith.constant 0.0 : f32"), "most negative")
    cases["exp(max - x)"] = (good.replace("%d = arith.subf %x, %m : f32", "%d = arith.subf %m, %x : f32"), "math.exp(x - row_max)")
    cases["min instead of max"] = (good.replace("arith.maximumf", "arith.minimumf"), "row maximum")
    sq = gen.chain(batch=1, M=64, N=64, K=64, aliases=False)
    cases["B . A"] = (sq.replace("ins(%A, %B :", "ins(%B, %A :"), "first and second argument")
    cases["an operation outside the chain"] = (good.replace("    return %P16", "    %dead_empty = tensor.empty() : tensor<256x512xf32>\n"
                                               "    %dead = linalg.fill ins(%zero : f32) outs(%dead_empty : tensor<256x512xf32>) -> tensor<256x512xf32>\n    return %P16"), "outside the chain")
    for name, (text, needle) in cases.items():
        path = tmp_path / "bad.mlir"
        path.write_text(text)
        r = run(["--input", str(path), "--out-dir", str(tmp_path / "o"), "--search-only", "--backend-mode", "api"])
        assert r.returncode == 1, name
        assert "canonicalize failed" in r.stderr and needle in r.stderr, (name, r.stderr)
    # and the unbroken chain, in both spellings, is accepted
    for text in (gen.chain(**ok), good):
        path = tmp_path / "good.mlir"
        path.write_text(text)
        assert run(["--input", str(path), "--out-dir", str(tmp_path / "g"), "--search-only", "--backend-mode", "api"]).returncode == 0


# the reference tree: $WTC_REFERENCE_ROOT, else a directory `reference` beside this repository
REFERENCE_ROOT = os.environ.get("WTC_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_ROOT, "mlir")), reason="the reference tree is not mounted here")
def test_the_reference_inputs_compile_unmodified(tmp_path):
    """The reference's own operator inputs, read where they lie (they are not copied into this
    repository), go through the whole front-end: canonicalize, tag, search, compile."""
    files = [os.path.join(REFERENCE_ROOT, "mlir", f) for f in ("matmul_softmax_chain.mlir", "matmul_softmax_chain_f16_native.mlir",
                                                               "matmul_softmax_chain_named_softmax.mlir")]
    files.append(os.path.join(REFERENCE_ROOT, "backend/welder/mlir_pipeline/matmul_softmax_chain_f16_matmul.mlir"))
    want = {"matmul_softmax_chain.mlir": ("f32", "f32", "f32", "decomposed"), "matmul_softmax_chain_f16_native.mlir": ("f16", "f16", "f32", "decomposed"),
            "matmul_softmax_chain_named_softmax.mlir": ("f32", "f32", "f32", "named"), "matmul_softmax_chain_f16_matmul.mlir": ("f16", "f16", "f32", "decomposed")}
    for f in files:
        out = tmp_path / os.path.basename(f)
        r = run(["--input", f, "--out-dir", str(out), "--backend-mode", "api"])
        assert r.returncode == 0, (f, r.stderr)
        c = json.load(open(out / "ir" / "chain.json"))
        assert (c["batch"], c["M"], c["N"], c["K"], c["scale"]) == (1, 8192, 128, 64, 1), f
        assert (c["in_dtype"], c["acc_dtype"], c["out_dtype"], c["softmax_form"]) == want[os.path.basename(f)], f
        assert (out / "fused/05.out.nvvm.runnable.mlir").exists()


def test_generated_chains_round_trip_through_the_recogniser(tmp_path):
    """Every spelling the generator can write (decomposed / named softmax, batched, scaled, f16
    operands and results, f32 arguments rounded to f16) parses back to the shapes, types and
    scale it was written with, through the search-only front-end."""
    import random
    gen = _chain_gen()
    rng = random.Random(7)
    for case in range(24):
        batch = rng.choice([1, 1, 3, 8])
        M, N, K = rng.randrange(1, 5000), rng.randrange(1, 40000), rng.randrange(1, 3000)
        in_t = rng.choice(["f32", "f16"])
        arg_t = "f32" if (in_t == "f16" and rng.random() < 0.3) else None
        acc_t = rng.choice(["f32", "f16"]) if in_t == "f16" else "f32"
        out_t = rng.choice(["f32", "f16"]) if in_t == "f16" else "f32"
        scale = rng.choice([1.0, 0.125, 1.0 / 3.0, 17.5])
        named = rng.random() < 0.4
        path = tmp_path / f"c{case}.mlir"
        path.write_text(gen.chain(batch, M, N, K, in_t=in_t, acc_t=acc_t, out_t=out_t, scale=scale, named=named, title=f"case {case}", arg_t=arg_t,
                                  aliases=rng.random() < 0.5))
        out = tmp_path / f"o{case}"
        r = run(["--input", str(path), "--out-dir", str(out), "--search-only", "--backend-mode", "api"])
        assert r.returncode == 0, (case, r.stderr)
        c = json.load(open(out / "ir" / "chain.json"))
        assert (c["batch"], c["M"], c["N"], c["K"]) == (batch, M, N, K), case
        assert (c["arg_dtype"], c["in_dtype"], c["acc_dtype"], c["out_dtype"]) == (arg_t or in_t, in_t, acc_t, out_t), case
        assert abs(c["scale"] - scale) <= 1e-6 * scale and c["softmax_form"] == ("named" if named else "decomposed"), case
        best = json.load(open(out / "search" / "best.json"))
        assert best["tileM"] > 0 and best["tileN"] > 0 and best["tileK"] > 0


def test_row_only_chains_through_the_backend_compiler(tmp_path):
    """The two chains without a matmul (row softmax of a given matrix; the layernorm-style
    variance chain) are recognised by their dataflow and compiled to a one-kernel plan by the
    backend compiler; the front-end refuses them at the canonicalize stage, as the reference's
    does (its canonical form must contain a matmul)."""
    gen = _chain_gen()
    wc = os.path.join(BK, "welder-compiler")
    tiles = ["--force-tile-m", "32", "--force-tile-n", "64", "--force-tile-k", "16", "--thread-tile-m", "2", "--thread-tile-n", "2"]
    cases = [("softmax_row_chain.mlir", None, "row_softmax", 32, 256), ("layernorm_variance_chain.mlir", None, "layernorm_variance", 32, 256),
             (None, gen.row_softmax_chain(1000, 4104, named=True), "row_softmax", 1000, 4104),
             (None, gen.row_softmax_chain(7, 24, aliases=False), "row_softmax", 7, 24),
             (None, gen.layernorm_variance_chain(513, 1000, aliases=False), "layernorm_variance", 513, 1000)]
    for name, text, kind, M, N in cases:
        if text is None:
            path = os.path.join(MLIR, name)
        else:
            path = str(tmp_path / "in.mlir")
            open(path, "w").write(text)
        out = tmp_path / f"o_{kind}_{M}"
        r = subprocess.run([wc, path, *tiles, "--emit-all-stages", "--output", str(out / "03.after_postbufferize.mlir")], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        plan = open(out / "05.out.nvvm.runnable.mlir").read()
        assert f'kind = "{kind}"' in plan and f"M = {M}, N = {N}, K = 0" in plan and "launches = 1" in plan
        if kind == "layernorm_variance":
            m = re.search(r"mean_factor = ([-+0-9.e]+), var_factor = ([-+0-9.e]+)", plan)
            assert abs(float(m.group(1)) - 1.0 / N) < 1e-9 and abs(float(m.group(2)) - 1.0 / N) < 1e-9
        for f in ("03.after_postbufferize.mlir", "04.after_workgroup_launch.mlir", "04c.after_linalg_to_loops.mlir", "compile.log"):
            assert (out / f).stat().st_size > 0
    r = run(["--input", os.path.join(MLIR, "softmax_row_chain.mlir"), "--out-dir", str(tmp_path / "fe")])
    assert r.returncode == 1 and "matmul" in r.stderr
    # broken variants are refused by the backend compiler too
    bad = gen.layernorm_variance_chain(32, 256, aliases=False).replace("%s = arith.mulf %d, %d : f32", "%s = arith.mulf %d, %a : f32")
    open(tmp_path / "bad.mlir", "w").write(bad)
    r = subprocess.run([wc, str(tmp_path / "bad.mlir"), *tiles, "--emit-all-stages", "--output", str(tmp_path / "b" / "03.mlir")], capture_output=True, text=True)
    assert r.returncode != 0 and "(a - mean)^2" in r.stderr
