#!/usr/bin/env python3
"""Regenerates the fixtures in this folder.  Needs the reference tree (it imports
the reference's Python checker and loads the shim built around the reference
profiler's generator headers), so it runs only where that tree is mounted; the
fixtures it writes are what travels.

    python tests/golden/make_golden.py [--reference /path/to/reference]

Writes:
  generators.npz   input streams and f32->f16 conversions taken FROM THE REFERENCE:
                   * `py_*`  : backend/welder/bench/verify_matmul_softmax.py
                               (_linear_val, _random_vals, _f32_to_f16_bits)
                   * `cxx_*` : backend/welder/compiler/solver/WelderProfilerRuntime.h
                               (initMemrefF32/F16) and WelderProfilerEval.h (f32ToF16Bits),
                               compiled where they lie into oracle/_ref/libref_gen.so
  chain_kat.npz    small known-answer cases: inputs, and probabilities from this
                   repo's CPU checker, each of which the reference's unmodified
                   checker script accepted at rtol=1e-5/atol=1e-7 when the fixture
                   was made (its verdict lines are stored in chain_kat.json).
"""
import argparse
import contextlib
import ctypes
import importlib.util
import io
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402


def load_ref_checker(ref_root):
    path = os.path.join(ref_root, "backend/welder/bench/verify_matmul_softmax.py")
    spec = importlib.util.spec_from_file_location("ref_verify", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def special_floats():
    vals = [0.0, -0.0, 1.0, -1.0, 0.5, 65504.0, 65520.0, 65519.99, 70000.0, 1e-8, 5.96e-8, 2.98e-8,
            2.9802322e-8, 6.1035156e-5, 6.0975552e-5, 1.0009765625, 1.00048828125, 1.00146484375,
            0.33325195, 0.1, -0.1, 3.14159, 1e-5, 1e-6, 1e-7, 2049.0, 2051.0, 2050.0, 4098.0, 1023.5]
    rng = np.random.Generator(np.random.PCG64(7))
    vals += list(rng.standard_normal(200).astype(np.float32))
    vals += list((rng.standard_normal(100) * 1e-5).astype(np.float32))
    # exact ties between two f16 neighbours, both parities
    for base in (1.0, 2.0, 0.25, 1024.0):
        for k in range(6):
            vals.append(base * (1.0 + (2 * k + 1) / 2048.0))
    return np.array(vals, dtype=np.float32)


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--reference", default=os.environ.get("WTC_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"),
                    help="the reference tree ($WTC_REFERENCE_ROOT, else a directory `reference` beside this repository)")
    args = ap.parse_args()
    ref = load_ref_checker(args.reference)

    out = {}
    n = 4096
    out["py_linear"] = np.array([ref._linear_val(i) for i in range(n)], dtype=np.float64)
    for seed in (0, 1, 12345):
        out[f"py_random_seed{seed}"] = np.array(ref._random_vals(n, seed), dtype=np.float64)
    sp = special_floats()
    out["special_f32"] = sp
    out["py_f16_bits"] = np.array([ref._f32_to_f16_bits(float(x)) for x in sp], dtype=np.uint16)

    so = os.path.join(ROOT, "oracle", "_ref", "libref_gen.so")
    L = ctypes.CDLL(so)
    L.ref_f32_to_f16_bits.restype = ctypes.c_uint16
    L.ref_f32_to_f16_bits.argtypes = [ctypes.c_float]
    L.ref_init_f32.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_char_p, ctypes.c_uint64]
    L.ref_init_f16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_char_p, ctypes.c_uint64]
    out["cxx_f16_bits"] = np.array([L.ref_f32_to_f16_bits(float(x)) for x in sp], dtype=np.uint16)
    for mode in ("linear", "random"):
        for seed in (0, 1, 12345):
            if mode == "linear" and seed != 1:
                continue
            b32 = np.zeros((37, 111), dtype=np.float32)
            L.ref_init_f32(b32.ctypes.data, 37, 111, mode.encode(), seed)
            out[f"cxx_{mode}_f32_seed{seed}"] = b32
            b16 = np.zeros((37, 111), dtype=np.uint16)
            L.ref_init_f16(b16.ctypes.data, 37, 111, mode.encode(), seed)
            out[f"cxx_{mode}_f16_seed{seed}"] = b16
    np.savez_compressed(os.path.join(HERE, "generators.npz"), **out)

    # ---- chain known answers, each accepted by the reference's own checker
    kat = {}
    verdicts = {}
    cases = [
        # name, M, K, N, pattern, f16 operands
        ("lin_16x8x12", 16, 8, 12, "linear", False),
        ("rnd_16x8x12", 16, 8, 12, "random", False),
        ("rnd_128x128x128", 128, 128, 128, "random", False),   # benchmark configuration 1
        ("lin_f16_64x64x128", 64, 64, 128, "linear", True),    # the reference's own K and N
        ("rnd_f16_32x64x128", 32, 64, 128, "random", True),
    ]
    for name, M, K, N, pat, f16 in cases:
        A = oracle.fill((M, K), pat, 1)
        B = oracle.fill((K, N), pat, 1)
        if f16:
            # The checker's --matmul-f16 rounds ITS OWN f64 streams to nearest-even
            # f16 (the profiler computes the streams in f32, which can land one f16
            # step away), so take the operands from the checker's generators.
            if pat == "random":
                a64 = ref._random_vals(M * K, 1)
                b64 = ref._random_vals(K * N, 1)
            else:
                a64 = [ref._linear_val(i) for i in range(M * K)]
                b64 = [ref._linear_val(i) for i in range(K * N)]
            A = np.array([ref._to_f16_f32(x) for x in a64], dtype=np.float32).reshape(M, K)
            B = np.array([ref._to_f16_f32(x) for x in b64], dtype=np.float32).reshape(K, N)
        p = oracle.chain(A, B, 1.0)
        with tempfile.TemporaryDirectory() as td:
            dump = os.path.join(td, "out.bin")
            oracle.write_dump(dump, p.astype(np.float32))
            argv = ["verify", "--out", dump, "--k", str(K), "--pattern", pat, "--seed", "1",
                    "--rtol", "1e-5", "--atol", "1e-7",
                    "--rows", ",".join(str(i) for i in range(M))]
            if f16:
                argv.append("--matmul-f16")
            old = sys.argv
            sys.argv = argv
            buf = io.StringIO()
            try:
                with contextlib.redirect_stdout(buf):
                    rc = ref.main()
            finally:
                sys.argv = old
        line = buf.getvalue().strip()
        if rc != 0:
            raise SystemExit(f"reference checker rejected the oracle on {name}: {line}")
        verdicts[name] = line
        kat[name + "_A"] = A
        kat[name + "_B"] = B
        kat[name + "_P"] = p
    np.savez_compressed(os.path.join(HERE, "chain_kat.npz"), **kat)
    with open(os.path.join(HERE, "chain_kat.json"), "w") as f:
        json.dump(dict(cases=[c[0] for c in cases], reference_checker_verdicts=verdicts,
                       reference_checker="backend/welder/bench/verify_matmul_softmax.py",
                       rtol=1e-5, atol=1e-7), f, indent=2)
    for k, v in verdicts.items():
        print(k, "->", v)


if __name__ == "__main__":
    main()
