#!/usr/bin/env python3
"""Checks a dumped Matmul->Softmax result against a CPU computation on sampled rows.

Same role and verdict line as the reference harness' checker
(backend/welder/bench/verify_matmul_softmax.py:134-272 behind bench/verify.py:13-60): the inputs
are regenerated from the profiler's pattern and seed, each sampled row is contracted in float64,
softmax-ed with max subtraction, and every element must satisfy |out - ref| <= atol + rtol*|ref|.
Unlike the reference's wrapper this one forwards the chain's own M/N/K, scale and element types:
it reads them from the compiled plan (--plan <05.out.nvvm.runnable.mlir>) or from flags.

  verify.py --out out.bin [--plan PLAN | --k K [--scale S] [--matmul-f16]] [--pattern linear] [--seed 1]
            [--rows 0,1,2,...] [--rtol 1e-2] [--atol 1e-2] [--f16-rne]
"""
import argparse
import json
import re
import sys

import numpy as np


def linear_vals(count):
    return (np.arange(count, dtype=np.int64) % 1024).astype(np.float32) * np.float32(0.001) - np.float32(0.5)


def random_vals(count, seed):
    s = 1 if seed == 0 else int(seed) & 0xFFFFFFFF
    out = np.empty(count, dtype=np.float32)
    inv = np.float32(1.0 / 4294967296.0)
    for i in range(count):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32(s) * inv * np.float32(2.0) - np.float32(1.0)
    return out


def to_f16_profiler(x):
    """f32 -> f16 the way the profiler's f16 initialiser rounds: add half an ulp, truncate."""
    u = x.astype(np.float32).view(np.uint32).astype(np.int64)
    sign = (u >> 31) & 1
    exp = (u >> 23) & 0xFF
    mant = u & 0x7FFFFF
    he = exp - 127 + 15
    r = mant + 0x1000
    carry = (r & 0x800000) != 0
    he_n = np.where(carry, he + 1, he)
    r = np.where(carry, 0, r)
    normal = (he_n << 10) | ((r >> 13) & 0x3FF)
    normal = np.where(he_n >= 31, 0x7C00, normal)
    shift = np.clip(14 - he, 1, 31)
    sub = ((mant | 0x800000) + (1 << (shift - 1))) >> shift
    sub = np.where(he < -10, 0, sub)
    bits = np.where(he <= 0, sub, normal)
    bits = np.where(exp == 0xFF, np.where(mant == 0, 0x7C00, 0x7E00), bits)
    return ((sign << 15) | bits).astype(np.uint16).view(np.float16)


def plan_attrs(path):
    text = open(path).read()
    def geti(k, d=None):
        m = re.search(r"\b%s\s*=\s*(-?[0-9]+)" % k, text)
        return int(m.group(1)) if m else d
    def gets(k, d=None):
        m = re.search(r'\b%s\s*=\s*"([^"]*)"' % k, text)
        return m.group(1) if m else d
    m = re.search(r"\bscale\s*=\s*([-+0-9.eE]+)", text)
    def getf(k, d=0.0):
        mm = re.search(r"\b%s\s*=\s*([-+0-9.eE]+)" % k, text)
        return float(mm.group(1)) if mm else d
    return dict(batch=geti("batch", 1), M=geti("M"), N=geti("N"), K=geti("K"), in_dtype=gets("in_dtype", "f32"),
                arg_dtype=gets("arg_dtype", None), acc_dtype=gets("acc_dtype", "f32"), scale=float(m.group(1)) if m else 1.0,
                kind=gets("kind", "matmul_softmax"), mean_factor=getf("mean_factor"), var_factor=getf("var_factor"))


def main():
    ap = argparse.ArgumentParser(description="Verify a Matmul->Softmax output dump against a CPU reference (sampled rows).")
    ap.add_argument("--out", required=True)
    ap.add_argument("--plan", default="")
    ap.add_argument("--m", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=64)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--pattern", default="linear", choices=["zero", "linear", "random"])
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--rows", default="0,1,2,3,7,15,31,63,127,255,511,1023")
    ap.add_argument("--rtol", type=float, default=1e-2)
    ap.add_argument("--atol", type=float, default=1e-2)
    ap.add_argument("--matmul-f16", action="store_true", help="operands were f16 buffers")
    ap.add_argument("--f16-rne", action="store_true", help="f16 operands were rounded to nearest even (runner --f16-rne)")
    ap.add_argument("--backend-root", default="", help="accepted for compatibility; unused")
    args = ap.parse_args()

    meta = json.load(open(args.out + ".json"))
    if int(meta.get("rank", 0)) != 2 or int(meta.get("elem_bytes", 0)) not in (2, 4):
        raise SystemExit(f"error: expected a rank-2 dump of 2- or 4-byte elements, got {meta}")
    dump_m, dump_n = (int(x) for x in meta["sizes"])
    s0, s1 = (int(x) for x in meta["strides"])
    raw = np.fromfile(args.out, dtype=np.float16 if meta["elem_bytes"] == 2 else np.float32)
    out = np.lib.stride_tricks.as_strided(raw[int(meta["offset"]):], shape=(dump_m, dump_n),
                                          strides=(s0 * raw.itemsize, s1 * raw.itemsize)).astype(np.float64)
    k, scale, f16 = args.k, args.scale, args.matmul_f16
    kind, c1, c2 = "matmul_softmax", 0.0, 0.0
    if args.plan:
        p = plan_attrs(args.plan)
        k, scale, f16 = p["K"], p["scale"], p["in_dtype"] == "f16"
        kind, c1, c2 = p["kind"], p["mean_factor"], p["var_factor"]
        if f16 and p["arg_dtype"] == "f32":
            args.f16_rne = True      # f32 buffers rounded on the device by arith.truncf: round to nearest even
    m = dump_m if args.m <= 0 else args.m
    n = dump_n if args.n <= 0 else args.n
    if m > dump_m or n > dump_n:
        raise SystemExit(f"error: runtime extents exceed dump extents: runtime=({m},{n}) dump=({dump_m},{dump_n})")
    rows = [int(t) for t in args.rows.split(",") if t.strip()]
    rows = [r for r in rows if 0 <= r < m]
    if not rows:
        raise SystemExit("error: no valid --rows selected")

    def gen(count):
        if args.pattern == "zero":
            return np.zeros(count, dtype=np.float32)
        return linear_vals(count) if args.pattern == "linear" else random_vals(count, args.seed)

    def as_operand(x):
        if not f16:
            return x.astype(np.float64)
        return (x.astype(np.float16) if args.f16_rne else to_f16_profiler(x)).astype(np.float64)

    row_only = kind in ("row_softmax", "layernorm_variance")   # the chains without a matmul: one input X[m, n]
    if row_only:
        x_flat = gen((max(rows) + 1) * n)
    else:
        B = as_operand(gen(k * n)).reshape(k, n)
        a_flat = gen((max(rows) + 1) * k)
    ok, max_abs, max_rel = True, 0.0, 0.0
    for i in rows:
        if row_only:
            x = as_operand(x_flat[i * n:(i + 1) * n])
            if kind == "row_softmax":
                e = np.exp(x - x.max())
                ref = e / e.sum()
            else:
                mean = x.sum() * c1
                ref = np.full(n, ((x - mean) ** 2).sum() * c2)
        else:
            a = as_operand(a_flat[i * k:(i + 1) * k])
            c = scale * (a @ B)
            e = np.exp(c - c.max())
            ref = e / e.sum()
        got = out[i, :n]
        if not np.isfinite(got).all():
            print("FAIL: output contains NaN/Inf")
            return 1
        diff = np.abs(got - ref)
        max_abs = max(max_abs, float(diff.max()))
        max_rel = max(max_rel, float((diff / np.maximum(np.abs(ref), 1e-6)).max()))
        if (diff > args.atol + args.rtol * np.abs(ref)).any():
            ok = False
    print(f"{'PASS' if ok else 'FAIL'}: max_abs={max_abs:.6e} max_rel={max_rel:.6e} shape=({m},{n}) rows={len(rows)}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
