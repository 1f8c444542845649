"""TEST INFRASTRUCTURE ONLY: numpy/ctypes front of the CPU checker in chain_oracle.c.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import
this module; the product never does, and has no CPU fallback.

The functions restate, on the CPU, the chain the reference spells in MLIR
(mlir/matmul_softmax_chain.mlir:15-80; casts as in
mlir/matmul_softmax_chain_f16_native.mlir:13-31) with the math of the reference's
own checker (backend/welder/bench/verify_matmul_softmax.py:242-265), plus the
reference profiler's input generators
(backend/welder/compiler/solver/WelderProfilerRuntime.h:128-168,193-231).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

DT_F32, DT_F16 = 0, 1
ACC_F64, ACC_F32_SEQ, ACC_F16_SEQ = 0, 1, 2
MODES = {"zero": 0, "linear": 1, "random": 2}

# tolerances of the parity contract
TOL_PROB_ABS = 2e-3
TOL_ROWSUM = 1e-3


def build(force: bool = False) -> str:
    """Compile chain_oracle.c into liboracle.so next to it (gcc, seconds)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "chain_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        c = ctypes
        L.wtc_oracle_chain.restype = c.c_int
        L.wtc_oracle_chain.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                                       c.c_int64, c.c_int64, c.c_int64, c.c_int64,
                                       c.c_int, c.c_double, c.c_int, c.c_int64, c.c_int]
        L.wtc_oracle_chain_loops_f32.restype = c.c_int
        L.wtc_oracle_chain_loops_f32.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p,
                                                 c.c_int64, c.c_int64, c.c_int64, c.c_int64,
                                                 c.c_int, c.c_float, c.c_int64, c.c_int]
        L.wtc_oracle_fill_f32.argtypes = [c.c_void_p, c.c_int64, c.c_int, c.c_uint64]
        L.wtc_oracle_fill_f16.argtypes = [c.c_void_p, c.c_int64, c.c_int, c.c_uint64, c.c_int]
        L.wtc_oracle_f32_to_f16_rne.restype = c.c_uint16
        L.wtc_oracle_f32_to_f16_rne.argtypes = [c.c_float]
        L.wtc_oracle_f32_to_f16_profiler.restype = c.c_uint16
        L.wtc_oracle_f32_to_f16_profiler.argtypes = [c.c_float]
        L.wtc_oracle_max_threads.restype = c.c_int
        _LIB = L
    return _LIB


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def max_threads() -> int:
    return int(lib().wtc_oracle_max_threads())


# ---------------------------------------------------------------- inputs

def fill(shape, pattern: str, seed: int = 1, dtype=np.float32, f16_conv: str = "profiler") -> np.ndarray:
    """A dense row-major buffer filled the way the reference profiler fills it
    (`--init=zero|linear|random --seed=S`).  f16 buffers use the profiler's own
    f32->f16 conversion unless f16_conv == "rne"."""
    count = int(np.prod(shape))
    if np.dtype(dtype) == np.float32:
        out = np.empty(count, dtype=np.float32)
        lib().wtc_oracle_fill_f32(_ptr(out), count, MODES[pattern], seed)
    elif np.dtype(dtype) == np.float16:
        out = np.empty(count, dtype=np.uint16)
        lib().wtc_oracle_fill_f16(_ptr(out), count, MODES[pattern], seed, 1 if f16_conv == "rne" else 0)
        out = out.view(np.float16)
    else:
        raise TypeError(dtype)
    return out.reshape(shape)


def normal(shape, seed: int, sigma: float = 1.0, dtype=np.float16) -> np.ndarray:
    """Seeded N(0, sigma) stand-in for the benchmark configurations the reference
    has no generator for; PCG64 so the same seed gives the same bits everywhere."""
    g = np.random.Generator(np.random.PCG64(seed))
    x = g.standard_normal(size=shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x.astype(dtype)


# ---------------------------------------------------------------- the chain

def _dt(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return DT_F32
    if a.dtype == np.float16:
        return DT_F16
    raise TypeError(f"unsupported dtype {a.dtype}")


def chain(A: np.ndarray, B: np.ndarray, scale: float = 1.0, acc: int = ACC_F64,
          threads: int = 0, return_logits: bool = False):
    """softmax_row(scale * A @ B) in f64.  A is [M,K] or [batch,M,K]; B is [K,N]
    (shared by every batch) or [batch,K,N]."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    if A.dtype != B.dtype:
        raise TypeError("A and B must share a dtype")
    squeeze = A.ndim == 2
    A3 = A[None] if squeeze else A
    batch, M, K = A3.shape
    if B.ndim == 2:
        Kb, N = B.shape
        bstride = 0
    else:
        if B.shape[0] != batch:
            raise ValueError("batch mismatch")
        _, Kb, N = B.shape
        bstride = Kb * N
    if Kb != K:
        raise ValueError(f"K mismatch: A has {K}, B has {Kb}")
    probs = np.empty((batch, M, N), dtype=np.float64)
    logits = np.empty((batch, M, N), dtype=np.float64) if return_logits else None
    rc = lib().wtc_oracle_chain(_ptr(A3), _ptr(B), _ptr(probs),
                                _ptr(logits) if logits is not None else None,
                                batch, M, N, K, _dt(A), float(scale), acc, bstride, threads)
    if rc != 0:
        raise ValueError(f"wtc_oracle_chain rejected its arguments (rc={rc})")
    if squeeze:
        probs = probs[0]
        logits = logits[0] if logits is not None else None
    return (probs, logits) if return_logits else probs


def chain_loops_f32(A: np.ndarray, B: np.ndarray, scale: float = 1.0, threads: int = 0) -> np.ndarray:
    """The timed CPU baseline: the scalar loop nest a linalg->loops lowering gives
    (f32 accumulate, separate max/exp/sum/div passes), rows spread over threads."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    squeeze = A.ndim == 2
    A3 = A[None] if squeeze else A
    batch, M, K = A3.shape
    N = B.shape[-1]
    bstride = 0 if B.ndim == 2 else K * N
    out = np.empty((batch, M, N), dtype=np.float32)
    rc = lib().wtc_oracle_chain_loops_f32(_ptr(A3), _ptr(B), _ptr(out), batch, M, N, K,
                                          _dt(A), float(scale), bstride, threads)
    if rc != 0:
        raise ValueError(f"wtc_oracle_chain_loops_f32 rejected its arguments (rc={rc})")
    return out[0] if squeeze else out


# ---------------------------------------------------------------- comparison

def row_softmax(X: np.ndarray) -> np.ndarray:
    """Row softmax of a given matrix in float64, op for op as the row-only chain spells it
    (backend/welder/mlir_pipeline/softmax_row_chain.mlir:10-75: max from -3.4028235e38, exp(x - max),
    sum from 0, divide)."""
    x = np.asarray(X, dtype=np.float64)
    m = np.maximum(x.max(axis=-1, keepdims=True), -3.4028235e38)
    e = np.exp(x - m)
    return e / e.sum(axis=-1, keepdims=True)


def row_variance(A: np.ndarray, mean_factor: float | None = None, var_factor: float | None = None) -> np.ndarray:
    """The layernorm-style variance chain in float64 (backend/welder/mlir_pipeline/layernorm_variance_chain.mlir:12-104):
    sum -> mean = sum * c1 -> (a - mean)^2 -> sum -> var = sum * c2 -> broadcast along the row.
    c1 and c2 default to 1/N as in the reference input (0.00390625 for N = 256)."""
    a = np.asarray(A, dtype=np.float64)
    n = a.shape[-1]
    c1 = 1.0 / n if mean_factor is None else float(mean_factor)
    c2 = 1.0 / n if var_factor is None else float(var_factor)
    mean = a.sum(axis=-1, keepdims=True) * c1
    var = ((a - mean) ** 2).sum(axis=-1, keepdims=True) * c2
    return np.broadcast_to(var, a.shape).copy()


def compare(out: np.ndarray, ref_probs: np.ndarray, out_is_f16: bool | None = None) -> dict:
    """The parity contract: max |p - p_ref| <= 2e-3, |row sum - 1| <= 1e-3 and the
    same row argmax.  Near-ties: the kernel's argmax must lie in the set of
    columns whose oracle probability is within one output ulp of the oracle's
    row maximum (a different accumulation order may flip exact near-ties)."""
    o = np.asarray(out).astype(np.float64).reshape(-1, out.shape[-1])
    r = np.asarray(ref_probs, dtype=np.float64).reshape(-1, ref_probs.shape[-1])
    if o.shape != r.shape:
        raise ValueError(f"shape mismatch {o.shape} vs {r.shape}")
    if out_is_f16 is None:
        out_is_f16 = np.asarray(out).dtype == np.float16
    finite = bool(np.isfinite(o).all())
    if o.size == 0:
        return dict(ok=finite, finite=finite, max_abs=0.0, max_rowsum_err=0.0,
                    argmax_mismatch=0, argmax_ambiguous=0, rows=0)
    max_abs = float(np.abs(o - r).max())
    rowsum_err = float(np.abs(o.sum(axis=1) - 1.0).max())
    am_o = o.argmax(axis=1)
    am_r = r.argmax(axis=1)
    rmax = r.max(axis=1)
    if out_is_f16:
        ulp = np.maximum(np.spacing(rmax.astype(np.float16)).astype(np.float64), 2.0 ** -24)
    else:
        ulp = np.spacing(rmax.astype(np.float32)).astype(np.float64)
    differs = am_o != am_r
    picked = r[np.arange(r.shape[0]), am_o]
    within = picked >= rmax - ulp
    mismatch = int((differs & ~within).sum())
    ambiguous = int((differs & within).sum())
    ok = finite and max_abs <= TOL_PROB_ABS and rowsum_err <= TOL_ROWSUM and mismatch == 0
    return dict(ok=bool(ok), finite=finite, max_abs=max_abs, max_rowsum_err=rowsum_err,
                argmax_mismatch=mismatch, argmax_ambiguous=ambiguous, rows=int(o.shape[0]))


# ---------------------------------------------------------------- dump format

def write_dump(path: str, arr: np.ndarray, sym: str = "%out") -> None:
    """Raw bytes plus the `.json` side file the reference profiler writes for
    `--dump-last-2d` (solver/WelderProfilerRuntime.h:104-126): sym, rank,
    elem_bytes, offset, sizes, strides (in elements), bytes."""
    import json
    a = np.ascontiguousarray(arr)
    if a.ndim != 2:
        raise ValueError("rank-2 dumps only")
    a.tofile(path)
    meta = dict(sym=sym, rank=2, elem_bytes=int(a.itemsize), offset=0,
                sizes=[int(a.shape[0]), int(a.shape[1])], strides=[int(a.shape[1]), 1],
                bytes=int(a.nbytes))
    with open(path + ".json", "w") as f:
        json.dump(meta, f, indent=2)
