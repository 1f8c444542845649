"""ctypes binding of the C-ABI launch layer (include/wtc_launch.h).

Mirrors what a host-side caller of the reference does around `welder-profiler`
(backend/welder/compiler/solver/WelderProfiler.cpp:601-677 copy-in, :752-793 launch
loop, :808-864 dump): describe the chain, hand over device buffers, launch, read
back.  torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16 = 0, 1
VARIANT_FUSED, VARIANT_BASELINE = 0, 1
FLAG_FORCE_SIMT, FLAG_FORCE_TILED, FLAG_MATMUL_F16 = 0x1, 0x2, 0x4
FLAG_EPILOGUE_SPLIT, FLAG_EPILOGUE_RELAY, FLAG_NO_PAIR, FLAG_PAIR = 0x8, 0x10, 0x20, 0x40
FLAG_OPERANDS_READY = 0x80   # A and B do not depend on earlier work on the stream: only the stores wait for it
KERNEL_SIMT_FUSED, KERNEL_TC_CLUSTER, KERNEL_TC_TILED, KERNEL_SIMT_UNFUSED, KERNEL_TC_UNFUSED = 0, 1, 2, 3, 4
KERNEL_NAMES = {0: "simt_fused", 1: "tc_cluster", 2: "tc_tiled", 3: "simt_unfused", 4: "tc_unfused"}

EXPORTS = [
    "wtc_abi_version", "wtc_last_error", "wtc_plan_query", "wtc_matmul_softmax_workspace_bytes",
    "wtc_matmul_softmax_launch", "wtc_matmul_softmax_partial_launch", "wtc_matmul_softmax_finish_launch",
    "wtc_matmul_softmax_host", "wtc_matmul_softmax_host_submit", "wtc_matmul_softmax_host_wait",
    "wtc_check_device_status", "wtc_matmul_softmax_time",
    "wtc_matmul_softmax_launch_static", "wtc_row_chain_launch", "wtc_row_chain_time",
]


class WtcError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"wtc error {code}: {msg}")
        self.code = code


class ChainDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("batch", C.c_int32),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldo", C.c_int64),
        ("a_batch_stride", C.c_int64), ("b_batch_stride", C.c_int64), ("o_batch_stride", C.c_int64),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("acc_dtype", C.c_int32),
        ("scale", C.c_float),
        ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
        ("variant", C.c_int32), ("flags", C.c_int32),
    ]


class RowChainDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("kind", C.c_int32), ("rows", C.c_int64), ("N", C.c_int64),
        ("ld_in", C.c_int64), ("ld_out", C.c_int64), ("dtype", C.c_int32),
        ("mean_factor", C.c_float), ("var_factor", C.c_float), ("reserved", C.c_int32),
    ]


ROW_SOFTMAX, ROW_VARIANCE = 0, 1


class PlanInfo(C.Structure):
    _fields_ = [
        ("kernel", C.c_int32), ("launches", C.c_int32),
        ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
        ("cluster_n", C.c_int32), ("grid", C.c_int32), ("threads", C.c_int32), ("smem_bytes", C.c_int32),
        ("tmem_columns", C.c_int32), ("stages", C.c_int32), ("tile_substituted", C.c_int32),
        ("workspace_bytes", C.c_size_t),
        ("registers", C.c_int32), ("spill_bytes", C.c_int32), ("stack_bytes", C.c_int32), ("reserved", C.c_int32),
    ]


def lib_path() -> str:
    return os.path.join(_HERE, "libwtc_launch.so")


def lib() -> C.CDLL:
    """The launch library.  Raises if it has not been built: there is no fallback."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
                              "(or __graft_entry__.build()); this package has no CPU or PyTorch fallback")
        L = C.CDLL(path)
        L.wtc_last_error.restype = C.c_char_p
        vp, sz = C.c_void_p, C.c_size_t
        dp = C.POINTER(ChainDesc)
        L.wtc_plan_query.argtypes = [dp, C.POINTER(PlanInfo)]
        L.wtc_matmul_softmax_workspace_bytes.argtypes = [dp, C.POINTER(sz)]
        L.wtc_matmul_softmax_launch.argtypes = [dp, vp, vp, vp, vp, sz, vp, vp]
        L.wtc_matmul_softmax_partial_launch.argtypes = [dp, vp, vp, vp, vp, sz, vp, vp, vp]
        L.wtc_matmul_softmax_finish_launch.argtypes = [dp, vp, vp, vp, C.c_int32, vp]
        L.wtc_matmul_softmax_host.argtypes = [dp, vp, vp, vp]
        L.wtc_check_device_status.argtypes = [vp, vp]
        L.wtc_matmul_softmax_time.argtypes = [dp, vp, vp, vp, vp, sz, vp, C.c_int, C.c_int, C.POINTER(C.c_float)]
        L.wtc_matmul_softmax_launch_static.argtypes = [dp, vp, vp, vp, vp, vp]
        L.wtc_row_chain_launch.argtypes = [C.POINTER(RowChainDesc), vp, vp, vp]
        L.wtc_row_chain_time.argtypes = [C.POINTER(RowChainDesc), vp, vp, vp, C.c_int, C.c_int, C.POINTER(C.c_float)]
        _LIB = L
    return _LIB


def _check(rc: int) -> None:
    if rc != 0:
        raise WtcError(rc, lib().wtc_last_error().decode(errors="replace"))


def make_desc(batch: int, M: int, N: int, K: int, in_dtype: int = F16, out_dtype: int = F16,
              acc_dtype: int = F32, scale: float = 1.0, shared_b: bool = False, variant: int = VARIANT_FUSED,
              flags: int = 0, tile_m: int = 0, tile_n: int = 0, tile_k: int = 0,
              lda: int = 0, ldb: int = 0, ldo: int = 0) -> ChainDesc:
    d = ChainDesc()
    d.struct_size = C.sizeof(ChainDesc)
    d.batch, d.M, d.N, d.K = batch, M, N, K
    d.lda, d.ldb, d.ldo = lda, ldb, ldo
    d.a_batch_stride = 0
    d.b_batch_stride = -1 if shared_b else 0
    d.o_batch_stride = 0
    d.in_dtype, d.out_dtype, d.acc_dtype = in_dtype, out_dtype, acc_dtype
    d.scale = scale
    d.tile_m, d.tile_n, d.tile_k = tile_m, tile_n, tile_k
    d.variant, d.flags = variant, flags
    return d


def plan_query(desc: ChainDesc) -> PlanInfo:
    p = PlanInfo()
    _check(lib().wtc_plan_query(C.byref(desc), C.byref(p)))
    return p


def workspace_bytes(desc: ChainDesc) -> int:
    n = C.c_size_t(0)
    _check(lib().wtc_matmul_softmax_workspace_bytes(C.byref(desc), C.byref(n)))
    return int(n.value)


# ------------------------------------------------------------------ torch side

def _torch():
    import torch
    return torch


def _dt(t) -> int:
    torch = _torch()
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise TypeError(f"unsupported dtype {t.dtype}")


def _desc_for(A, B, out_dtype, scale, acc_dtype, variant, flags, tiles) -> ChainDesc:
    if A.dim() not in (2, 3) or B.dim() not in (2, 3):
        raise ValueError("A must be [M,K] or [batch,M,K]; B must be [K,N] or [batch,K,N]")
    if not (A.is_contiguous() and B.is_contiguous()):
        raise ValueError("operands must be contiguous (row-major)")
    if A.dtype != B.dtype:
        raise TypeError("A and B must share a dtype")
    batch = A.shape[0] if A.dim() == 3 else 1
    M, K = A.shape[-2], A.shape[-1]
    if B.shape[-2] != K:
        raise ValueError(f"K mismatch: A has {K}, B has {B.shape[-2]}")
    N = B.shape[-1]
    shared_b = B.dim() == 2 and batch > 1
    if B.dim() == 3 and B.shape[0] != batch:
        raise ValueError("batch mismatch")
    tm, tn, tk = tiles or (0, 0, 0)
    return make_desc(batch, M, N, K, _dt(A), out_dtype, acc_dtype, scale, shared_b, variant, flags, tm, tn, tk)


def _stream_ptr():
    torch = _torch()
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def matmul_softmax(A, B, scale: float = 1.0, out=None, out_dtype=None, acc_dtype: int = F32,
                   variant: int = VARIANT_FUSED, flags: int = 0, tiles=None, workspace=None, status=None):
    """softmax_row(scale * A @ B) on the current CUDA device and stream.
    A: [M,K] or [batch,M,K]; B: [K,N] (shared by every batch) or [batch,K,N]."""
    torch = _torch()
    if not A.is_cuda:
        raise WtcError(-4, "operands must be CUDA tensors: this library has no CPU path")
    if out_dtype is None:
        out_dtype = _dt(A)
    d = _desc_for(A, B, out_dtype, scale, acc_dtype, variant, flags, tiles)
    shape = (*A.shape[:-1], B.shape[-1])
    if out is None:
        out = torch.empty(shape, device=A.device, dtype=torch.float16 if out_dtype == F16 else torch.float32)
    elif tuple(out.shape) != tuple(shape) or not out.is_contiguous():
        raise ValueError("out has the wrong shape or is not contiguous")
    need = workspace_bytes(d)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=A.device, dtype=torch.uint8)
    ws_ptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
    st_ptr = C.c_void_p(status.data_ptr()) if status is not None else None
    with torch.cuda.device(A.device):
        _check(lib().wtc_matmul_softmax_launch(C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                               C.c_void_p(out.data_ptr()), ws_ptr, ws_len, _stream_ptr(), st_ptr))
    return out


def matmul_softmax_partial(A, B, scale: float, out, workspace, row_stats, acc_dtype: int = F32):
    """One N-shard: un-normalised exp values into `out`, per-row (max, sum) into
    row_stats[rows, 2] (f32)."""
    torch = _torch()
    d = _desc_for(A, B, F16, scale, acc_dtype, VARIANT_FUSED, 0, None)
    with torch.cuda.device(A.device):
        _check(lib().wtc_matmul_softmax_partial_launch(
            C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_void_p(workspace.data_ptr()), workspace.numel() * workspace.element_size(),
            C.c_void_p(row_stats.data_ptr()), _stream_ptr(), None))
    return d


def matmul_softmax_finish(desc: ChainDesc, out, workspace, all_stats, num_parts: int):
    torch = _torch()
    with torch.cuda.device(out.device):
        _check(lib().wtc_matmul_softmax_finish_launch(C.byref(desc), C.c_void_p(out.data_ptr()),
                                                      C.c_void_p(workspace.data_ptr()),
                                                      C.c_void_p(all_stats.data_ptr()), num_parts, _stream_ptr()))


class PreparedCall:
    """One chain call with every argument converted once: launch() is a single
    foreign call, for loops where Python overhead would otherwise outweigh a
    10-microsecond kernel."""

    def __init__(self, A, B, out, scale: float = 1.0, workspace=None, acc_dtype: int = F32,
                 variant: int = VARIANT_FUSED, flags: int = 0):
        torch = _torch()
        self.desc = _desc_for(A, B, _dt(out), scale, acc_dtype, variant, flags, None)
        need = workspace_bytes(self.desc)
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, device=A.device, dtype=torch.uint8)
        self._keep = (A, B, out, workspace)
        self._fn = lib().wtc_matmul_softmax_launch
        self._args = (C.byref(self.desc), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                      C.c_void_p(out.data_ptr()),
                      C.c_void_p(workspace.data_ptr()) if workspace is not None else None,
                      workspace.numel() * workspace.element_size() if workspace is not None else 0)
        self.out = out

    def launch(self, stream_ptr) -> None:
        rc = self._fn(*self._args, stream_ptr, None)
        if rc != 0:
            _check(rc)


class PreparedShardCall:
    """One column shard of the chain with every argument converted once: partial(stream)
    leaves exp values in `out` and the shard's per-row (max, sum) in `row_stats`;
    finish(stream) normalises `out` against the gathered pairs of all shards."""

    def __init__(self, A, B, out, scale, workspace, row_stats, all_stats, num_parts, acc_dtype: int = F32):
        self.desc = _desc_for(A, B, F16, scale, acc_dtype, VARIANT_FUSED, 0, None)
        self._keep = (A, B, out, workspace, row_stats, all_stats)
        L = lib()
        self._partial, self._finish = L.wtc_matmul_softmax_partial_launch, L.wtc_matmul_softmax_finish_launch
        ws_len = workspace.numel() * workspace.element_size()
        self._pargs = (C.byref(self.desc), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(out.data_ptr()),
                       C.c_void_p(workspace.data_ptr()), ws_len, C.c_void_p(row_stats.data_ptr()))
        self._fargs = (C.byref(self.desc), C.c_void_p(out.data_ptr()), C.c_void_p(workspace.data_ptr()),
                       C.c_void_p(all_stats.data_ptr()), num_parts)

    def partial(self, stream_ptr) -> None:
        rc = self._partial(*self._pargs, stream_ptr, None)
        if rc != 0:
            _check(rc)

    def finish(self, stream_ptr) -> None:
        rc = self._finish(*self._fargs, stream_ptr)
        if rc != 0:
            _check(rc)


def current_stream_ptr():
    return _stream_ptr()


def matmul_softmax_static(A, B, scale: float, out, status=None, acc_dtype: int = F32):
    """The entry point that allocates nothing: scratch lives in the library image."""
    torch = _torch()
    d = _desc_for(A, B, _dt(out), scale, acc_dtype, VARIANT_FUSED, 0, None)
    with torch.cuda.device(A.device):
        _check(lib().wtc_matmul_softmax_launch_static(
            C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(out.data_ptr()),
            _stream_ptr(), C.c_void_p(status.data_ptr()) if status is not None else None))
    return out


def _row_chain(kind, X, out, mean_factor, var_factor):
    torch = _torch()
    if not X.is_cuda:
        raise WtcError(-4, "operands must be CUDA tensors: this library has no CPU path")
    if X.dim() < 2 or not X.is_contiguous():
        raise ValueError("X must be a contiguous matrix (or a stack of matrices)")
    N = X.shape[-1]
    rows = X.numel() // N if N else 0
    if out is None:
        out = torch.empty_like(X)
    elif tuple(out.shape) != tuple(X.shape) or out.dtype != X.dtype or not out.is_contiguous():
        raise ValueError("out must match X in shape and dtype and be contiguous")
    d = RowChainDesc()
    d.struct_size = C.sizeof(RowChainDesc)
    d.kind, d.rows, d.N, d.ld_in, d.ld_out = kind, rows, N, 0, 0
    d.dtype = _dt(X)
    d.mean_factor, d.var_factor = mean_factor, var_factor
    with torch.cuda.device(X.device):
        _check(lib().wtc_row_chain_launch(C.byref(d), C.c_void_p(X.data_ptr()), C.c_void_p(out.data_ptr()), _stream_ptr()))
    return out


def row_softmax(X, out=None):
    """softmax over the last dimension of X (f32 or f16), one fused kernel: the row-only chain
    max -> exp(x - max) -> sum -> divide."""
    return _row_chain(ROW_SOFTMAX, X, out, 0.0, 0.0)


def row_variance(X, mean_factor=None, var_factor=None, out=None):
    """out[i, :] = var_factor * sum_j (X[i,j] - mean_factor * sum_j X[i,j])^2 (both factors default
    to 1/N: the biased row variance, broadcast along the row)."""
    n = X.shape[-1]
    return _row_chain(ROW_VARIANCE, X, out, 1.0 / n if mean_factor is None else mean_factor, 1.0 / n if var_factor is None else var_factor)


def check_device_status(status=None) -> None:
    ptr = C.c_void_p(status.data_ptr()) if status is not None else None
    _check(lib().wtc_check_device_status(ptr, _stream_ptr()))


def time_launch(A, B, out, scale: float = 1.0, warmup: int = 10, iters: int = 200, acc_dtype: int = F32,
                variant: int = VARIANT_FUSED, flags: int = 0, workspace=None) -> float:
    """avg ms per call: `warmup` launches, then `iters` launches between two CUDA
    events on the current stream (the reference profiler's method)."""
    torch = _torch()
    d = _desc_for(A, B, _dt(out), scale, acc_dtype, variant, flags, None)
    need = workspace_bytes(d)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=A.device, dtype=torch.uint8)
    ms = C.c_float(0)
    with torch.cuda.device(A.device):
        _check(lib().wtc_matmul_softmax_time(
            C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_void_p(workspace.data_ptr()) if workspace is not None else None,
            workspace.numel() * workspace.element_size() if workspace is not None else 0,
            _stream_ptr(), warmup, iters, C.byref(ms)))
    return float(ms.value)


# ------------------------------------------------------------------ host buffers

class HostChain:
    """A chain of fixed shape called again and again with HOST arrays (numpy; pinned memory makes the
    copies asynchronous).  submit() enqueues copy in, kernels and copy back and returns a ticket; wait()
    blocks until that call's result is in `out`.  Keep two calls in flight (submit i+1, then wait i) and
    both directions of the link stay busy; the arrays of a call must stay alive, and `out` unread,
    until its wait returns."""

    def __init__(self, batch, M, N, K, scale: float = 1.0, in_dtype: int = F16, out_dtype: int = F16, acc_dtype: int = F32,
                 shared_b: bool = False, variant: int = VARIANT_FUSED, flags: int = 0):
        self.desc = make_desc(batch, M, N, K, in_dtype, out_dtype, acc_dtype, scale, shared_b, variant, flags)
        self._lib = lib()
        self._lib.wtc_matmul_softmax_host_submit.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
        self._lib.wtc_matmul_softmax_host_wait.argtypes = [C.c_int64]
        self._ref = C.byref(self.desc)

    def submit(self, A, B, out) -> int:
        t = C.c_int64(-1)
        _check(self._lib.wtc_matmul_softmax_host_submit(self._ref, A.ctypes.data, B.ctypes.data, out.ctypes.data, C.byref(t)))
        return int(t.value)

    def wait(self, ticket: int) -> None:
        _check(self._lib.wtc_matmul_softmax_host_wait(ticket))


def matmul_softmax_host(A, B, scale: float = 1.0, out=None, out_dtype=None, acc_dtype: int = F32,
                        variant: int = VARIANT_FUSED, flags: int = 0):
    """Same chain with numpy HOST arrays: copy in, launch, copy out, synchronise."""
    import numpy as np
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    if A.dtype != B.dtype:
        raise TypeError("A and B must share a dtype")
    in_dt = {np.dtype(np.float16): F16, np.dtype(np.float32): F32}.get(A.dtype)
    if in_dt is None:
        raise TypeError(f"unsupported dtype {A.dtype}")
    if out_dtype is None:
        out_dtype = in_dt
    batch = A.shape[0] if A.ndim == 3 else 1
    M, K = A.shape[-2], A.shape[-1]
    if B.shape[-2] != K:
        raise ValueError(f"K mismatch: A has {K}, B has {B.shape[-2]}")
    N = B.shape[-1]
    d = make_desc(batch, M, N, K, in_dt, out_dtype, acc_dtype, scale, B.ndim == 2 and batch > 1, variant, flags)
    if out is None:
        out = np.empty((*A.shape[:-1], N), dtype=np.float16 if out_dtype == F16 else np.float32)
    _check(lib().wtc_matmul_softmax_host(C.byref(d), C.c_void_p(A.ctypes.data), C.c_void_p(B.ctypes.data),
                                         C.c_void_p(out.ctypes.data)))
    return out
