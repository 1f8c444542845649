"""B200-native fused Matmul -> row-Softmax chain behind the reference's operator surface.

The compute lives in libwtc_launch.so (hand-written sm_100a CUDA, C ABI declared in
include/wtc_launch.h); this package is the Python host-side binding used by the
tests, the benchmark and the verification harness.  There is no CPU fallback.
"""
from .launch import (  # noqa: F401
    ChainDesc, PlanInfo, WtcError, lib, make_desc, plan_query, workspace_bytes,
    matmul_softmax, matmul_softmax_host, HostChain, matmul_softmax_partial, matmul_softmax_finish,
    time_launch, check_device_status, row_softmax, row_variance, RowChainDesc, ROW_SOFTMAX, ROW_VARIANCE, PreparedCall, PreparedShardCall, current_stream_ptr, matmul_softmax_static,
    F32, F16, VARIANT_FUSED, VARIANT_BASELINE, FLAG_FORCE_SIMT, FLAG_FORCE_TILED, FLAG_MATMUL_F16,
    FLAG_EPILOGUE_SPLIT, FLAG_EPILOGUE_RELAY, FLAG_NO_PAIR, FLAG_PAIR, FLAG_OPERANDS_READY,
    KERNEL_SIMT_FUSED, KERNEL_TC_CLUSTER, KERNEL_TC_TILED, KERNEL_SIMT_UNFUSED, KERNEL_TC_UNFUSED,
)

__all__ = [n for n in dir() if not n.startswith("_")]
