"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and resolves descriptors to the documented kernel plans.  No compute."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols(name):
    text = open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:wtc|welder)_[a-z0-9_]+)\s*\(", text)))


def test_launch_header_symbols_exported(wtc_lib):
    L = wtc_lib.lib()
    syms = header_symbols("wtc_launch.h")
    assert len(syms) >= 10
    for s in syms:
        assert hasattr(L, s), f"{s} declared in include/wtc_launch.h but not exported"
    assert sorted(wtc_lib.launch.EXPORTS) == [s for s in syms if s in wtc_lib.launch.EXPORTS]
    assert L.wtc_abi_version() == 2


def test_struct_layout_matches_header(wtc_lib):
    # the library checks struct_size; a mismatch between the ctypes mirror and the C struct shows here
    d = wtc_lib.make_desc(1, 8, 8, 8)
    wtc_lib.plan_query(d)
    d.struct_size += 4
    with pytest.raises(wtc_lib.WtcError) as e:
        wtc_lib.plan_query(d)
    assert e.value.code == -1 and "struct_size" in str(e.value)


@pytest.mark.parametrize("shape,kernel,cluster,launches,threads,stages", [
    ((1, 4096, 1024, 1024), "tc_cluster", 4, 1, 576, 4),      # f16 native chain: one tile per CTA, sixteen epilogue warps, staging over the operand stages (four stages)
    ((64, 2048, 2048, 128), "tc_cluster", 8, 1, 640, 2),      # batched attention scores: many tiles per CTA, relay epilogue (short K: two operand stages, two staging tiles)
    ((1, 8192, 32000, 4096), "tc_tiled", 1, 2, 320, 6),       # vocab-wide logits: online two-pass, CTA pairs
    ((1, 16, 32000, 4096), "tc_tiled", 1, 2, 320, 4),         # skinny decode
    ((1, 8192, 128, 64), "tc_cluster", 1, 1, 320, 4),         # the reference's own shape: rows of 128 columns take the 128-column tile
])
def test_plans_for_benchmark_configs(wtc_lib, shape, kernel, cluster, launches, threads, stages):
    p = wtc_lib.plan_query(wtc_lib.make_desc(*shape))
    assert wtc_lib.launch.KERNEL_NAMES[p.kernel] == kernel
    assert (p.cluster_n, p.launches) == (cluster, launches)
    tn = 128 if shape[2] <= 128 else 256
    assert (p.tile_m, p.tile_n, p.tile_k) == (128, tn, 64)
    assert p.tmem_columns == 2 * tn and (p.threads, p.stages) == (threads, stages)
    if kernel == "tc_tiled":
        b, M, N, K = shape
        assert p.workspace_bytes == b * M * ((N + 255) // 256) * 8
        assert wtc_lib.workspace_bytes(wtc_lib.make_desc(*shape)) == p.workspace_bytes


def test_plan_fallbacks_and_variants(wtc_lib):
    w = wtc_lib
    assert w.plan_query(w.make_desc(1, 128, 128, 128, w.F32, w.F32)).kernel == w.KERNEL_SIMT_FUSED
    assert w.plan_query(w.make_desc(1, 100, 70, 64)).kernel == w.KERNEL_SIMT_FUSED        # N % 8 != 0
    assert w.plan_query(w.make_desc(1, 100, 72, 60)).kernel == w.KERNEL_SIMT_FUSED        # K % 8 != 0
    assert w.plan_query(w.make_desc(1, 100, 72, 64, out_dtype=w.F32)).kernel == w.KERNEL_TC_CLUSTER   # f16 in, f32 out
    assert w.plan_query(w.make_desc(1, 100, 72, 64, out_dtype=w.F32, tile_n=128)).tile_n == 128       # f32 output has both column tiles too
    assert w.plan_query(w.make_desc(1, 100, 72, 64, tile_n=256)).tile_n == 256                        # a hint wins over the narrow-row default
    # without a hint: 128-column tiles when 256-column ones would leave most SMs idle and the narrower clusters all fit at once
    assert w.plan_query(w.make_desc(1, 100, 136, 64)).tile_n == 128
    assert w.plan_query(w.make_desc(1, 4096, 512, 1024)).tile_n == 128 and w.plan_query(w.make_desc(1, 4096, 512, 1024)).cluster_n == 4
    assert w.plan_query(w.make_desc(1, 2048, 1024, 1024)).tile_n == 256        # sixteen 8-CTA clusters would need two rounds
    assert w.plan_query(w.make_desc(1, 8192, 512, 128)).tile_n == 256          # 256-column tiles already fill the chip
    assert w.plan_query(w.make_desc(1, 256, 1024, 1024, flags=w.FLAG_FORCE_TILED)).tile_n == 256
    assert w.plan_query(w.make_desc(1, 100, 72, 64, flags=w.FLAG_FORCE_SIMT)).kernel == w.KERNEL_SIMT_FUSED
    assert w.plan_query(w.make_desc(1, 100, 512, 64, flags=w.FLAG_FORCE_TILED)).kernel == w.KERNEL_TC_TILED
    # the baseline variant: five kernels; f16 chains keep the tcgen05 contraction, f32 chains (and shapes TMA cannot take) run SIMT
    p = w.plan_query(w.make_desc(2, 100, 72, 64, variant=w.VARIANT_BASELINE))
    assert p.kernel == w.KERNEL_TC_UNFUSED and p.launches == 5 and p.tile_n == 128 and p.registers > 0
    assert p.workspace_bytes == (2 * 200 * 72 + 2 * 200) * 4
    for d in (w.make_desc(2, 100, 72, 64, w.F32, w.F32, variant=w.VARIANT_BASELINE), w.make_desc(2, 100, 70, 64, variant=w.VARIANT_BASELINE)):
        assert w.plan_query(d).kernel == w.KERNEL_SIMT_UNFUSED and w.plan_query(d).launches == 5
    # tile hints: legal ones pass, others are replaced and flagged
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=128, tile_n=256, tile_k=64)).tile_substituted == 0
    # the reference's own pinned search result, 64 x 128 x 32, is honoured as given
    p = w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=64, tile_n=128, tile_k=32))
    assert (p.tile_m, p.tile_n, p.tile_k, p.tile_substituted, p.cluster_n, p.stages) == (64, 128, 32, 0, 8, 8)
    # stage depths 32 / 128 and 64-row tiles belong to the eight-warp family: f16 probabilities, no forced form
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=128, tile_n=128, tile_k=128)).tile_substituted == 0
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=128, tile_n=256, tile_k=128)).tile_k == 64     # no room beside a cluster's statistics
    assert w.plan_query(w.make_desc(1, 4096, 4096, 1024, tile_m=128, tile_n=256, tile_k=128)).tile_k == 128    # tiled flavour
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=64, tile_n=128, tile_k=128)).tile_m == 128
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=32, tile_n=64, tile_k=16)).tile_substituted == 1
    assert w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=64, tile_k=32, flags=w.FLAG_EPILOGUE_RELAY)).tile_m == 128
    # the second legal column tile is honoured as given: 128 columns per CTA, eight CTAs per cluster
    p = w.plan_query(w.make_desc(1, 4096, 1024, 1024, tile_m=128, tile_n=128, tile_k=64))
    assert (p.tile_n, p.cluster_n, p.tile_substituted, p.tmem_columns) == (128, 8, 0, 256)
    assert w.plan_query(w.make_desc(1, 4096, 2048, 1024, tile_n=128)).kernel == w.KERNEL_TC_TILED   # 16 column blocks


def test_plan_for_f32_operands_rounded_to_f16(wtc_lib):
    """WTC_FLAG_MATMUL_F16: the plan is the f16 chain's plus one launch that rounds both operands, and the
    workspace holds the rounded copies (each padded to 256 bytes) ahead of the chain's own."""
    w = wtc_lib
    p = w.plan_query(w.make_desc(1, 8192, 128, 64, in_dtype=w.F32, out_dtype=w.F32, acc_dtype=w.F16, flags=w.FLAG_MATMUL_F16))
    assert (p.kernel, p.launches, p.workspace_bytes) == (w.KERNEL_TC_CLUSTER, 2, 8192 * 64 * 2 + 64 * 128 * 2)
    d = w.make_desc(2, 100, 32000, 64, in_dtype=w.F32, flags=w.FLAG_MATMUL_F16)          # tiled schedule behind the rounding, B per batch
    p = w.plan_query(d)
    stage = -(-2 * 100 * 64 * 2 // 256) * 256 + -(-2 * 64 * 32000 * 2 // 256) * 256
    assert p.kernel == w.KERNEL_TC_TILED and p.launches == 3 and p.workspace_bytes == stage + 2 * 100 * 125 * 8
    assert w.workspace_bytes(d) == p.workspace_bytes
    p = w.plan_query(w.make_desc(1, 33, 100, 50, in_dtype=w.F32, out_dtype=w.F32, flags=w.FLAG_MATMUL_F16))
    assert p.kernel == w.KERNEL_SIMT_FUSED and p.launches == 2
    with pytest.raises(w.WtcError) as e:                                                   # the flag needs f32 buffers
        w.plan_query(w.make_desc(1, 16, 16, 16, in_dtype=w.F16, flags=w.FLAG_MATMUL_F16))
    assert e.value.code == -1


@pytest.mark.parametrize("kw", [dict(batch=0), dict(M=-1), dict(in_dtype=7), dict(variant=3), dict(tile_m=-2),
                                dict(lda=3)])
def test_bad_descriptors_rejected(wtc_lib, kw):
    args = dict(batch=1, M=16, N=16, K=16)
    args.update(kw)
    with pytest.raises(wtc_lib.WtcError) as e:
        wtc_lib.plan_query(wtc_lib.make_desc(**args))
    assert e.value.code == -1


def test_no_cpu_fallback(wtc_lib):
    """Without a device a launch must fail loudly, never compute on the host."""
    import numpy as np
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(wtc_lib.WtcError) as e:
        wtc_lib.matmul_softmax_host(np.zeros((4, 8), np.float32), np.zeros((8, 8), np.float32))
    assert e.value.code == -4
    with pytest.raises(wtc_lib.WtcError):
        wtc_lib.matmul_softmax(torch.zeros(4, 8), torch.zeros(8, 8))


def test_host_call_tickets_without_a_device(wtc_lib):
    """The ticket rules of the two-halved host-buffer call need no device: an empty chain is complete at
    once (ticket -1), waiting for a ticket nobody issued is an argument error, and without a device a
    submit fails loudly like every other launch."""
    import ctypes as C
    import numpy as np
    import torch
    L = wtc_lib.lib()
    L.wtc_matmul_softmax_host_submit.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    L.wtc_matmul_softmax_host_wait.argtypes = [C.c_int64]
    t = C.c_int64(123)
    empty = wtc_lib.make_desc(1, 0, 64, 64)
    assert L.wtc_matmul_softmax_host_submit(C.byref(empty), None, None, None, C.byref(t)) == 0 and t.value == -1
    assert L.wtc_matmul_softmax_host_wait(-1) == 0
    assert L.wtc_matmul_softmax_host_submit(C.byref(empty), None, None, None, None) == -1
    assert L.wtc_matmul_softmax_host_wait(1 << 40) == -1 and b"not issued" in L.wtc_last_error()
    if not torch.cuda.is_available():
        a = np.zeros((128, 64), np.float16)
        d = wtc_lib.make_desc(1, 128, 64, 64)
        assert L.wtc_matmul_softmax_host_submit(C.byref(d), a.ctypes.data, a.ctypes.data, a.ctypes.data, C.byref(t)) == -4
        assert t.value == -1
