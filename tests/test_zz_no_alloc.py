"""The entry point for callers that cannot allocate device memory.

Some hosts of the library -- a server whose own pool owns all of HBM, a loop that
cannot afford the device-wide stall an allocation causes -- still need the chain.
wtc_matmul_softmax_launch_static keeps its scratch in an array inside the library
image instead of asking for a workspace.  This file checks, through the C ABI,
that it gives what the ordinary entry point gives on the same schedule, twice in
a row with different shapes (the second call finds the first call's leftovers in
the shared array), and that it refuses shapes whose scratch would not fit.
It is named to be collected last.
"""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_point(wtc_lib, cuda_dev):
    import torch
    w = wtc_lib
    L = w.lib()
    g = torch.Generator(device=cuda_dev)
    g.manual_seed(99)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # first a many-tile shape, then a smaller one whose tiles land on stale pairs
    for (M, N, K, scale) in [(700, 2304, 192, 0.07), (130, 520, 72, 0.2)]:
        A = torch.randn((M, K), device=cuda_dev, generator=g).half()
        B = torch.randn((K, N), device=cuda_dev, generator=g).half()
        d = w.make_desc(1, M, N, K, scale=scale, flags=w.FLAG_FORCE_TILED)
        ws = torch.empty(w.workspace_bytes(d), device=cuda_dev, dtype=torch.uint8)
        ref = torch.empty((M, N), device=cuda_dev, dtype=torch.float16)
        st = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
        rc = L.wtc_matmul_softmax_launch(C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                         C.c_void_p(ref.data_ptr()), C.c_void_p(ws.data_ptr()), ws.numel(), stream,
                                         C.c_void_p(st.data_ptr()))
        assert rc == 0, L.wtc_last_error()
        out = torch.full((M, N), float("nan"), device=cuda_dev, dtype=torch.float16)
        st2 = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
        d2 = w.make_desc(1, M, N, K, scale=scale)            # no flag: the entry point picks the schedule itself
        rc = L.wtc_matmul_softmax_launch_static(C.byref(d2), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                                C.c_void_p(out.data_ptr()), stream, C.c_void_p(st2.data_ptr()))
        assert rc == 0, L.wtc_last_error()
        torch.cuda.synchronize()
        assert int(st.item()) == 0 and int(st2.item()) == 0
        # same kernels on the same schedule: within the parity tolerance, and in fact equal
        assert float((out.float() - ref.float()).abs().max()) <= 2e-3
        assert torch.equal(out, ref)
        assert float((out.float().sum(-1) - 1).abs().max()) <= 1e-3
        # with no status pointer the call still runs (its word lives in the static array)
        out3 = torch.empty_like(out)
        w.matmul_softmax_static(A, B, scale, out3)
        torch.cuda.synchronize()
        assert torch.equal(out3, ref)


def test_static_scratch_rejects_what_does_not_fit(wtc_lib, cuda_dev):
    w = wtc_lib
    L = w.lib()
    one = C.c_void_p(256)   # never dereferenced: the size check comes first
    big = w.make_desc(1, 65536, 32000, 64)                   # 65536 * 125 * 8 bytes = 62.5 MiB of pairs
    assert L.wtc_matmul_softmax_launch_static(C.byref(big), one, one, one, None, None) == -3
    msg = L.wtc_last_error().decode()
    assert "65536000" in msg and str((16 << 20) - 256) in msg
    f32 = w.make_desc(1, 64, 64, 64, w.F32, w.F32)
    assert L.wtc_matmul_softmax_launch_static(C.byref(f32), one, one, one, None, None) == -2
