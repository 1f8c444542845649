"""The entry point for callers that cannot allocate device memory.

Some hosts of the library -- a server whose own pool owns all of HBM, a loop that
cannot afford the device-wide stall an allocation causes -- still need the chain.
wtc_matmul_softmax_launch_static keeps its scratch in an array inside the library
image instead of asking for a workspace.  This file checks, through the C ABI,
that it gives what the ordinary entry point gives on the same schedule and what
the CPU checker gives, on calls in a row with different shapes (each call finds
the previous call's leftovers in the shared array), that a warm call leaves the
device's free memory untouched, and that it refuses shapes whose scratch would
not fit.  It is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


def _pair_of_calls(w, dev, A, B, scale):
    """The same chain through the workspace entry point (forced onto the two-pass schedule) and
    through the static-scratch entry point; returns (reference output, static output)."""
    import torch
    L = w.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    batch = A.shape[0] if A.dim() == 3 else 1
    M, K, N = A.shape[-2], A.shape[-1], B.shape[-1]
    shared_b = B.dim() == 2 and batch > 1
    d = w.make_desc(batch, M, N, K, scale=scale, shared_b=shared_b, flags=w.FLAG_FORCE_TILED)
    ws = torch.empty(w.workspace_bytes(d), device=dev, dtype=torch.uint8)
    shape = (*A.shape[:-1], N)
    ref = torch.empty(shape, device=dev, dtype=torch.float16)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = L.wtc_matmul_softmax_launch(C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                     C.c_void_p(ref.data_ptr()), C.c_void_p(ws.data_ptr()), ws.numel(), stream,
                                     C.c_void_p(st.data_ptr()))
    assert rc == 0, L.wtc_last_error()
    out = torch.full(shape, float("nan"), device=dev, dtype=torch.float16)
    st2 = torch.zeros(1, dtype=torch.int32, device=dev)
    d2 = w.make_desc(batch, M, N, K, scale=scale, shared_b=shared_b)   # no flag: the entry point picks the schedule itself
    rc = L.wtc_matmul_softmax_launch_static(C.byref(d2), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                            C.c_void_p(out.data_ptr()), stream, C.c_void_p(st2.data_ptr()))
    assert rc == 0, L.wtc_last_error()
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and int(st2.item()) == 0
    return ref, out


def test_static_scratch_matches_workspace_entry_point_and_checker(wtc_lib, cuda_dev):
    import torch
    w = wtc_lib
    # a many-tile shape; a smaller one whose tiles land on stale pairs; a long K (the CTA-pair
    # schedule: two row blocks, K >= 512); a batched call with its own B per batch
    cases = [((700, 192), (192, 2304), 0.07), ((130, 72), (72, 520), 0.2), ((300, 576), (576, 768), 0.05),
             ((3, 200, 64), (3, 64, 520), 0.125)]
    for i, (sa, sb, scale) in enumerate(cases):
        A = oracle.normal(sa, 40 + i)
        B = oracle.normal(sb, 50 + i)
        tA, tB = torch.from_numpy(A).to(cuda_dev), torch.from_numpy(B).to(cuda_dev)
        ref, out = _pair_of_calls(w, cuda_dev, tA, tB, scale)
        # same kernels on the same schedule: within the parity tolerance, and in fact equal
        assert float((out.float() - ref.float()).abs().max()) <= 2e-3
        assert torch.equal(out, ref)
        # and against the CPU checker: max abs error 2e-3, row sums within 1e-3, same argmax
        got = out.cpu().numpy()
        want = np.stack([oracle.chain(A[b], B[b], scale) for b in range(A.shape[0])]) if A.ndim == 3 else oracle.chain(A, B, scale)
        res = oracle.compare(got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1]))
        assert res["ok"], res
        # with no status pointer the call still runs, and its status word (a word of the library
        # image, shared with the other entry points) can be read back without any allocation
        out3 = torch.empty_like(out)
        w.matmul_softmax_static(tA, tB, scale, out3)
        w.check_device_status()
        assert torch.equal(out3, ref)


def test_static_scratch_warm_call_allocates_nothing(wtc_lib, cuda_dev):
    import torch
    w = wtc_lib
    A = torch.from_numpy(oracle.normal((260, 128), 7)).to(cuda_dev)
    B = torch.from_numpy(oracle.normal((128, 1032), 8)).to(cuda_dev)
    out = torch.empty((260, 1032), device=cuda_dev, dtype=torch.float16)
    w.matmul_softmax_static(A, B, 0.1, out)      # first call on the device: module load, address look-up
    w.check_device_status()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(cuda_dev)
    for _ in range(3):
        w.matmul_softmax_static(A, B, 0.1, out)
    w.check_device_status()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(cuda_dev)
    assert free1 == free0, f"free device memory changed across warm calls: {free0} -> {free1}"
    ref = oracle.chain(A.cpu().numpy(), B.cpu().numpy(), 0.1)
    assert oracle.compare(out.cpu().numpy(), ref)["ok"]


def test_static_scratch_rejects_what_does_not_fit(wtc_lib, cuda_dev):
    w = wtc_lib
    L = w.lib()
    one = C.c_void_p(256)   # never dereferenced: the checks come first
    big = w.make_desc(1, 65536, 32000, 64)                   # 65536 * 125 * 8 bytes = 62.5 MiB of pairs
    assert L.wtc_matmul_softmax_launch_static(C.byref(big), one, one, one, None, None) == -3
    msg = L.wtc_last_error().decode()
    assert "65536000" in msg and str(16 << 20) in msg
    f32 = w.make_desc(1, 64, 64, 64, w.F32, w.F32)
    assert L.wtc_matmul_softmax_launch_static(C.byref(f32), one, one, one, None, None) == -2
    odd = C.c_void_p(264)                                    # 8-byte aligned only: the tensor-core path needs 16
    ok = w.make_desc(1, 64, 64, 64)
    assert L.wtc_matmul_softmax_launch_static(C.byref(ok), odd, one, one, None, None) == -2
    empty = w.make_desc(1, 0, 64, 64)                        # nothing to compute: accepted like everywhere else
    assert L.wtc_matmul_softmax_launch_static(C.byref(empty), one, one, one, None, None) == 0
