"""Parity of the CUDA path (through the C ABI) against the CPU checker.

Tolerances are the contract's: max |p - p_ref| <= 2e-3, |row sum - 1| <= 1e-3,
identical row argmax (an argmax may differ only between columns whose checker
probabilities are within one output ulp of each other)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def w(wtc_lib, cuda_dev):
    return wtc_lib


def _run(w, dev, A, B, scale, **kw):
    import torch
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    out = w.matmul_softmax(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev), scale, status=st, **kw)
    torch.cuda.synchronize()
    assert int(st.item()) == 0, f"device status {int(st.item())}"
    return out.cpu().numpy()


def _check(out, ref):
    r = oracle.compare(out.reshape(-1, out.shape[-1]), ref.reshape(-1, ref.shape[-1]))
    assert r["ok"], r
    return r


# ---------------------------------------------------------------- golden fixtures

def test_golden_known_answers(w, cuda_dev, golden_dir):
    kat = np.load(os.path.join(golden_dir, "chain_kat.npz"))
    meta = json.load(open(os.path.join(golden_dir, "chain_kat.json")))
    for name in meta["cases"]:
        A, B, P = kat[name + "_A"], kat[name + "_B"], kat[name + "_P"]
        _check(_run(w, cuda_dev, A, B, 1.0), P)                       # f32 chain, SIMT
        if "f16" in name:                                             # operands are exact f16 values
            _check(_run(w, cuda_dev, A.astype(np.float16), B.astype(np.float16), 1.0), P)   # tcgen05
            _check(_run(w, cuda_dev, A.astype(np.float16), B.astype(np.float16), 1.0, out_dtype=w.F32), P)


# ---------------------------------------------------------------- benchmark configurations

def test_cfg1_decomposed_f32(w, cuda_dev):
    A = oracle.fill((128, 128), "random", 1)
    B = oracle.fill((128, 128), "random", 1)
    r = _check(_run(w, cuda_dev, A, B, 1.0), oracle.chain(A, B, 1.0))
    assert r["max_abs"] < 1e-5
    assert w.plan_query(w.make_desc(1, 128, 128, 128, w.F32, w.F32)).kernel == w.KERNEL_SIMT_FUSED


def test_cfg2_f16_native_full_size(w, cuda_dev):
    A = oracle.normal((4096, 1024), 21)
    B = oracle.normal((1024, 1024), 22)
    out = _run(w, cuda_dev, A, B, 1 / 32)
    _check(out, oracle.chain(A, B, 1 / 32))


def test_cfg3_batched_named_softmax_slice(w, cuda_dev):
    A = oracle.normal((4, 2048, 128), 31)
    B = oracle.normal((4, 128, 2048), 32)
    _check(_run(w, cuda_dev, A, B, 128 ** -0.5), oracle.chain(A, B, 128 ** -0.5))


def test_cfg3_full_batch_properties(w, cuda_dev):
    """All 64 batches: every batch must equal the same batch run alone (no cross-batch
    leakage), rows sum to one, and a sampled batch matches the checker."""
    import torch
    g = torch.Generator(device=cuda_dev); g.manual_seed(5)
    A = torch.randn((64, 2048, 128), device=cuda_dev, generator=g).half()
    B = torch.randn((64, 128, 2048), device=cuda_dev, generator=g).half()
    out = w.matmul_softmax(A, B, 128 ** -0.5)
    w.check_device_status()
    sums = out.float().sum(-1)
    assert float((sums - 1).abs().max()) <= 1e-3
    for b in (0, 37, 63):
        # (the epilogue schedule may differ between the two launches, so allow the last f16 bit)
        alone = w.matmul_softmax(A[b].contiguous(), B[b].contiguous(), 128 ** -0.5)
        assert float((alone.float() - out[b].float()).abs().max()) <= 2.0 ** -10 * float(out[b].max())
    ref = oracle.chain(A[37].cpu().numpy(), B[37].cpu().numpy(), 128 ** -0.5)
    _check(out[37].cpu().numpy(), ref)


def test_cfg4_vocab_wide_sampled_rows(w, cuda_dev):
    import torch
    g = torch.Generator(device=cuda_dev); g.manual_seed(7)
    A = torch.randn((8192, 4096), device=cuda_dev, generator=g).half()
    B = (torch.randn((4096, 32000), device=cuda_dev, generator=g) * 0.02).half()
    out = w.matmul_softmax(A, B, 1.0)
    w.check_device_status()
    assert w.plan_query(w.make_desc(1, 8192, 32000, 4096)).kernel == w.KERNEL_TC_TILED
    sums = out.float().sum(-1)
    assert float((sums - 1).abs().max()) <= 1e-3
    idx = [0, 1, 127, 128, 129, 4095, 4096, 8191]
    ref = oracle.chain(A[idx].cpu().numpy(), B.cpu().numpy(), 1.0)
    _check(out[idx].cpu().numpy(), ref)
    # the row split is invisible: the first 128 rows alone give the same bits
    alone = w.matmul_softmax(A[:128].contiguous(), B, 1.0)
    assert float((alone.float() - out[:128].float()).abs().max()) <= 2.0 ** -10 * float(out[:128].max())


def test_cfg5_skinny_decode(w, cuda_dev):
    A = oracle.normal((16, 4096), 51)
    B = oracle.normal((4096, 32000), 52, 0.02)
    _check(_run(w, cuda_dev, A, B, 1.0), oracle.chain(A, B, 1.0))


# ---------------------------------------------------------------- shapes and edges

@pytest.mark.parametrize("M,N,K,scale", [
    (128, 256, 64, 0.125), (128, 256, 16, 0.25), (128, 256, 1024, 1 / 32), (256, 1024, 256, 1 / 16),
    (200, 520, 72, 0.2), (64, 128, 64, 0.125), (1, 8, 8, 1.0), (129, 2048, 40, 0.1), (777, 264, 136, -0.07),
    (8192, 128, 64, 1.0),
])
def test_tensor_core_cluster_shapes(w, cuda_dev, M, N, K, scale):
    assert w.plan_query(w.make_desc(1, M, N, K)).kernel == w.KERNEL_TC_CLUSTER
    A = oracle.normal((M, K), M + N)
    B = oracle.normal((K, N), K)
    _check(_run(w, cuda_dev, A, B, scale), oracle.chain(A, B, scale))


@pytest.mark.parametrize("M,N,K,flags", [(300, 1024, 256, "tiled"), (256, 4096, 128, 0), (50, 2304, 64, 0),
                                           (130, 520, 72, "tiled")])
def test_tiled_two_pass_shapes(w, cuda_dev, M, N, K, flags):
    fl = w.FLAG_FORCE_TILED if flags == "tiled" else 0
    d = w.make_desc(1, M, N, K, flags=fl)
    assert w.plan_query(d).kernel == w.KERNEL_TC_TILED
    A = oracle.normal((M, K), 3)
    B = oracle.normal((K, N), 4)
    _check(_run(w, cuda_dev, A, B, 0.09, flags=fl), oracle.chain(A, B, 0.09))


def test_persistent_many_tiles(w, cuda_dev):
    """More row blocks than resident clusters: accumulator double buffering, barrier
    phases and the statistics exchange wrap around many times."""
    for M, N in ((20000, 256), (40000, 512), (9000, 2048)):
        A = oracle.normal((M, 64), 9)
        B = oracle.normal((64, N), 10)
        _check(_run(w, cuda_dev, A, B, 0.125), oracle.chain(A, B, 0.125))


def test_batched_shared_and_own_b(w, cuda_dev):
    A = oracle.normal((3, 300, 128), 1)
    B = oracle.normal((3, 128, 512), 2)
    _check(_run(w, cuda_dev, A, B, 0.09), oracle.chain(A, B, 0.09))
    _check(_run(w, cuda_dev, A, B[0], 0.09), oracle.chain(A, B[0], 0.09))


@pytest.mark.parametrize("M,N,K", [(100, 72, 40), (33, 70, 17), (5, 1, 3), (16, 3000, 50)])
def test_simt_odd_shapes(w, cuda_dev, M, N, K):
    for dt in (np.float32, np.float16):
        A = oracle.normal((M, K), 5, 1.0, dt)
        B = oracle.normal((K, N), 6, 1.0, dt)
        _check(_run(w, cuda_dev, A, B, 0.3, flags=w.FLAG_FORCE_SIMT), oracle.chain(A, B, 0.3))


def test_baseline_variant_matches_fused(w, cuda_dev):
    """The five-kernel baseline (logits, max, exp, sum, divide through global memory): the tcgen05
    contraction for f16 chains -- ragged shapes, both column tiles, batched, a long K loop, the f16
    matmul result -- and SIMT FMAs for f32 chains and for shapes TMA cannot take."""
    A = oracle.normal((257, 96), 7)
    B = oracle.normal((96, 200), 8)
    ref = oracle.chain(A, B, 0.2)
    _check(_run(w, cuda_dev, A, B, 0.2, variant=w.VARIANT_BASELINE), ref)
    _check(_run(w, cuda_dev, A, B, 0.2, variant=w.VARIANT_BASELINE, out_dtype=w.F32), ref)
    _check(_run(w, cuda_dev, A, B, 0.2, variant=w.VARIANT_BASELINE, flags=w.FLAG_FORCE_SIMT), ref)
    for (sa, sb, scale) in (((300, 640), (640, 1032), 0.05), ((3, 200, 64), (3, 64, 520), 0.125), ((130, 72), (72, 96), -0.3)):
        A = oracle.normal(sa, 17); B = oracle.normal(sb, 18)
        ref = np.stack([oracle.chain(A[i], B[i], scale) for i in range(sa[0])]) if len(sa) == 3 else oracle.chain(A, B, scale)
        _check(_run(w, cuda_dev, A, B, scale, variant=w.VARIANT_BASELINE), ref)
    A = oracle.normal((200, 72), 9) * np.float16(0.25); B = oracle.normal((72, 768), 10) * np.float16(0.25)
    got = _run(w, cuda_dev, A, B, 1.0, variant=w.VARIANT_BASELINE, acc_dtype=w.F16, out_dtype=w.F32)
    assert np.abs(got.astype(np.float64) - oracle.chain(A, B, 1.0, acc=oracle.ACC_F16_SEQ)).max() < 5e-3
    A32 = oracle.fill((64, 48), "random", 1); B32 = oracle.fill((48, 80), "random", 1)
    _check(_run(w, cuda_dev, A32, B32, 1.0, variant=w.VARIANT_BASELINE), oracle.chain(A32, B32, 1.0))


def test_f16_matmul_result_chain(w, cuda_dev):
    """The reference's f16-native file spells the matmul with an f16 result; the logits
    are then f16 values.  Checked against the checker's f16-accumulate mode with the
    looser bound that mode needs (a different accumulation order in f16)."""
    A = oracle.normal((256, 64), 11) * np.float16(0.25)
    B = oracle.normal((64, 128), 12) * np.float16(0.25)
    out = _run(w, cuda_dev, A, B, 1.0, acc_dtype=w.F16, out_dtype=w.F32)
    ref16 = oracle.chain(A, B, 1.0, acc=oracle.ACC_F16_SEQ)
    assert np.abs(out - ref16).max() < 5e-3
    out_tc = _run(w, cuda_dev, A, B, 1.0, acc_dtype=w.F16)
    assert np.abs(out_tc.astype(np.float64) - ref16).max() < 5e-3
    # what the kernel is specified to compute -- the f32-accumulated logit rounded to f16 ONCE, then an f32
    # softmax -- restated here in f64 and held to the chain's own tolerance (2e-3 / 1e-3 / argmax)
    logits = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float16).astype(np.float64)
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    once = e / e.sum(axis=1, keepdims=True)
    for got in (out, out_tc):
        r = oracle.compare(got, once)
        assert r["ok"], r


def test_f32_arguments_rounded_to_f16_before_the_matmul(w, cuda_dev):
    """WTC_FLAG_MATMUL_F16: f32 buffers, arith.truncf to f16 on the device, then the f16 chain
    (mlir_pipeline/matmul_softmax_chain_f16_matmul.mlir in the reference).  Same results as
    handing the launch layer operands rounded on the host; the checker sees the rounded values."""
    import torch
    cases = [(1, 300, 1024, 136, 0.07, 0, w.F32, w.F32),           # cluster kernel, ragged M, f32 probabilities
             (1, 256, 128, 64, 1.0, 0, w.F16, w.F32),              # the reference file's types: f16 matmul result, f32 out
             (3, 130, 520, 72, 0.2, 0, w.F32, w.F16),              # batched, B shared
             (1, 64, 2304, 128, 0.1, 0, w.F32, w.F16),             # two-pass tiled schedule behind the rounding
             (1, 33, 100, 50, 0.3, 0, w.F32, w.F32),               # K, N not multiples of 8: SIMT kernel on the rounded copies
             (1, 200, 256, 64, 0.5, w.FLAG_FORCE_SIMT, w.F32, w.F32)]
    for batch, M, N, K, scale, flags, acc, outd in cases:
        rng = np.random.default_rng(M + N)
        A = rng.standard_normal((batch, M, K) if batch > 1 else (M, K)).astype(np.float32)
        B = rng.standard_normal((K, N)).astype(np.float32)
        got = _run(w, cuda_dev, A, B, scale, flags=flags | w.FLAG_MATMUL_F16, acc_dtype=acc, out_dtype=outd)
        same = _run(w, cuda_dev, A.astype(np.float16), B.astype(np.float16), scale, flags=flags, acc_dtype=acc, out_dtype=outd)
        assert np.array_equal(got, same), (batch, M, N, K)
        if acc == w.F32:
            A16, B16 = A.astype(np.float16), B.astype(np.float16)
            ref = np.stack([oracle.chain(A16[i], B16, scale) for i in range(batch)]) if batch > 1 else oracle.chain(A16, B16, scale)
            _check(got, ref)
    # the unfused baseline takes the flag too
    A = np.random.default_rng(5).standard_normal((96, 64)).astype(np.float32)
    B = np.random.default_rng(6).standard_normal((64, 128)).astype(np.float32)
    got = _run(w, cuda_dev, A, B, 1.0, flags=w.FLAG_MATMUL_F16, variant=w.VARIANT_BASELINE)
    _check(got, oracle.chain(A.astype(np.float16), B.astype(np.float16), 1.0))
    # f16 buffers with the flag are a caller error
    with pytest.raises(w.WtcError):
        w.matmul_softmax(torch.zeros((8, 8), device=cuda_dev).half(), torch.zeros((8, 8), device=cuda_dev).half(), flags=w.FLAG_MATMUL_F16)


def test_empty_and_degenerate(w, cuda_dev):
    import torch
    out = w.matmul_softmax(torch.zeros((0, 8), device=cuda_dev).half(), torch.zeros((8, 16), device=cuda_dev).half())
    assert out.shape == (0, 16)
    out = w.matmul_softmax(torch.zeros((4, 0), device=cuda_dev), torch.zeros((0, 5), device=cuda_dev))
    torch.cuda.synchronize()
    assert torch.allclose(out, torch.full((4, 5), 0.2, device=cuda_dev))
    # all-equal logits, and one dominant column
    A = np.zeros((130, 64), np.float16); B = oracle.normal((64, 256), 1)
    out = _run(w, cuda_dev, A, B, 1.0)
    assert np.allclose(out.astype(np.float64), 1 / 256, atol=1e-5)
    A = np.ones((128, 64), np.float16); B = np.zeros((64, 512), np.float16); B[:, 300] = 1
    out = _run(w, cuda_dev, A, B, 1.0)
    assert (out.argmax(1) == 300).all() and np.abs(out[:, 300] - 1).max() < 1e-3


def test_host_buffer_entry_point(w, cuda_dev):
    A = oracle.normal((512, 256), 13)
    B = oracle.normal((256, 1024), 14)
    out = w.matmul_softmax_host(A, B, 1 / 16)
    _check(out, oracle.chain(A, B, 1 / 16))
    out2 = w.matmul_softmax_host(A, B, 1 / 16)          # cached device buffers
    assert np.array_equal(out, out2)
    A32 = oracle.fill((64, 32), "linear"); B32 = oracle.fill((32, 48), "linear")
    _check(w.matmul_softmax_host(A32, B32, 1.0), oracle.chain(A32, B32, 1.0))


def test_host_calls_in_flight(w, cuda_dev):
    """submit / wait: several calls with different operands through the two slots of device buffers, two in
    flight at a time, waited for in order, out of order and twice; each result against the CPU checker."""
    import torch
    M, N, K = 700, 1024, 192
    hc = w.HostChain(1, M, N, K, 0.07)
    As = [torch.from_numpy(oracle.normal((M, K), 90 + i)).pin_memory().numpy() for i in range(5)]
    B = torch.from_numpy(oracle.normal((K, N), 99)).pin_memory().numpy()
    outs = [torch.empty((M, N), dtype=torch.float16).pin_memory().numpy() for _ in range(5)]
    tickets = []
    for i in range(5):
        tickets.append(hc.submit(As[i], B, outs[i]))       # the third submit waits for the first call itself
        if i >= 1 and i % 2 == 1:
            hc.wait(tickets[i - 1])
    assert tickets == list(range(tickets[0], tickets[0] + 5))
    for t in reversed(tickets):
        hc.wait(t)
    hc.wait(tickets[2])                                     # waiting twice is fine
    hc.wait(-1)
    with pytest.raises(w.WtcError):
        hc.wait(tickets[-1] + 7)                            # never issued
    for i in range(5):
        _check(outs[i], oracle.chain(As[i], B, 0.07))
    # a batched chain with a B per batch, two-pass tiled schedule per slab, between two cluster calls
    hb = w.HostChain(3, 200, 2304, 64, 0.125)
    Ab = torch.from_numpy(oracle.normal((3, 200, 64), 81)).pin_memory().numpy()
    Bb = torch.from_numpy(oracle.normal((3, 64, 2304), 82)).pin_memory().numpy()
    ob = torch.empty((3, 200, 2304), dtype=torch.float16).pin_memory().numpy()
    t0 = hc.submit(As[0], B, outs[1])
    t1 = hb.submit(Ab, Bb, ob)
    hb.wait(t1)
    hc.wait(t0)
    _check(ob, np.stack([oracle.chain(Ab[b], Bb[b], 0.125) for b in range(3)]))
    assert np.array_equal(outs[1], outs[0])
    assert np.array_equal(w.matmul_softmax_host(As[3], B, 0.07), outs[3])   # the one-call form is submit + wait


@pytest.mark.parametrize("slabs", ["1", "3", "8"])
def test_host_entry_point_slabs(w, cuda_dev, monkeypatch, slabs):
    """The host-buffer call moves row ranges (or batch ranges) through copy-in, compute and
    copy-out streams; any cut gives the same bytes as the single-slab call."""
    monkeypatch.setenv("WTC_HOST_SLABS", slabs)
    cases = [((1000, 136), (136, 1024), 0.07),             # ragged M: the last slab is short
             ((5, 300, 72), (5, 72, 520), 0.2),            # batched, B per batch: slabs are batch ranges
             ((4, 130, 64), (64, 256), 0.5),               # batched, B shared
             ((700, 64), (64, 2304), 0.1)]                 # two-pass tiled schedule per slab
    for sa, sb, scale in cases:
        A = oracle.normal(sa, sa[-2]); B = oracle.normal(sb, sb[-1])
        out = w.matmul_softmax_host(A, B, scale)
        if A.ndim == 3:
            ref = np.stack([oracle.chain(A[i], B[i] if B.ndim == 3 else B, scale) for i in range(A.shape[0])])
        else:
            ref = oracle.chain(A, B, scale)
        _check(out, ref)
        monkeypatch.setenv("WTC_HOST_SLABS", "1")
        assert np.array_equal(out, w.matmul_softmax_host(A, B, scale)), (sa, slabs)
        monkeypatch.setenv("WTC_HOST_SLABS", slabs)
    A = np.random.default_rng(3).standard_normal((520, 64)).astype(np.float32)      # f32 buffers rounded on the device, per slab
    B = np.random.default_rng(4).standard_normal((64, 256)).astype(np.float32)
    out = w.matmul_softmax_host(A, B, 1.0, flags=w.FLAG_MATMUL_F16)
    _check(out, oracle.chain(A.astype(np.float16), B.astype(np.float16), 1.0))


def test_n_sharded_partial_and_finish(w, cuda_dev):
    """Two column shards on one GPU, combined the way two GPUs would combine them:
    per-row (max, sum) of each shard gathered, then each shard normalised."""
    import torch
    A = oracle.normal((300, 128), 15)
    B = oracle.normal((128, 1536), 16)
    ref = oracle.chain(A, B, 0.11)
    tA = torch.from_numpy(A).to(cuda_dev)
    splits = [(0, 768), (768, 1536)]
    outs, wss, stats, descs = [], [], [], []
    for c0, c1 in splits:
        tB = torch.from_numpy(np.ascontiguousarray(B[:, c0:c1])).to(cuda_dev)
        o = torch.empty((300, c1 - c0), device=cuda_dev, dtype=torch.float16)
        d0 = w.make_desc(1, 300, c1 - c0, 128)
        ws = torch.empty(max(16, w.workspace_bytes(d0)), device=cuda_dev, dtype=torch.uint8)
        rs = torch.empty((300, 2), device=cuda_dev, dtype=torch.float32)
        descs.append(w.matmul_softmax_partial(tA, tB, 0.11, o, ws, rs))
        outs.append(o); wss.append(ws); stats.append(rs)
    allst = torch.stack(stats).contiguous()
    for i in range(2):
        w.matmul_softmax_finish(descs[i], outs[i], wss[i], allst, 2)
    w.check_device_status()
    full = torch.cat(outs, dim=1).cpu().numpy()
    _check(full, ref)


def test_linearity_and_shift_properties(w, cuda_dev):
    """Size-independent properties at the full f16 size: scaling the logits by 0 gives
    the uniform row; permuting B's columns permutes the probabilities."""
    import torch
    g = torch.Generator(device=cuda_dev); g.manual_seed(3)
    A = torch.randn((4096, 1024), device=cuda_dev, generator=g).half()
    B = torch.randn((1024, 1024), device=cuda_dev, generator=g).half()
    uni = w.matmul_softmax(A, B, 0.0)
    assert torch.allclose(uni.float(), torch.full_like(uni, 1 / 1024).float(), atol=1e-6)
    p = w.matmul_softmax(A, B, 1 / 32)
    perm = torch.randperm(1024, device=cuda_dev, generator=g)
    pp = w.matmul_softmax(A, B[:, perm].contiguous(), 1 / 32)
    w.check_device_status()
    assert float((pp.float() - p[:, perm].float()).abs().max()) <= 2e-3
    assert float((p.float().sum(-1) - 1).abs().max()) <= 1e-3


@pytest.mark.parametrize("M,N,K,flags", [(8192, 128, 64, 0), (777, 1024, 136, 0), (200, 520, 72, 0), (300, 1024, 256, "tiled"),
                                           (64, 4096, 128, 0)])
def test_f32_probabilities_on_the_tensor_core_path(w, cuda_dev, M, N, K, flags):
    """f16 operands, f32 result (the reference's f16-native chain returns f32)."""
    fl = w.FLAG_FORCE_TILED if flags == "tiled" else 0
    assert w.plan_query(w.make_desc(1, M, N, K, out_dtype=w.F32, flags=fl)).kernel in (w.KERNEL_TC_CLUSTER, w.KERNEL_TC_TILED)
    A = oracle.normal((M, K), 71)
    B = oracle.normal((K, N), 72)
    out = _run(w, cuda_dev, A, B, 0.11, out_dtype=w.F32, flags=fl)
    assert out.dtype == np.float32
    r = _check(out, oracle.chain(A, B, 0.11))
    assert r["max_abs"] < 2e-5          # no f16 rounding of the result


def test_tile_choice_from_best_json_is_honoured(w, cuda_dev):
    """tileN = 128 selects the 128-column kernels (cluster of 8 for N = 1024; tiled beyond)."""
    for M, N, K in ((4096, 1024, 1024), (300, 520, 72), (256, 2304, 128)):
        A = oracle.normal((M, K), 61)
        B = oracle.normal((K, N), 62)
        ref = oracle.chain(A, B, 1 / 32)
        _check(_run(w, cuda_dev, A, B, 1 / 32, tiles=(128, 128, 64)), ref)
        _check(_run(w, cuda_dev, A, B, 1 / 32, tiles=(128, 256, 64)), ref)
        _check(_run(w, cuda_dev, A, B, 1 / 32, tiles=(64, 128, 32)), ref)     # the reference's pinned tile, honoured as given


@pytest.mark.parametrize("tile_k", [32, 128])
@pytest.mark.parametrize("M,N,K,tile_n,flags,used_k", [
    (777, 1024, 200, 128, 0, None),          # cluster of 8 x 128 columns, ragged M, K tail shorter than a stage
    (300, 520, 72, 128, 0, None),            # ragged N and K
    (4096, 1024, 1024, 256, 0, {128: 64}),   # cluster of 4 x 256 columns: 128-deep stages have no kernel there
    (256, 2304, 128, 256, 0, None),          # two-pass tiled schedule, 256-column tiles
    (300, 1024, 256, 128, "tiled", None),    # two-pass tiled schedule, 128-column tiles
    (130, 520, 40, 256, "tiled", None),      # K shorter than one 128-deep stage: the second box of A is all padding
])
def test_stage_depth_from_best_json_is_honoured(w, cuda_dev, M, N, K, tile_n, flags, used_k, tile_k):
    """tileK = 32 / 128 is the K depth of one pipeline stage (64-byte-swizzled A rows; two 64-column
    blocks of A per stage); the plan reports the depth it runs and whether it replaced the request."""
    fl = w.FLAG_FORCE_TILED if flags == "tiled" else 0
    want_k = (used_k or {}).get(tile_k, tile_k)
    plan = w.plan_query(w.make_desc(1, M, N, K, flags=fl, tile_m=128, tile_n=tile_n, tile_k=tile_k))
    assert (plan.tile_m, plan.tile_n, plan.tile_k) == (128, tile_n, want_k)
    assert plan.tile_substituted == (0 if want_k == tile_k else 1)
    A = oracle.normal((M, K), 71)
    B = oracle.normal((K, N), 72)
    _check(_run(w, cuda_dev, A, B, 0.05, flags=fl, tiles=(128, tile_n, tile_k)), oracle.chain(A, B, 0.05))


@pytest.mark.parametrize("tile_n,tile_k", [(128, 32), (128, 64), (256, 32), (256, 64)])
@pytest.mark.parametrize("M,N,K,flags", [
    (777, 1024, 200, 0),            # clusters, ragged M (a last tile of 9 rows), K tail
    (64, 520, 72, 0),               # exactly one 64-row tile, ragged N
    (4096, 1024, 1024, 0),          # the headline shape
    (300, 2304, 128, 0),            # two-pass tiled schedule
    (130, 520, 40, "tiled"),        # tiled by request
])
def test_64_row_tiles_from_best_json_are_honoured(w, cuda_dev, M, N, K, flags, tile_n, tile_k):
    """tileM = 64 runs tcgen05.mma with M = 64 (accumulator rows in lanes 0-15 of each quarter of tensor
    memory); 64 x 128 x 32 is the tile the reference's own pinned search result names."""
    fl = w.FLAG_FORCE_TILED if flags == "tiled" else 0
    plan = w.plan_query(w.make_desc(1, M, N, K, flags=fl, tile_m=64, tile_n=tile_n, tile_k=tile_k))
    assert (plan.tile_m, plan.tile_n, plan.tile_k, plan.tile_substituted) == (64, tile_n, tile_k, 0)
    A = oracle.normal((M, K), 75)
    B = oracle.normal((K, N), 76)
    _check(_run(w, cuda_dev, A, B, 0.05, flags=fl, tiles=(64, tile_n, tile_k)), oracle.chain(A, B, 0.05))


def test_64_row_tiles_batched_and_replaced(w, cuda_dev):
    A = oracle.normal((3, 1000, 160), 77)
    B = oracle.normal((3, 160, 1024), 78)
    ref = np.stack([oracle.chain(A[b], B[b], 0.08) for b in range(3)])
    _check(_run(w, cuda_dev, A, B, 0.08, tiles=(64, 128, 32)), ref)
    # no 64-row kernel with 128-deep stages or f32 probabilities: the row tile is replaced and reported
    plan = w.plan_query(w.make_desc(1, 256, 1024, 256, tile_m=64, tile_n=128, tile_k=128))
    assert (plan.tile_m, plan.tile_k, plan.tile_substituted) == (128, 128, 1)
    plan = w.plan_query(w.make_desc(1, 256, 1024, 256, out_dtype=w.F32, tile_m=64, tile_n=128, tile_k=32))
    assert (plan.tile_m, plan.tile_k, plan.tile_substituted) == (128, 64, 1)
    _check(_run(w, cuda_dev, A[0], B[0], 0.08, out_dtype=w.F32, tiles=(64, 128, 32)), ref[0])


def test_stage_depth_batched_many_tiles(w, cuda_dev):
    """Several tiles per CTA and a B per batch with 32- and 128-deep stages (the operand ring runs on across tiles)."""
    A = oracle.normal((3, 5000, 160), 73)
    B = oracle.normal((3, 160, 1024), 74)
    ref = np.stack([oracle.chain(A[b], B[b], 0.08) for b in range(3)])
    for tile_k in (32, 128):
        _check(_run(w, cuda_dev, A, B, 0.08, tiles=(128, 128, tile_k)), ref)
    _check(_run(w, cuda_dev, A, B, 0.08, tiles=(128, 256, 32)), ref)


def test_narrow_rows_take_the_128_column_tile(w, cuda_dev):
    """Rows of at most 128 columns run the 128-column kernels by default (f16 and f32
    probabilities, one-CTA cluster and two-pass schedule); a 256 hint still gets the wide tile."""
    for M, N, K, scale in ((8192, 128, 64, 1.0), (300, 72, 136, 0.3), (1000, 120, 64, 0.2), (64, 8, 8, 1.0)):
        A = oracle.normal((M, K), M + 1)
        B = oracle.normal((K, N), N + 1)
        ref = oracle.chain(A, B, scale)
        for kw in (dict(), dict(out_dtype=w.F32), dict(flags=w.FLAG_FORCE_TILED), dict(flags=w.FLAG_FORCE_TILED, out_dtype=w.F32),
                   dict(tiles=(128, 256, 64))):
            _check(_run(w, cuda_dev, A, B, scale, **kw), ref)
    A = oracle.normal((512, 64), 3); B = oracle.normal((64, 2304), 4)          # f32 probabilities on 128-column tiles, tiled and cluster
    ref = oracle.chain(A, B, 0.125)
    _check(_run(w, cuda_dev, A, B, 0.125, out_dtype=w.F32, tiles=(128, 128, 64)), ref)
    _check(_run(w, cuda_dev, A[:, :64], B[:, :1024], 0.125, out_dtype=w.F32, tiles=(128, 128, 64)), oracle.chain(A[:, :64], B[:, :1024], 0.125))


def test_few_rows_wide_row_rescale_is_split_over_ctas(w, cuda_dev):
    """With few rows and a wide row the rescale pass runs several CTAs per row, each on a column
    range; same numbers as the one-CTA-per-row form (checked against the checker)."""
    for M, N, K, kw in ((16, 32000, 64, {}), (5, 10008, 72, {}), (40, 4104, 64, dict(out_dtype=w.F32)), (1, 8200, 128, {})):
        A = oracle.normal((M, K), M + 3)
        B = oracle.normal((K, N), N + 3) * np.float16(0.5)
        _check(_run(w, cuda_dev, A, B, 0.25, **kw), oracle.chain(A, B, 0.25))


# ---------------------------------------------------------------- kernel variants

@pytest.mark.parametrize("extra", [
    "FLAG_EPILOGUE_RELAY",      # two warp groups overlap consecutive tiles, exp values parked in TMEM
    "FLAG_EPILOGUE_SPLIT",      # eight epilogue warps share a tile
    "FLAG_PAIR",                # tcgen05 cta_group::2 whenever the tiled flavour has two row blocks
    "FLAG_NO_PAIR",             # never pair
    "FLAG_OPERANDS_READY",      # loads do not wait for the previous launch on the stream, only the stores do
    None,                       # the launch layer's own choice
])
def test_every_kernel_variant_matches_the_checker(w, cuda_dev, extra):
    xf = getattr(w, extra) if extra else 0
    cases = [
        (777, 1024, 136, 0.07, 0),                  # cluster of 4, ragged M and K, several tiles per cluster
        (9000, 2048, 64, 0.125, 0),                 # cluster of 8, many tiles per CTA
        (200, 520, 72, 0.2, 0),                     # ragged N
        (300, 1024, 256, 1 / 16, w.FLAG_FORCE_TILED),
        (2500, 2304, 520, 0.05, 0),                 # tiled, long K (pairs by default)
    ]
    for M, N, K, scale, flags in cases:
        A = oracle.normal((M, K), M)
        B = oracle.normal((K, N), N)
        _check(_run(w, cuda_dev, A, B, scale, flags=flags | xf), oracle.chain(A, B, scale))
    # a negative scale turns the row maximum into a minimum of the raw accumulators; logits
    # rounded to f16 (the f16 matmul result) take the epilogue's general path; batched with B per batch
    A = oracle.normal((1500, 64), 7); B = oracle.normal((64, 1024), 8)
    _check(_run(w, cuda_dev, A, B, -0.11, flags=xf), oracle.chain(A, B, -0.11))
    A = oracle.normal((3, 520, 72), 9) * np.float16(0.25); B = oracle.normal((3, 72, 768), 10) * np.float16(0.25)
    got = _run(w, cuda_dev, A, B, 1.0, acc_dtype=w.F16, flags=xf)
    ref = np.stack([oracle.chain(A[i], B[i], 1.0, acc=oracle.ACC_F16_SEQ) for i in range(3)])
    assert np.abs(got.astype(np.float64) - ref).max() < 5e-3


def test_operands_ready_keeps_the_order_of_the_stores(w, cuda_dev):
    """With WTC_FLAG_OPERANDS_READY a call's loads run under the tail of the call before it, but its
    stores still come after: back-to-back calls with different operands into ONE output buffer leave
    the last call's result, for every epilogue form (single tile, several tiles per CTA, split, tiled)."""
    import torch
    for (M, N, K, extra) in ((4096, 1024, 256, 0), (9000, 2048, 64, 0), (1024, 1024, 128, w.FLAG_EPILOGUE_SPLIT),
                             (600, 2304, 128, 0)):
        As = [torch.from_numpy(oracle.normal((M, K), 300 + i)).to(cuda_dev) for i in range(6)]
        B = torch.from_numpy(oracle.normal((K, N), 310)).to(cuda_dev)
        out = torch.empty((M, N), dtype=torch.float16, device=cuda_dev)
        calls = [w.PreparedCall(a, B, out, 0.05, flags=w.FLAG_OPERANDS_READY | extra) for a in As]
        sp = w.current_stream_ptr()
        for rep in range(3):
            for c in calls:
                c.launch(sp)
        w.check_device_status()
        torch.cuda.synchronize()
        _check(out.cpu().numpy(), oracle.chain(As[-1].cpu().numpy(), B.cpu().numpy(), 0.05))
