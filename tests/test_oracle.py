"""CPU checks of the checker itself: generators and f16 conversions bit-for-bit
against vectors taken from the reference, the chain against known answers the
reference's own checker accepted, and the comparison rules."""
import json
import os

import numpy as np
import pytest

from oracle import oracle


@pytest.fixture(scope="module")
def gen(golden_dir):
    return np.load(os.path.join(golden_dir, "generators.npz"))


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(os.path.join(golden_dir, "chain_kat.npz"))


def test_linear_matches_reference_checker(gen):
    # verify_matmul_softmax.py:43-45 computes in f64; the profiler in f32
    ours = oracle.fill((4096,), "linear").astype(np.float64)
    assert np.abs(ours - gen["py_linear"]).max() < 2e-7      # two f32 roundings of values up to 0.52


@pytest.mark.parametrize("seed", [0, 1, 12345])
def test_xorshift_matches_reference_checker(gen, seed):
    ours = oracle.fill((4096,), "random", seed).astype(np.float64)
    assert np.abs(ours - gen[f"py_random_seed{seed}"]).max() < 2e-7


@pytest.mark.parametrize("mode,seed", [("linear", 1), ("random", 0), ("random", 1), ("random", 12345)])
def test_generators_bit_exact_against_reference_profiler(gen, mode, seed):
    f32 = oracle.fill((37, 111), mode, seed, np.float32)
    assert np.array_equal(f32.view(np.uint32), gen[f"cxx_{mode}_f32_seed{seed}"].view(np.uint32))
    f16 = oracle.fill((37, 111), mode, seed, np.float16)
    assert np.array_equal(f16.view(np.uint16), gen[f"cxx_{mode}_f16_seed{seed}"])


def test_f16_conversions_bit_exact(gen):
    L = oracle.lib()
    sp = gen["special_f32"]
    rne = np.array([L.wtc_oracle_f32_to_f16_rne(float(x)) for x in sp], dtype=np.uint16)
    prof = np.array([L.wtc_oracle_f32_to_f16_profiler(float(x)) for x in sp], dtype=np.uint16)
    assert np.array_equal(rne, gen["py_f16_bits"])
    assert np.array_equal(prof, gen["cxx_f16_bits"])
    # nearest-even agrees with numpy's conversion on everything finite
    finite = np.isfinite(sp)
    assert np.array_equal(rne[finite], sp[finite].astype(np.float16).view(np.uint16))
    # the two conversions differ exactly where the reference's do (ties)
    assert (rne != prof).sum() == (gen["py_f16_bits"] != gen["cxx_f16_bits"]).sum() > 0


def test_chain_known_answers(kat, golden_dir):
    meta = json.load(open(os.path.join(golden_dir, "chain_kat.json")))
    for name in meta["cases"]:
        assert meta["reference_checker_verdicts"][name].startswith("PASS")
        p = oracle.chain(kat[name + "_A"], kat[name + "_B"], 1.0)
        assert np.abs(p - kat[name + "_P"]).max() < 1e-14, name
        assert np.abs(p.sum(axis=1) - 1).max() < 1e-12


def test_chain_against_numpy_f64():
    rng = np.random.default_rng(3)
    A = rng.standard_normal((5, 33, 17)).astype(np.float32)
    B = rng.standard_normal((5, 17, 29)).astype(np.float32)
    s = 0.37 * np.einsum("bmk,bkn->bmn", A.astype(np.float64), B.astype(np.float64))
    e = np.exp(s - s.max(-1, keepdims=True))
    ref = e / e.sum(-1, keepdims=True)
    assert np.abs(oracle.chain(A, B, 0.37) - ref).max() < 1e-14
    # one B shared by every batch
    ref0 = oracle.chain(A, B[0], 0.37)
    for b in range(5):
        assert np.array_equal(ref0[b], oracle.chain(A[b], B[0], 0.37))


def test_accumulate_modes_and_loop_baseline():
    A = oracle.normal((64, 256), 1)
    B = oracle.normal((256, 96), 2)
    p64 = oracle.chain(A, B, 1 / 16)
    p32 = oracle.chain(A, B, 1 / 16, acc=oracle.ACC_F32_SEQ)
    p16 = oracle.chain(A, B, 1 / 16, acc=oracle.ACC_F16_SEQ)
    loops = oracle.chain_loops_f32(A, B, 1 / 16)
    assert np.abs(p64 - p32).max() < 1e-5
    assert np.abs(p64 - loops).max() < 1e-5
    assert 1e-6 < np.abs(p64 - p16).max() < 5e-2       # f16 accumulation is visibly coarser
    one = oracle.chain_loops_f32(A, B, 1 / 16, threads=1)
    assert np.array_equal(one, loops)                  # row-parallel only: thread count cannot change bits


def test_edge_shapes():
    assert oracle.chain(np.zeros((0, 4), np.float32), np.zeros((4, 3), np.float32)).shape == (0, 3)
    p = oracle.chain(np.ones((2, 0), np.float32), np.ones((0, 5), np.float32))
    assert np.allclose(p, 0.2)                         # K = 0: all logits 0 -> uniform
    p = oracle.chain(np.ones((3, 2), np.float32), np.ones((2, 1), np.float32))
    assert np.array_equal(p, np.ones((3, 1)))          # N = 1
    with pytest.raises(ValueError):
        oracle.chain(np.ones((3, 2), np.float32), np.ones((3, 2), np.float32))
    with pytest.raises(TypeError):
        oracle.chain(np.ones((3, 2), np.float32), np.ones((2, 2), np.float16))


def test_compare_rules():
    ref = np.array([[0.5, 0.3, 0.2], [0.1, 0.45, 0.45]])
    assert oracle.compare(ref.astype(np.float16), ref)["ok"]
    bad = ref.copy(); bad[0, 0] += 3e-3; bad[0, 1] -= 3e-3
    assert not oracle.compare(bad, ref, out_is_f16=False)["ok"]
    flipped = np.array([[0.3, 0.5, 0.2], [0.1, 0.45, 0.45]])
    assert oracle.compare(flipped, ref, out_is_f16=False)["argmax_mismatch"] == 1
    # an exact tie may resolve either way
    tie = np.array([[0.5, 0.3, 0.2], [0.1, 0.4497, 0.4503]])
    r = oracle.compare(tie.astype(np.float16), ref)
    assert r["argmax_mismatch"] == 0
    assert not oracle.compare(np.array([[np.nan, 0.5, 0.5]]), ref[:1], out_is_f16=False)["ok"]


def test_dump_format_roundtrip(tmp_path):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    path = str(tmp_path / "out.bin")
    oracle.write_dump(path, a)
    meta = json.load(open(path + ".json"))
    assert meta == dict(sym="%out", rank=2, elem_bytes=4, offset=0, sizes=[3, 4], strides=[4, 1], bytes=48)
    assert np.array_equal(np.fromfile(path, dtype=np.float32).reshape(3, 4), a)
