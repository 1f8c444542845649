"""The N > 1 protocol on CPU ranks (gloo, world size 2): shard maps, the layout of the
gathered per-row (max, sum) pairs and the log2-domain combination that the GPU `finish`
kernel performs, checked against the whole-row CPU checker.  No GPU is involved: each
rank computes its shard's partial softmax with numpy in the test itself."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from welder_typical_chain_b200 import sharding  # noqa: E402

LOG2E = 1.4426950408889634


def test_shard_maps():
    assert sharding.split_batches(64, 8) == [(i * 8, i * 8 + 8) for i in range(8)]
    assert sharding.split_batches(5, 2) == [(0, 3), (3, 5)]
    cols = sharding.split_columns(32000, 8)
    assert [(b - a) // 256 for a, b in cols[:5]] == [16] * 5 and [(b - a + 255) // 256 for a, b in cols[5:]] == [15] * 3
    assert cols[0][0] == 0 and cols[-1][1] == 32000 and all(cols[i][1] == cols[i + 1][0] for i in range(7))
    assert all(a % 256 == 0 for a, _ in cols)
    assert sharding.split_columns(1000, 2) == [(0, 512), (512, 1000)]
    assert sharding.split_columns(256, 4) == [(0, 256), (256, 256), (256, 256), (256, 256)]      # fewer tiles than ranks
    assert sharding.split_rows(4096, 3) == [(0, 1408), (1408, 2816), (2816, 4096)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, M, N, K, scale, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.Generator(np.random.PCG64(42))          # same inputs on every rank
        A = rng.standard_normal((M, K)).astype(np.float16)
        B = (rng.standard_normal((K, N)) * 0.5).astype(np.float16)
        c0, c1 = sharding.split_columns(N, world)[rank]
        v = scale * LOG2E * (A.astype(np.float64) @ B[:, c0:c1].astype(np.float64))
        if c1 > c0:
            m = v.max(1)
            e = np.exp2(v - m[:, None])
            pair = np.stack([m, e.sum(1)], axis=1).astype(np.float32)
        else:                                                     # a rank without columns contributes nothing
            e = np.zeros((M, 0))
            pair = np.stack([np.full(M, -np.inf), np.zeros(M)], axis=1).astype(np.float32)
        mine = torch.from_numpy(pair)
        gathered = torch.empty((world * M, 2), dtype=torch.float32)   # rank-major: [world][rows][2]
        dist.all_gather_into_tensor(gathered, mine)               # the one collective of the path
        gm, gl = sharding.combine_pairs(gathered.view(world, M, 2).numpy().astype(np.float64))
        probs = e * np.exp2(pair[:, 0].astype(np.float64) - gm)[:, None] / gl[:, None] if c1 > c0 else e
        np.save(os.path.join(out_dir, f"p{rank}.npy"), probs)
        # timing contract of the benchmark: max over ranks of a per-rank number
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [1000, 256])
def test_column_sharded_softmax_over_gloo(tmp_path, N):
    from oracle import oracle
    world, M, K, scale = 2, 37, 48, 0.3
    mp.spawn(_rank_main, args=(world, _free_port(), M, N, K, scale, str(tmp_path)), nprocs=world, join=True)
    full = np.concatenate([np.load(tmp_path / f"p{r}.npy") for r in range(world)], axis=1)
    rng = np.random.Generator(np.random.PCG64(42))
    A = rng.standard_normal((M, K)).astype(np.float16)
    B = (rng.standard_normal((K, N)) * 0.5).astype(np.float16)
    ref = oracle.chain(A, B, scale)
    assert full.shape == ref.shape
    assert np.abs(full - ref).max() < 1e-6            # f32 pairs, f64 everywhere else
    assert np.abs(full.sum(1) - 1).max() < 1e-6
