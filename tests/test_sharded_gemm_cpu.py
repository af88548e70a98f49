"""Host logic of the column-sharded FP4 linear layer on two gloo ranks, with a CPU stand-in for the kernel."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds():
    from wush_b200.sharded import shard_bounds
    assert [shard_bounds(1024, 4, r) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    assert shard_bounds(8192, 8, 7) == (7168, 8192)
    with pytest.raises(ValueError):
        shard_bounds(1000, 8, 0)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from wush_b200.sharded import ColumnShardedFP4Linear, shard_bounds
    g = torch.Generator().manual_seed(5)
    n, k, m = 64, 32, 6
    w = torch.randn(n, k, generator=g)
    x = torch.randn(m, k, generator=g)
    c0, c1 = shard_bounds(n, world, rank)
    # stand-in "quantized" operands: the float matrices themselves, viewed as bytes
    fake_gemm = lambda xq, wq, xs, ws: xq.view(torch.float32) @ wq.view(torch.float32).T
    layer = ColumnShardedFP4Linear(w[c0:c1].contiguous().view(torch.uint8), torch.zeros(1), n, gemm_fn=fake_gemm)
    assert (layer.world, layer.rank, layer.col0, layer.n_shard, layer.fused) == (world, rank, c0, n // world, False)
    y = layer.forward(x.contiguous().view(torch.uint8), torch.zeros(1))
    assert y.shape == (m, n)
    assert torch.allclose(y, x @ w.T, atol=1e-5)
    if rank == 0:
        np.save(out, y.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_layout(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "y.npy")
    mp.spawn(_worker, args=(2, 29800 + os.getpid() % 150, out), nprocs=2, join=True)
    assert np.load(out).shape == (6, 64)
