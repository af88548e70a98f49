"""Column-sharded FP4 GEMM: the sharded entry point on one GPU (writing a column range of a wider buffer) and the
two-GPU layer (peer-store epilogue, and the NCCL all-gather baseline) against the oracle."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _operands(m, n, k, fmt, seed):
    rng = np.random.default_rng(seed)
    a = wo.rtn_xxfp4(rng.standard_normal((m, k)), fmt)
    b = wo.rtn_xxfp4(rng.standard_normal((n, k)) * 0.02, fmt)
    return a, b


@pytest.mark.parametrize("fmt,m", [("mxfp4", 300), ("nvfp4", 300), ("mxfp4", 40)])
def test_sharded_entry_writes_its_column_range(fmt, m):
    """world = 1: the kernel must fill columns [col0, col0 + n) of a wider buffer and leave the rest alone
    (M > 128 runs the CTA-pair kernel, M = 40 the single-CTA one)."""
    from wush_b200 import _lib
    from wush_b200 import qutlass_ops as ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    n, k, ldy, col0 = 264, 512, 1024, 128
    a, b = _operands(m, n, k, fmt, 3)
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(dev)
    xs, ws = ops.to_blocked(t(a["scale_quant"])).view(-1), ops.to_blocked(t(b["scale_quant"])).view(-1)
    xq, wq = t(a["e2m1"]), t(b["e2m1"])
    alpha = 1.0 / 9.0 if fmt == "mxfp4" else 1.0 / 100.0
    al = torch.tensor([alpha], device=dev)
    y = torch.full((m, ldy), 7.0, dtype=torch.bfloat16, device=dev)
    ptrs = (ctypes.c_void_p * 1)(y.data_ptr())
    rc = lib.wush_gemm_fp4_bf16_tn_sharded(_lib.FORMAT_MXFP4 if fmt == "mxfp4" else _lib.FORMAT_NVFP4, xq.data_ptr(),
                                           wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), al.data_ptr(), ptrs, 1, 0, ldy,
                                           col0, m, n, k, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    want = wo.fp4_gemm(a["e2m1"], a["scale_quant"], b["e2m1"], b["scale_quant"], alpha, fmt)
    got = y.double().cpu().numpy()
    assert np.linalg.norm(got[:, col0:col0 + n] - want) <= 1e-2 * np.linalg.norm(want)
    assert (got[:, :col0] == 7.0).all() and (got[:, col0 + n:] == 7.0).all()
    # argument checks
    assert lib.wush_gemm_fp4_bf16_tn_sharded(0, xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), al.data_ptr(),
                                             ptrs, 1, 0, 256, col0, m, n, k, None, None) == -2
    assert lib.wush_gemm_fp4_bf16_tn_sharded(0, xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), al.data_ptr(),
                                             ptrs, 9, 0, ldy, col0, m, n, k, None, None) == -2


def _worker(rank, world, port, out, peer):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wush_b200 import qutlass_ops as ops
    from wush_b200.sharded import ColumnShardedFP4Linear, shard_bounds
    m, n, k = 384, 1024, 512
    a, b = _operands(m, n, k, "mxfp4", 17)
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(dev)
    c0, c1 = shard_bounds(n, world, rank)
    layer = ColumnShardedFP4Linear(t(b["e2m1"][c0:c1]), t(b["scale_quant"][c0:c1]), n, "mx", 1.0 / 9.0, max_tokens=512, peer=peer)
    assert layer.fused == peer
    xq, xs = t(a["e2m1"]), ops.to_blocked(t(a["scale_quant"])).view(-1)
    for _ in range(2):                                    # the second pass reuses the output buffer
        y = layer.forward(xq, xs)
    torch.cuda.synchronize()
    mine = y.clone()
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(mine, ref)                         # every rank holds the same complete output
    if rank == 0:
        np.save(out, y.float().cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("peer", [True, False])
def test_two_gpu_column_sharded_layer(tmp_path, peer):
    import torch.multiprocessing as mp
    out = str(tmp_path / "y.npy")
    mp.spawn(_worker, args=(2, 29950 + os.getpid() % 200 + (11 if peer else 0), out, peer), nprocs=2, join=True)
    a, b = _operands(384, 1024, 512, "mxfp4", 17)
    want = wo.fp4_gemm(a["e2m1"], a["scale_quant"], b["e2m1"], b["scale_quant"], 1.0 / 9.0, "mxfp4")
    got = np.load(out).astype(np.float64)
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
