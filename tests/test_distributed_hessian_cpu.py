"""Host logic of the token-sharded Hessian on CPU ranks (gloo, world size 2): panel partition,
packed panel all-reduce, token counting, final 1/N scaling and mirror.  The CUDA kernels are
replaced by float32 torch stand-ins injected through the class's hooks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _acc(h, x, r0, r1, lower_only):
    xf = x.float()
    upd = xf[:, r0:r1].t() @ xf[:, :r1]
    rows = torch.arange(r0, r1)[:, None]
    cols = torch.arange(r1)[None, :]
    h[r0:r1, :r1] += torch.where(cols <= rows, upd, torch.zeros_like(upd))


def _fin(h, scale):
    low = torch.tril(h) * scale
    h.copy_(low + torch.tril(low, -1).t())


def _worker(rank, world, port, mode, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import synth
    from wush_b200.hessian import DistributedHessian
    hidden = 384
    x = synth.activations(96 + 32 * rank, hidden, seed=40 + rank)     # ragged shards
    dh = DistributedHessian(hidden, "cpu", panels=3, accumulate_fn=_acc, finalize_fn=_fin)
    if mode == "update":
        dh.update(x[:50][None])
        dh.update(x[50:])
    else:
        dh.accumulate_overlapped(x)
    h = dh.finalize()
    if rank == 0:
        np.save(out, h.numpy())
        assert dh.num_samples == sum(96 + 32 * r for r in range(world))
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["update", "overlapped"])
def test_two_rank_hessian_matches_single_process(tmp_path, mode):
    from oracle import synth
    from oracle import wush_oracle as wo
    out = str(tmp_path / "h.npy")
    port = 29500 + (os.getpid() % 1000) + (0 if mode == "update" else 1)
    mp.spawn(_worker, args=(2, port, mode, out), nprocs=2, join=True)
    got = np.load(out).astype(np.float64)
    xs = [synth.bf16_to_f64(synth.activations(96 + 32 * r, 384, seed=40 + r)) for r in range(2)]
    want = wo.wush_update_sequence(xs)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    assert np.array_equal(got, got.T)


def test_panel_bounds_cover_rows():
    from wush_b200.hessian import panel_bounds
    for hidden in (128, 384, 4096, 14336, 1000):
        for panels in (1, 3, 8):
            b = panel_bounds(hidden, panels)
            assert b[0][0] == 0 and b[-1][1] == hidden
            assert all(b[i][1] == b[i + 1][0] for i in range(len(b) - 1))
            assert all(r0 % 256 == 0 for r0, _ in b)
