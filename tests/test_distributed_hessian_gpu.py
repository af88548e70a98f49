"""Token-sharded Hessian over NCCL on 2 GPUs (skipped on a single-GPU box), and the single-GPU path of
the same class against a float64 accumulation."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_gpu_update_and_overlapped():
    from wush_b200.hessian import DistributedHessian
    dev = torch.device("cuda:0")
    hidden = 640
    xs = [synth.activations(t, hidden, seed=60 + i) for i, t in enumerate((2048, 100, 1500))]
    want = wo.wush_update_sequence([synth.bf16_to_f64(x) for x in xs])
    a = DistributedHessian(hidden, dev)
    for x in xs:
        a.update(x.to(dev)[None])
    ha = a.finalize().double().cpu().numpy()
    b = DistributedHessian(hidden, dev, panels=3)
    b.accumulate_overlapped(torch.cat(xs).to(dev))
    hb = b.finalize().double().cpu().numpy()
    for h in (ha, hb):
        assert np.abs(h - want).max() <= 1e-5 * np.abs(want).max()
        assert np.array_equal(h, h.T)
    assert a.num_samples == b.num_samples == 3648


def test_update_staging_matches_direct_launches():
    """Short updates are staged and flushed by capacity, by a long input, by a dtype change and by finalize();
    the result must equal launching on every call."""
    from wush_b200.hessian import DistributedHessian
    dev = torch.device("cuda:0")
    hidden = 512
    sizes = (300, 300, 300, 200, 2000, 17, 300)          # capacity 1000: overflow, then a long input, then a tail
    xs = [synth.activations(t, hidden, seed=80 + i).to(dev) for i, t in enumerate(sizes)]
    staged = DistributedHessian(hidden, dev, stage_tokens=1000)
    direct = DistributedHessian(hidden, dev, stage_tokens=0)
    launches = []
    inner = staged._accumulate
    staged._accumulate = lambda h, x, *a: (launches.append(x.shape[0]), inner(h, x, *a))[1]
    for x in xs:
        staged.update(x)
        direct.update(x)
    hs, hd = staged.finalize(), direct.finalize()
    assert launches == [900, 200, 2000, 317]
    assert staged.num_samples == direct.num_samples == sum(sizes)
    assert (hs - hd).abs().max() <= 1e-6 * hd.abs().max()
    want = wo.wush_update_sequence([synth.bf16_to_f64(x.cpu()) for x in xs])
    assert np.abs(hs.double().cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    # fp32 inputs share the class (TF32 products): staged and direct agree to TF32 accuracy
    f = DistributedHessian(hidden, dev)
    for x in xs[:3]:
        f.update(x.float())
    hf = f.finalize().double().cpu().numpy()
    w3 = wo.wush_update_sequence([synth.bf16_to_f64(x.cpu()) for x in xs[:3]])
    assert np.linalg.norm(hf - w3) <= 2e-3 * np.linalg.norm(w3)


def _worker(rank, world, port, out, peer, multimem, per_panel, tokens0, kernel_barrier):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      WUSH_B200_HESSIAN_PEER="1" if peer else "0", WUSH_B200_HESSIAN_MULTIMEM="1" if multimem else "0",
                      WUSH_B200_HESSIAN_TILES_PER_PANEL=str(per_panel),
                      WUSH_B200_HESSIAN_KERNEL_BARRIER="1" if kernel_barrier else "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wush_b200.hessian import DistributedHessian
    x = synth.activations(tokens0 + 256 * rank, 1024, seed=70 + rank).to(dev)
    dh = DistributedHessian(1024, dev, panels=4)
    assert (dh._peer is not None) == peer
    if peer and rank == 0:
        print(f"multicast address available: {bool(dh._peer.mc_ptr)} (asked for: {multimem})", flush=True)
    dh.accumulate_overlapped(x)
    h = dh.finalize()
    torch.cuda.synchronize()
    assert dh.num_samples == sum(tokens0 + 256 * r for r in range(world))
    # every rank must hold the same bits
    mine = h.clone()
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(mine, ref)
    if rank == 0:
        np.save(out, h.cpu().numpy())
    dh.release()
    # second job on the pooled buffer (update path: one combine over the whole tile list)
    dh2 = DistributedHessian(1024, dev)
    dh2.update(x[:512])
    dh2.update(x[512:])
    h2 = dh2.finalize()
    torch.cuda.synchronize()
    assert (h2 - mine).abs().max() <= 1e-5 * mine.abs().max()
    assert torch.equal(h2, h2.t())
    dh2.release()
    # third job: the same tokens again must reproduce the first result bit for bit (no state left in the pool)
    dh3 = DistributedHessian(1024, dev, panels=4)
    dh3.accumulate_overlapped(x)
    h3 = dh3.finalize()
    torch.cuda.synchronize()
    if tokens0 <= 32768:
        assert torch.equal(h3, mine)
    else:
        # launches that add to an existing sum may split the tokens and combine the splits with atomic adds
        assert (h3 - mine).abs().max() <= 1e-6 * mine.abs().max()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("peer,multimem,per_panel,tokens0,kernel_barrier",
                         [(True, True, 0, 1024, True), (True, False, 3, 1024, True), (True, True, 4, 50000, True),
                          (True, True, 3, 1024, False), (False, False, 0, 1024, True)])
def test_two_gpu_hessian(tmp_path, peer, multimem, per_panel, tokens0, kernel_barrier):
    """peer=True: ranks combined by the reduce kernel over NVLink (multimem: sums formed inside the NVSwitch when
    a multicast address is available; per_panel > 0: the tile list is combined in several overlapped panels;
    50000 tokens: two 32768-token segments per rank; kernel_barrier: the reduce and mirror kernels run the cross-rank
    barriers themselves instead of separate barrier kernels); peer=False: NCCL all-reduce of row panels."""
    import torch.multiprocessing as mp
    out = str(tmp_path / "h.npy")
    port = 29650 + os.getpid() % 300 + 7 * per_panel + (3 if multimem else 0) + (1 if kernel_barrier else 0)
    mp.spawn(_worker, args=(2, port, out, peer, multimem, per_panel, tokens0, kernel_barrier), nprocs=2, join=True)
    got = np.load(out).astype(np.float64)
    want = wo.wush_update_sequence([synth.bf16_to_f64(synth.activations(tokens0 + 256 * r, 1024, seed=70 + r)) for r in range(2)])
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    assert np.array_equal(got, got.T)


def test_layers_on_the_second_gpu_of_one_process():
    """One process driving two GPUs (layers placed on cuda:0 and cuda:1): the kernels' shared-memory opt-in and
    cluster occupancy are per device, so the first launch on the second device must set them up again."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from wush_b200 import qutlass_ops as ops
    from wush_b200.hessian import accumulate_hessian
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        x = synth.activations(300, 512, seed=3).to(dev)
        had = synth.to_bf16_tensor(synth.hadamard_matrix(32)).to(dev)
        q, sf = ops._quantize(x, had, "mx", None, sf_layout=1)
        wq, wsf = ops._quantize(synth.weights(256, 512, seed=4).to(dev), had, "mx", None, sf_layout=1)
        y = ops.matmul_fp4_blocked(q, wq, sf.view(-1), wsf.view(-1), torch.tensor([1 / 9.0], device=dev), "mx")
        y16 = ops.matmul_fp4_blocked(q[:16], wq, sf.view(-1), wsf.view(-1), torch.tensor([1 / 9.0], device=dev), "mx")
        h = accumulate_hessian(torch.zeros(512, 512, device=dev), x)
        torch.cuda.synchronize(dev)
        outs.append((q.cpu(), y.cpu(), y16.cpu(), h.cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
