"""Decoder block with column-sharded W4A4 linears (wush_b200/block.py).

Single GPU: the block against a plain restatement of the same arithmetic (dequantized codes, fp32 matmuls, torch
attention).  Two GPUs: the sharded block must reproduce the single-GPU block's output (1e-2 relative Frobenius;
the only differences are the order in which the row norms are summed and bf16 roundings that follow from it).
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEQ, TOKENS = 128, 512


def _setup(fmt, dev):
    from wush_b200.block import BlockConfig, quantize_block_weights
    cfg = BlockConfig(hidden=1024, n_heads=8, n_kv_heads=2, ffn=1536, head_dim=128, fmt=fmt)
    kv = cfg.n_kv_heads * cfg.head_dim
    shapes = {"q": (1024, 1024), "k": (kv, 1024), "v": (kv, 1024), "o": (1024, 1024), "gate": (1536, 1024),
              "up": (1536, 1024), "down": (1024, 1536)}
    weights = {n: synth.weights(*s, seed=100 + i) for i, (n, s) in enumerate(shapes.items())}
    g = cfg.group
    transforms = {"attn_in": synth.to_bf16_tensor(synth.wush_matrix(1024, g, seed=11)),
                  "o": synth.to_bf16_tensor(synth.hadamard_matrix(g)),
                  "mlp_in": synth.to_bf16_tensor(synth.wush_matrix(1024, g, seed=12)),
                  "down": synth.to_bf16_tensor(synth.wush_matrix(1536, g, seed=13))}
    gammas = tuple((1.0 + 0.1 * torch.randn(1024, generator=torch.Generator().manual_seed(s))).to(torch.bfloat16) for s in (1, 2))
    qw = quantize_block_weights(cfg, weights, transforms, dev)
    h = (synth.activations(TOKENS, 1024, seed=5).float() * 0.1).to(torch.bfloat16)
    return cfg, qw, transforms, gammas, h


def _reference_forward(cfg, qw, transforms, gammas, h, dev):
    """The same block from separate steps: quantize + dequantize the layer input (kernel output -> float), fp32
    matmul with the dequantized weights, bf16 roundings where the layers round."""
    from wush_b200 import qutlass_ops as ops
    from wush_b200.gptq import dequantize
    name = "mxfp4" if cfg.fmt == "mx" else "nvfp4"
    gsv = 3.0 if cfg.fmt == "mx" else 10.0
    gs = torch.tensor([10.0], device=dev) if cfg.fmt == "nv" else None

    def linear(x, t, wname):
        q, sf = ops._quantize(x.contiguous(), t.to(dev), cfg.fmt, gs)
        xd = dequantize(q, sf[: x.shape[0], : x.shape[1] // cfg.group], name)
        wq, ws = qw[wname]
        wd = dequantize(wq, ws, name)
        # dequantize() divides by the format's tensor scale; the layer's alpha is 1 / (w_scale * a_scale)
        fix = 1.0 if cfg.fmt == "nv" else (3.0 * 3.0) / (gsv * gsv)
        return ((xd @ wd.t()) * fix).to(torch.bfloat16)

    def norm(x, gamma):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)).to(torch.bfloat16) * gamma.to(dev)

    h = h.to(dev).clone()
    x = norm(h, gammas[0])
    q, k, v = (linear(x, transforms["attn_in"], n) for n in ("q", "k", "v"))
    b, d = TOKENS // SEQ, cfg.head_dim
    sh = lambda t, nh: t.view(b, SEQ, nh, d).transpose(1, 2)
    o = F.scaled_dot_product_attention(sh(q, cfg.n_heads), sh(k, cfg.n_kv_heads), sh(v, cfg.n_kv_heads), is_causal=True,
                                       enable_gqa=True)
    h = linear(o.transpose(1, 2).reshape(TOKENS, -1), transforms["o"], "o") + h
    x = norm(h, gammas[1])
    act = F.silu(linear(x, transforms["mlp_in"], "gate")) * linear(x, transforms["mlp_in"], "up")
    return linear(act, transforms["down"], "down") + h


@pytest.mark.parametrize("fmt", ["mx", "nv"])
def test_block_matches_stepwise_reference(fmt):
    from wush_b200.block import ShardedDecoderBlock
    dev = torch.device("cuda:0")
    cfg, qw, transforms, gammas, h = _setup(fmt, dev)
    want = _reference_forward(cfg, qw, transforms, gammas, h, dev).float()
    for mbs in (1, 2):
        blk = ShardedDecoderBlock(cfg, qw, transforms, gammas, SEQ, TOKENS, dev, micro_batches=mbs)
        got = blk.forward(h.to(dev).clone()).float()
        torch.cuda.synchronize()
        rel = float((got - want).norm() / want.norm())
        assert rel <= 1e-2, (fmt, mbs, rel)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wush_b200.block import ShardedDecoderBlock
    cfg, qw, transforms, gammas, h = _setup("mx", dev)
    blk = ShardedDecoderBlock(cfg, qw, transforms, gammas, SEQ, TOKENS, dev, micro_batches=2)
    hs = cfg.hidden // world
    mine = h[:, rank * hs:(rank + 1) * hs].contiguous().to(dev)
    first = blk.forward(mine.clone()).clone()
    again = blk.forward(mine.clone())                      # the buffers are reused: same bits the second time
    torch.cuda.synchronize()
    assert torch.equal(first, again)
    gathered = [torch.empty_like(first) for _ in range(world)]
    dist.all_gather(gathered, first)
    if rank == 0:
        np.save(out, torch.cat(gathered, dim=1).float().cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("broadcast", ["0", "1"])
def test_two_gpu_block_matches_single_gpu_block(tmp_path, monkeypatch, broadcast):
    """broadcast "0": slots travel as one device-to-device copy per peer; "1": by the one-launch broadcast kernel
    (through the multicast address where the GPUs have one).  The spawned ranks inherit the environment."""
    import torch.multiprocessing as mp
    from wush_b200.block import ShardedDecoderBlock
    monkeypatch.setenv("WUSH_B200_BLOCK_BROADCAST", broadcast)
    out = str(tmp_path / "h.npy")
    mp.spawn(_worker, args=(2, 29950 + (os.getpid() + int(broadcast) * 150) % 300, out), nprocs=2, join=True)
    got = np.load(out)
    dev = torch.device("cuda:0")
    cfg, qw, transforms, gammas, h = _setup("mx", dev)
    # world size 1 here: no process group is initialised in the test process
    want = ShardedDecoderBlock(cfg, qw, transforms, gammas, SEQ, TOKENS, dev, micro_batches=1).forward(h.to(dev).clone())
    want = want.float().cpu().numpy()
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)


def test_peer_broadcast_kernel_plain_stores_on_one_gpu():
    """The one-launch delivery of a slot to several destination buffers, exercised with destinations on the same GPU
    (the plain-store form; the multicast form needs an NVSwitch multicast address and is covered by the 2-GPU block
    test with WUSH_B200_BLOCK_BROADCAST=1)."""
    import ctypes
    from wush_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    src = torch.randint(0, 256, ((1 << 20) + 48,), dtype=torch.uint8, device=dev)[:(1 << 20) + 32]
    dsts = [torch.zeros_like(src) for _ in range(3)]
    table = (ctypes.c_void_p * 3)(*[d.data_ptr() for d in dsts])
    rc = lib.wush_peer_broadcast(src.data_ptr(), None, table, 3, src.numel(), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert all(torch.equal(d, src) for d in dsts)
    assert lib.wush_peer_broadcast(src.data_ptr(), None, table, 3, 24, None) == -2          # not a multiple of 16
    assert lib.wush_peer_broadcast(src.data_ptr() + 4, None, table, 3, 32, None) == -3      # alignment
    assert lib.wush_peer_broadcast(src.data_ptr(), None, table, 0, 32, None) == 0           # nobody to deliver to
