"""Column sweep on the GPU (wush_b200.gptq) against the oracle's restatement of the reference's
gptq_babai_outer, and against the vectors the reference itself produced."""
import os

import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "sweep_vectors.npz"))
_ADJACENT = {(a, b) for a in range(16) for b in range(16) if (a & 8) == (b & 8) and abs((a & 7) - (b & 7)) == 1}


def _run(w64, h64, fmt, tt, rtn, transforms=None):
    from wush_b200 import gptq
    dev = torch.device("cuda:0")
    w = torch.from_numpy(w64).to(torch.bfloat16).to(dev)
    h = torch.from_numpy(h64).to(torch.float32).to(dev)
    t = None if transforms is None else torch.from_numpy(transforms).to(dev)
    out = gptq.gptq_babai_sweep(w, h, fmt, tt, force_rtn=rtn, transforms=t)
    torch.cuda.synchronize()
    return {
        "qweight": out["qweight"].cpu().numpy(),
        "scale_quant": out["scale_quant"].view(torch.uint8).cpu().numpy(),
        "fake_quant": out["fake_quant"].float().cpu().numpy(),
        "transform_basis": out["transform_basis"].float().cpu().numpy(),
    }


def _compare_codes(got, want, allow_ties):
    c0, c1 = wo.unpack_e2m1_codes(got), wo.unpack_e2m1_codes(want)
    bad = np.argwhere(c0 != c1)
    if not allow_ties:
        assert len(bad) <= 1e-4 * c0.size, f"{len(bad)} of {c0.size} codes differ"
    else:
        assert len(bad) <= 0.005 * c0.size
    assert all((int(c0[tuple(i)]), int(c1[tuple(i)])) in _ADJACENT for i in bad)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("tt", ["identity", "hadamard", "wush"])
@pytest.mark.parametrize("rtn", [True, False])
def test_sweep_matches_reference_vectors(fmt, tt, rtn):
    """Same inputs as the reference run; its transforms are fed back so that the comparison does not depend
    on the sign convention of an SVD."""
    tag = f"{fmt}_{tt}_{'rtn' if rtn else 'gptq'}"
    got = _run(GOLD[f"{fmt}_w"], GOLD[f"{fmt}_h"], fmt, tt, rtn, transforms=GOLD[tag + "_transform"])
    assert np.array_equal(got["scale_quant"], GOLD[tag + "_scale"])
    _compare_codes(got["qweight"], GOLD[tag + "_e2m1"], allow_ties=(tt == "identity"))
    if tt != "identity":
        want_fake = torch.from_numpy(GOLD[tag + "_fake"]).to(torch.bfloat16).float().numpy()
        assert np.array_equal(got["fake_quant"], want_fake)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("rtn", [True, False])
def test_sweep_own_transforms_against_oracle(fmt, rtn):
    """Larger layer, transforms computed on the GPU: the oracle re-runs the sweep with exactly those
    matrices (codes and scales must agree), and every matrix must be a valid WUSH transform of its block:
    T basis^T (T basis^T)^T = Had diag(s) Had^T, which does not depend on the signs of the singular vectors."""
    g = wo.FORMATS[fmt]["group"]
    c, r = 256, 192
    x = synth.bf16_to_f64(synth.activations(1024, c, seed=91))
    h = x.T @ x / x.shape[0]
    w = synth.bf16_to_f64(synth.weights(r, c, seed=92))
    got = _run(w, h.astype(np.float32).astype(np.float64), fmt, "wush", rtn)
    t_gpu = got["transform_basis"].astype(np.float64)
    seen = {}

    def feed(b, basis, y):
        seen[b] = (basis, y)
        return t_gpu[b]

    want = wo.gptq_babai_outer(w, h.astype(np.float32).astype(np.float64), fmt, "wush", rtn, transform_fn=feed)
    assert np.array_equal(got["scale_quant"], want["scale_quant"])
    _compare_codes(got["qweight"], want["e2m1"], allow_ties=False)
    had = wo.normalized_hadamard(g)
    for b, (basis, y) in seen.items():
        s = np.linalg.svd(y, compute_uv=False) * y.shape[1] ** -0.5
        s = s + s.mean() * 1e-2
        m = t_gpu[b] @ basis.T
        ref = (had * s) @ had.T
        assert np.abs(m @ m.T - ref).max() <= 2e-2 * np.abs(ref).max()      # T is rounded to bf16


def test_quantize_layers_splits_and_layers_run():
    """quantize_layers keeps the reference's return structure and the pseudo-quantized layers reproduce the
    original layer's output up to the quantization error."""
    from wush_b200 import gptq
    dev = torch.device("cuda:0")
    c = 256
    xs = synth.activations(2048, c, seed=93).to(dev)
    h = (xs.float().T @ xs.float()) / xs.shape[0]
    w1, w2 = synth.weights(64, c, seed=94).to(dev), synth.weights(96, c, seed=95).to(dev)
    layers, results = gptq.quantize_layers(w1, w2, hessian=h, quant_type="mxfp4", transform_class="wush")
    assert [r["qweight"].shape for r in results] == [(64, c // 2), (96, c // 2)]
    assert [r["scale_quant"].shape for r in results] == [(64, c // 32), (96, c // 32)]
    assert results[0]["scale_quant"].dtype == torch.float8_e8m0fnu and results[0]["global_scale"] == 3.0
    assert results[0]["transform_basis"].shape == (c // 32, 32, 32)
    xt = synth.activations(128, c, seed=96).to(dev)
    for layer, w in zip(layers, (w1, w2)):
        y, want = layer(xt).float(), xt.float() @ w.float().T
        rel = (y - want).norm() / want.norm()
        assert rel < 0.2, rel


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_prepare_kernel_matches_torch_linear_algebra(fmt):
    """wush_gptq_block_prepare against the same algebra done with torch.linalg in float64 (gptq.get_transform,
    torch.linalg.qr): transforms equal up to the bf16 rounding of a few entries, R^T R = M^T M, Q^T orthogonal
    and Q^T M = R."""
    from wush_b200 import _lib, gptq
    dev = torch.device("cuda:0")
    g = wo.FORMATS[fmt]["group"]
    nb, rows = 6, 320
    gen = torch.Generator(device=dev).manual_seed(5)
    m = torch.randn(nb, g, g, generator=gen, device=dev, dtype=torch.float64)
    basis = torch.linalg.cholesky(m @ m.transpose(-2, -1) + 0.5 * torch.eye(g, device=dev, dtype=torch.float64), upper=True).contiguous()
    y = torch.randn(nb, g, rows, generator=gen, device=dev, dtype=torch.float64) * torch.logspace(0, -2, g, device=dev, dtype=torch.float64)[None, :, None]
    y = (torch.linalg.qr(torch.randn(nb, g, g, generator=gen, device=dev, dtype=torch.float64)).Q @ y).contiguous()
    gram = (y @ y.transpose(-2, -1)).contiguous()
    tm, rn, qt = (torch.empty(nb, g, g, dtype=torch.float64, device=dev) for _ in range(3))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gptq._prepare(gram, basis, g, g * g, nb, wo.FORMATS[fmt]["group"] == 16 and _lib.FORMAT_NVFP4 or _lib.FORMAT_MXFP4,
                  "wush", False, rows, tm, rn, qt, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want_t = gptq.get_transform(basis, y, "wush", torch.bfloat16)
    # same sign convention on both sides; entries may differ by one bf16 step where the float64 values straddle a tie
    rel = (tm - want_t).abs() / want_t.abs().clamp_min(1e-3)
    assert float((rel > 2.0 ** -7).double().mean()) == 0.0
    assert float((tm != want_t).double().mean()) < 0.02
    mm = basis @ tm.transpose(-2, -1)
    eye = torch.eye(g, device=dev, dtype=torch.float64)
    assert float((qt @ qt.transpose(-2, -1) - eye).abs().max()) < 1e-12
    assert float((qt @ mm - rn).abs().max()) < 1e-11 * float(mm.abs().max())
    assert float(rn.tril(-1).abs().max()) == 0.0


def _row_shard_worker(rank, world, port, out, rtn):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from wush_b200 import gptq
    w, h = _row_shard_inputs()
    rows = w.shape[0] // world
    res = gptq.gptq_babai_sweep(w[rank * rows:(rank + 1) * rows].to(dev), h.to(dev), "mxfp4", "wush", force_rtn=rtn,
                                group=dist.group.WORLD, total_rows=w.shape[0])
    torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in res.items()}, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def _row_shard_inputs():
    x = synth.bf16_to_f64(synth.activations(2048, 256, seed=21))
    h = torch.from_numpy((x.T @ x / x.shape[0]).astype(np.float32))
    return synth.weights(512, 256, seed=22), h


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("rtn", [True, False])
def test_row_sharded_sweep_on_two_gpus_matches_the_unsharded_sweep(tmp_path, rtn):
    """Weight rows split over two GPUs; only the G x G Gram matrices of the block targets are all-reduced.  The
    transforms (same on both ranks) and each rank's codes and scales must be those of the sweep of the whole matrix
    (float64 summation order differs, which can flip a rounding-boundary case)."""
    import os
    import torch.multiprocessing as mp
    from wush_b200 import gptq
    out = str(tmp_path / "s")
    mp.spawn(_row_shard_worker, args=(2, 29400 + os.getpid() % 300 + int(rtn), out, rtn), nprocs=2, join=True)
    parts = [torch.load(f"{out}.{r}", weights_only=False) for r in range(2)]
    dev = torch.device("cuda:0")
    w, h = _row_shard_inputs()
    whole = gptq.gptq_babai_sweep(w.to(dev), h.to(dev), "mxfp4", "wush", force_rtn=rtn)
    assert torch.equal(parts[0]["transform_basis"], parts[1]["transform_basis"])
    assert float((parts[0]["transform_basis"].float() != whole["transform_basis"].cpu().float()).float().mean()) <= 1e-3
    codes = torch.cat([p["qweight"] for p in parts])
    scales = torch.cat([p["scale_quant"].view(torch.uint8) for p in parts])
    assert float((scales != whole["scale_quant"].view(torch.uint8).cpu()).float().mean()) <= 1e-3
    assert float((codes != whole["qweight"].cpu()).float().mean()) <= 2e-3
