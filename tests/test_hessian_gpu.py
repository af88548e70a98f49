"""Hessian accumulation kernel (through the C ABI) against a float64 accumulation.
Tolerance: 1e-5 relative (max-abs error over max-abs value, and relative Frobenius norm)."""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _rel(got: np.ndarray, want: np.ndarray):
    return np.abs(got - want).max() / np.abs(want).max(), np.linalg.norm(got - want) / np.linalg.norm(want)


@pytest.mark.parametrize("tokens,hidden", [(64, 128), (100, 256), (1, 64), (333, 1000), (2048, 512), (4096, 1024), (16384, 256),
                                           (70000, 256)])
def test_hessian_matches_float64(tokens, hidden):
    from wush_b200.hessian import accumulate_hessian
    dev = torch.device("cuda:0")
    x = synth.activations(tokens, hidden, seed=tokens + hidden)
    h0 = torch.randn(hidden, hidden, generator=torch.Generator().manual_seed(1), dtype=torch.float32)
    h0 = (h0 + h0.T) * 3.0
    h = h0.clone().to(dev)
    out = accumulate_hessian(h, x.to(dev))
    torch.cuda.synchronize()
    assert out.data_ptr() == h.data_ptr()
    want = h0.double().numpy() + wo.hessian_xtx(synth.bf16_to_f64(x))
    emax, efro = _rel(h.cpu().double().numpy(), want)
    assert emax <= TOL and efro <= TOL, (emax, efro)
    got = h.cpu().numpy()
    assert np.array_equal(got, got.T)          # the upper triangle is an exact mirror


def test_two_calls_and_lower_only():
    from wush_b200.hessian import accumulate_hessian
    dev = torch.device("cuda:0")
    hidden = 384
    xs = [synth.activations(256, hidden, seed=s) for s in (3, 4)]
    h = torch.zeros(hidden, hidden, device=dev)
    for x in xs:
        accumulate_hessian(h, x.to(dev))
    want = sum(wo.hessian_xtx(synth.bf16_to_f64(x)) for x in xs)
    emax, efro = _rel(h.cpu().double().numpy(), want)
    assert emax <= TOL and efro <= TOL
    # lower only: strict upper triangle keeps its previous content
    h2 = torch.full((hidden, hidden), 7.0, device=dev)
    accumulate_hessian(h2, xs[0].to(dev), save_lower_only=True)
    got = h2.cpu().double().numpy()
    iu = np.triu_indices(hidden, 1)
    assert (got[iu] == 7.0).all()
    il = np.tril_indices(hidden)
    w = 7.0 + wo.hessian_xtx(synth.bf16_to_f64(xs[0]))
    assert np.abs(got[il] - w[il]).max() <= TOL * np.abs(w).max()


def test_meta_batch_and_errors():
    from wush_b200.hessian import accumulate_hessian
    dev = torch.device("cuda:0")
    x = torch.stack([synth.activations(128, 128, seed=s) for s in (5, 6)]).to(dev)
    h = torch.zeros(2, 128, 128, device=dev)
    accumulate_hessian(h, x)
    for b in range(2):
        want = wo.hessian_xtx(synth.bf16_to_f64(x[b].cpu()))
        assert _rel(h[b].cpu().double().numpy(), want)[0] <= TOL
    with pytest.raises(Exception):
        accumulate_hessian(h.cpu(), x.cpu())
    with pytest.raises(NotImplementedError):
        accumulate_hessian(h, x.half())


def _tf32(x: np.ndarray, mode: str) -> np.ndarray:
    """float32 values reduced to TF32's 10 mantissa bits, by truncation or round-to-nearest-even."""
    b = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    if mode == "trunc":
        b = b & 0xFFFFE000
    else:
        b = (b + 0xFFF + ((b >> 13) & 1)) & 0xFFFFE000
    return b.astype(np.uint32).view(np.float32).astype(np.float64)


@pytest.mark.parametrize("tokens,hidden", [(300, 256), (2048, 1024), (40000, 128)])
def test_hessian_fp32_input_uses_tf32_products(tokens, hidden):
    """fp32 activations (what the reference's WUSH.update passes): TF32 products, fp32 accumulation.  Checked
    loosely against the exact float64 result (TF32 keeps 10 mantissa bits) and tightly against a float64
    accumulation of TF32-reduced inputs."""
    from wush_b200.hessian import accumulate_hessian
    dev = torch.device("cuda:0")
    x = synth.activations(tokens, hidden, seed=7, dtype=torch.float32) * 0.37     # not bf16-representable
    h = torch.zeros(hidden, hidden, device=dev)
    accumulate_hessian(h, x.to(dev))
    torch.cuda.synchronize()
    got = h.cpu().double().numpy()
    x64 = x.double().numpy()
    exact = x64.T @ x64
    assert np.abs(got - exact).max() <= 2e-3 * np.abs(exact).max()
    errs = []
    for mode in ("trunc", "rne"):
        xt = _tf32(x.numpy(), mode)
        ref = xt.T @ xt
        errs.append(np.abs(got - ref).max() / np.abs(ref).max())
    assert min(errs) <= 2e-5, errs
    assert np.array_equal(got, got.T)
