"""Parity at the configurations the benchmark times, through the production entry points.

The oracle cannot process the full tensors in seconds, so each case runs the kernel on the full benchmark
shape and compares sampled rows / columns / blocks with the oracle:
  * fused transform + quantize, 16384 x 14336, MXFP4 and NVFP4: codes and scale bytes of sampled rows,
    bit-exact except rounding-boundary ties (at most 1e-4 of the elements);
  * FP4 GEMM at 8192^3 and at (M, N, K) = (8192, 4096, 14336): operands quantized by the kernel, their sampled
    rows checked against the oracle quantizer, the sampled outputs within 1e-2 relative Frobenius of the oracle;
  * Hessian, 262144 tokens (8 launches) x 4096 channels and 32768 x 14336: sampled 256 x 256 blocks within 1e-5
    of a float64 accumulation.
"""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo
from tests.util import canon_codes, mismatch_fraction, np_u8

pytestmark = pytest.mark.gpu
TIE_BUDGET = 1e-4
DEV = "cuda:0"


def _sample_rows(rows: int, n: int) -> np.ndarray:
    fixed = [0, 1, 31, 32, 127, 128, rows - 129, rows - 1]
    rng = np.random.default_rng(rows)
    extra = rng.choice(rows, size=n - len(fixed), replace=False)
    return np.unique(np.concatenate([np.array(fixed), extra]))


@pytest.mark.parametrize("fmt", ["mx", "nv"])
def test_quantize_at_benchmark_shape(fmt):
    from wush_b200 import qutlass_ops as ops
    rows, cols = 16384, 14336
    g = 32 if fmt == "mx" else 16
    name = "mxfp4" if fmt == "mx" else "nvfp4"
    x = synth.activations(rows, cols, seed=100)
    mat = synth.wush_matrix(cols, g)
    xd, md = x.to(DEV), synth.to_bf16_tensor(mat).to(DEV)
    if fmt == "mx":
        q, sf, _ = ops.fused_quantize_mx_wush_op(xd, md, "abs_max", False)
    else:
        q, sf = ops.fused_quantize_nv_op(xd, md, torch.tensor([10.0], device=DEV))
    torch.cuda.synchronize()
    assert q.shape == (rows, cols // 2) and sf.shape == (rows, cols // g)
    idx = _sample_rows(rows, 96)
    ref = wo.fused_transform_quant(synth.bf16_to_f64(x[idx]), mat, name)
    keep = ~np.isnan(ref["fake_quant"]).any(axis=1)          # NVFP4: the reference's E4M3 cast overflows to NaN
    assert keep.sum() >= len(idx) // 2
    t = torch.from_numpy(idx).to(DEV)
    got_q, got_s = np_u8(q[t]), np_u8(sf[t])
    assert mismatch_fraction(canon_codes(got_q[keep]), canon_codes(ref["e2m1"][keep])) <= TIE_BUDGET
    assert mismatch_fraction(got_s[keep], ref["scale_quant"][keep]) <= TIE_BUDGET


@pytest.mark.parametrize("fmt", ["mx", "nv"])
@pytest.mark.parametrize("rows,cols", [(1, 32), (16, 64), (127, 256), (129, 4096), (1024, 4096), (33, 14336), (2048, 8192)])
@pytest.mark.parametrize("kind", ["wush", "hadamard"])
@pytest.mark.parametrize("blocked", [False, True])
def test_production_and_validation_kernels_emit_identical_bytes(fmt, rows, cols, kind, blocked):
    """The parity grid of test_fused_quantize_gpu.py runs the validation instantiation (which also stores the
    transformed values); the production instantiation must produce the same codes and scale bytes."""
    from wush_b200 import qutlass_ops as ops
    g = 32 if fmt == "mx" else 16
    x = synth.activations(rows, cols, seed=rows + cols).to(DEV)
    mat_np = synth.hadamard_matrix(g) if kind == "hadamard" else synth.wush_matrix(cols, g)
    mat = synth.to_bf16_tensor(mat_np).to(DEV)
    gs = torch.tensor([10.0], device=DEV) if fmt == "nv" else None
    layout = 1 if blocked else 0
    for rb in (False, True):
        q0, s0 = ops._quantize(x, mat, fmt, gs, sf_layout=layout, round_bf16=rb)
        q1, s1, _ = ops.fused_quantize_debug(x, mat, fmt, gs, round_bf16=rb, sf_layout=layout)
        assert torch.equal(q0, q1)
        assert torch.equal(s0, s1)


@pytest.mark.parametrize("m,n,k", [(8192, 8192, 8192), (8192, 4096, 14336)])
def test_gemm_at_benchmark_shapes(m, n, k):
    from wush_b200 import _lib
    from wush_b200 import qutlass_ops as ops
    had_np = synth.hadamard_matrix(32)
    had = synth.to_bf16_tensor(had_np).to(DEV)
    x = synth.activations(m, k, seed=7)
    w = synth.weights(n, k, seed=8)
    xq, xs = ops._quantize(x.to(DEV), had, "mx", None)
    wq, ws = ops._quantize(w.to(DEV), had, "mx", None)
    alpha = torch.tensor([1.0 / 9.0], device=DEV)
    y = ops.matmul_fp4_blocked(xq, wq, ops.to_blocked(xs).view(-1), ops.to_blocked(ws).view(-1), alpha, "mx")
    torch.cuda.synchronize()
    ra, rb = _sample_rows(m, 40), _sample_rows(n, 56)
    ta, tb = torch.from_numpy(ra).to(DEV), torch.from_numpy(rb).to(DEV)
    a_q, a_s = np_u8(xq[ta]), np_u8(xs[ta])[:, : k // 32]
    b_q, b_s = np_u8(wq[tb]), np_u8(ws[tb])[:, : k // 32]
    # the operands are what the oracle quantizer produces for these rows
    for q, s, src, idx in ((a_q, a_s, x, ra), (b_q, b_s, w, rb)):
        ref = wo.fused_transform_quant(synth.bf16_to_f64(src[idx]), had_np, "mxfp4")
        assert mismatch_fraction(canon_codes(q), canon_codes(ref["e2m1"])) <= TIE_BUDGET
        assert mismatch_fraction(s, ref["scale_quant"]) <= TIE_BUDGET
    want = wo.fp4_gemm(a_q, a_s, b_q, b_s, 1.0 / 9.0, "mxfp4")
    got = y[ta][:, tb].double().cpu().numpy()
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()      # one bf16 rounding of an exact fp32 sum
    del _lib


@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("m", [1, 16, 128])
def test_gemm_at_decoder_layer_shapes_small_m(n, k, m):
    """The decode shapes: few output tiles, so the K range is split over the CTAs of a cluster.  All outputs against
    the oracle, also for a forced split through a workspace (the two-kernel path)."""
    from wush_b200 import qutlass_ops as ops
    gen = torch.Generator().manual_seed(n + k + m)
    aq = torch.randint(0, 256, (m, k // 2), generator=gen, dtype=torch.uint8)
    bq = torch.randint(0, 256, (n, k // 2), generator=gen, dtype=torch.uint8)
    asf = torch.randint(122, 130, (m, k // 32), generator=gen, dtype=torch.uint8)
    bsf = torch.randint(118, 126, (n, k // 32), generator=gen, dtype=torch.uint8)
    alpha = torch.tensor([1.0 / 9.0], device=DEV)
    xb, wb = ops.to_blocked(asf.to(DEV)).view(-1), ops.to_blocked(bsf.to(DEV)).view(-1)
    y = ops.matmul_fp4_blocked(aq.to(DEV), bq.to(DEV), xb, wb, alpha, "mx")
    y2 = ops.matmul_fp4_blocked(aq.to(DEV), bq.to(DEV), xb, wb, alpha, "mx", splits=2)
    torch.cuda.synchronize()
    want = wo.fp4_gemm(aq.numpy(), asf.numpy(), bq.numpy(), bsf.numpy(), 1.0 / 9.0, "mxfp4")
    got = y.double().cpu().numpy()
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()
    got2 = y2.double().cpu().numpy()
    assert np.linalg.norm(got2 - want) <= 1e-2 * np.linalg.norm(want)
    assert np.abs(got2 - got).max() <= 2.0 ** -7 * np.abs(want).max()


def _gpu_activations(tokens: int, hidden: int, seed: int) -> torch.Tensor:
    """The benchmark's calibration activations: N(0,1) with 0.5 % outlier channels x 50, generated on the device in
    slices."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    outl = synth.outlier_channels(hidden).to(DEV)
    x = torch.empty(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    for r0 in range(0, tokens, 16384):
        blk = torch.randn(min(16384, tokens - r0), hidden, generator=g, device=DEV, dtype=torch.float32)
        blk[:, outl] *= 50.0
        x[r0:r0 + blk.shape[0]] = blk.to(torch.bfloat16)
    return x


@pytest.mark.parametrize("tokens,hidden,blocks", [(262144, 4096, [(0, 0), (15, 0), (7, 3), (15, 15), (9, 9)]),
                                                  (32768, 14336, [(0, 0), (55, 0), (55, 55), (31, 17)])])
def test_hessian_at_benchmark_shapes(tokens, hidden, blocks):
    from wush_b200.hessian import DistributedHessian
    x = _gpu_activations(tokens, hidden, seed=200)
    dh = DistributedHessian(hidden, torch.device(DEV))
    dh.accumulate_overlapped(x)
    h = dh.finalize()
    torch.cuda.synchronize()
    assert dh.num_samples == tokens
    scale_ref = None
    for bi, bj in blocks:
        xi = x[:, bi * 256:(bi + 1) * 256].double().cpu().numpy()
        xj = x[:, bj * 256:(bj + 1) * 256].double().cpu().numpy()
        want = xi.T @ xj / tokens
        got = h[bi * 256:(bi + 1) * 256, bj * 256:(bj + 1) * 256].double().cpu().numpy()
        scale_ref = max(scale_ref or 0.0, float(np.abs(want).max()))
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max(), (bi, bj)
        assert np.linalg.norm(got - want) <= 1e-5 * np.linalg.norm(want), (bi, bj)
        mirror = h[bj * 256:(bj + 1) * 256, bi * 256:(bi + 1) * 256].double().cpu().numpy()
        assert np.array_equal(mirror, got.T)


def test_bounded_wait_reports_through_the_status_word():
    """A kernel whose wait runs out returns by itself and sets the status word; the host turns that into an
    exception at its next check.  The barrier of the self-test kernel is one nothing arrives on."""
    from wush_b200 import _lib
    lib = _lib.load()
    dev = torch.device(DEV)
    _lib.check_status(dev)                                   # clean to begin with
    word = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.wush_selftest_bounded_wait(word.data_ptr(), 1000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    with pytest.raises(_lib.WushB200Error, match="timed out"):
        _lib.check_status(dev, "self-test")
    _lib.check_status(dev)                                   # the check cleared the word
    assert int(word.item()) == 0
    # the context is intact: an ordinary kernel still runs
    from wush_b200.hessian import accumulate_hessian
    h = torch.zeros(128, 128, device=dev)
    accumulate_hessian(h, synth.activations(64, 128, seed=1).to(dev))
    assert torch.isfinite(h).all()
