"""Parity of the fused transform+quantize kernel (through the C ABI) with the CPU oracle.

Tolerances (stated by the task this library was built for):
  * transformed values: 1e-5 relative, in fp32;
  * FP4 codes and scale bytes: bit-exact except at rounding-boundary ties, at most 1e-4 of the
    elements may differ (codes are compared with -0 folded onto +0).
"""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo
from tests.util import canon_codes, mismatch_fraction, np_u8

pytestmark = pytest.mark.gpu

TIE_BUDGET = 1e-4
GROUP = {"mx": 32, "nv": 16}
FMT = {"mx": "mxfp4", "nv": "nvfp4"}


def _ops():
    from wush_b200 import qutlass_ops
    return qutlass_ops


def _matrix(kind: str, fmt: str, cols: int) -> np.ndarray:
    g = GROUP[fmt]
    if kind == "hadamard":
        return synth.hadamard_matrix(g)
    if kind == "identity":
        return np.eye(g)
    return synth.wush_matrix(cols, g)


def _run(fmt, x_bf16, mat_np, round_bf16=False, blocked=False):
    ops = _ops()
    dev = torch.device("cuda:0")
    x = x_bf16.to(dev)
    mat = synth.to_bf16_tensor(mat_np).to(dev)
    gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
    q, sf, tr = ops.fused_quantize_debug(x, mat, fmt, gs, round_bf16=round_bf16, sf_layout=1 if blocked else 0)
    torch.cuda.synchronize()
    return np_u8(q), np_u8(sf), tr.cpu().numpy().astype(np.float64)


def _check(fmt, x_bf16, mat_np, round_bf16=False, exact=False):
    rows, cols = x_bf16.shape
    g = GROUP[fmt]
    q, sf, tr = _run(fmt, x_bf16, mat_np, round_bf16)
    x64 = synth.bf16_to_f64(x_bf16)
    ref = wo.fused_transform_quant(x64, mat_np, FMT[fmt], round_bf16=round_bf16)
    # transformed values, 1e-5 relative to the magnitude of the terms that were summed
    t3 = wo.matrix_to_transform(np.abs(mat_np)) if mat_np.shape[1] != g else np.abs(mat_np).T
    bound = wo.block_transform(np.abs(x64), t3)
    err = np.abs(tr - ref["transformed"])
    if round_bf16:
        # one bf16 ulp where the fp32 and fp64 sums straddle a rounding boundary, rarely
        assert np.mean(err > 1e-5 * bound + 1e-30) < 1e-3
    else:
        assert np.all(err <= 1e-5 * bound + 1e-30), float((err / (bound + 1e-30)).max())
    # scales and codes against the oracle's own pipeline
    sf_valid = sf[:rows, : cols // g]
    nan_rows = np.isnan(ref["fake_quant"]).any(axis=1)
    keep = ~nan_rows
    f_scale = mismatch_fraction(sf_valid[keep], ref["scale_quant"][keep])
    f_code = mismatch_fraction(canon_codes(q[keep]), canon_codes(ref["e2m1"][keep]))
    budget = 0.0 if exact else TIE_BUDGET
    assert f_scale <= budget, f_scale
    assert f_code <= budget, f_code
    # and, stricter, the oracle quantizer applied to the kernel's own transformed values: only
    # fp32-vs-fp64 rounding of the scaled value can differ
    ref2 = wo.rtn_xxfp4(tr, FMT[fmt])
    keep2 = ~np.isnan(ref2["fake_quant"]).any(axis=1)
    assert mismatch_fraction(sf_valid[keep2], ref2["scale_quant"][keep2]) <= 1e-5
    assert mismatch_fraction(canon_codes(q[keep2]), canon_codes(ref2["e2m1"][keep2])) <= 1e-5
    return q, sf


@pytest.mark.parametrize("fmt", ["mx", "nv"])
@pytest.mark.parametrize("rows,cols", [(1, 32), (16, 64), (127, 256), (129, 4096), (1024, 4096), (33, 14336)])
@pytest.mark.parametrize("kind", ["wush", "hadamard"])
def test_parity_random(fmt, rows, cols, kind):
    x = synth.activations(rows, cols, seed=rows + cols)
    _check(fmt, x, _matrix(kind, fmt, cols))


@pytest.mark.parametrize("fmt", ["mx", "nv"])
def test_parity_round_bf16(fmt):
    x = synth.activations(300, 1024, seed=5)
    _check(fmt, x, _matrix("wush", fmt, 1024), round_bf16=True)


@pytest.mark.parametrize("fmt", ["mx", "nv"])
def test_identity_transform_is_bit_exact(fmt, golden):
    """With an identity matrix nothing is summed, so codes and scales must match the
    reference-generated edge vectors exactly (ties, zeros, tiny and huge magnitudes)."""
    g = GROUP[fmt]
    e = torch.from_numpy(golden[f"{FMT[fmt]}_edge_in"]).to(torch.bfloat16)
    reps = 64 // g                       # pad to 64 channels: cols must be a multiple of 32
    x = torch.zeros(e.shape[0], 64, dtype=torch.bfloat16)
    x[:, :g] = e
    x[:, g:2 * g] = -e
    del reps
    q, sf = _check(fmt, x, np.eye(g), exact=True)
    # all-zero groups: reference encodes scale 0 and -0 codes for MX, scale 0 and code 7 for NV
    zero_rows = np.nonzero((x == 0).all(dim=1).numpy())[0]
    for r in zero_rows:
        assert (sf[r, : 64 // g] == 0).all()
        assert (q[r] == (0x88 if fmt == "mx" else 0x77)).all()


@pytest.mark.parametrize("fmt", ["mx", "nv"])
def test_blocked_scale_layout(fmt):
    rows, cols = 200, 1024 + 32 * 3
    cols = cols // 32 * 32
    x = synth.activations(rows, cols, seed=9)
    mat = _matrix("hadamard", fmt, cols)
    _, sf_rm, _ = _run(fmt, x, mat)
    _, sf_bl, _ = _run(fmt, x, mat, blocked=True)
    g = GROUP[fmt]
    want = wo.to_blocked(sf_rm[:rows, : cols // g])
    # padding is untouched by the kernel and zero-filled by the wrapper
    assert np.array_equal(sf_bl.reshape(-1), want)
    blk = _ops().to_blocked(torch.from_numpy(sf_rm[:rows, : cols // g].copy()).cuda())
    assert np.array_equal(np_u8(blk).reshape(-1), want)


def test_public_ops_shapes_and_errors():
    ops = _ops()
    dev = torch.device("cuda:0")
    x = synth.activations(130, 4096 + 64, seed=3).to(dev)
    wm = synth.to_bf16_tensor(synth.wush_matrix(4096 + 64, 32)).to(dev)
    q, sf, mask = ops.fused_quantize_mx_wush_op(x, wm, "abs_max", False)
    assert q.shape == (130, (4096 + 64) // 2) and q.dtype == torch.uint8
    assert sf.shape == (256, 132) and sf.dtype == torch.float8_e8m0fnu and mask is None
    h = synth.to_bf16_tensor(synth.hadamard_matrix(32)).to(dev)
    q2, sf2, mask2 = ops.fused_quantize_mx_op(x, h, "abs_max", True)
    assert mask2.shape == (130, (4096 + 64) // 8) and bool((mask2 == 0xFF).all())
    h16 = synth.to_bf16_tensor(synth.hadamard_matrix(16)).to(dev)
    q3, sf3 = ops.fused_quantize_nv_op(x, h16, torch.tensor([10.0], device=dev))
    assert sf3.shape == (256, 260) and sf3.dtype == torch.float8_e4m3fn
    with pytest.raises(Exception):
        ops.fused_quantize_mx_op(x.cpu(), h.cpu(), "abs_max", False)       # no CPU fallback
    with pytest.raises(ValueError):
        ops.fused_quantize_mx_op(x, h, "median", False)
    q4, sf4, mask4 = ops.fused_quantize_mx_op(x, h, "quest", True)
    assert q4.shape == q2.shape and sf4.shape == sf2.shape and mask4.shape == mask2.shape
    assert ops.fused_quantize_mx_op(x, h, "quest", False)[2] is None
    # the per-group op has no method of its own: whatever is passed, it scales by the absolute maximum
    q5, sf5, _ = ops.fused_quantize_mx_wush_op(x, wm, "quest", False)
    assert torch.equal(q5, q) and torch.equal(sf5.view(torch.uint8), sf.view(torch.uint8))
    empty = ops.fused_quantize_mx_op(x[:0], h, "abs_max", False)
    assert empty[0].shape == (0, (4096 + 64) // 2)


def test_full_size_properties():
    """Benchmark-size run (16384 x 8192): properties that need no full oracle pass --
    determinism, row independence (a row's codes do not depend on its neighbours) and a
    dequantization error bound."""
    ops = _ops()
    dev = torch.device("cuda:0")
    rows, cols = 16384, 8192
    x = synth.activations(rows, cols, seed=21).to(dev)
    wm = synth.to_bf16_tensor(synth.wush_matrix(cols, 32)).to(dev)
    q1, s1, _ = ops.fused_quantize_mx_wush_op(x, wm, "abs_max", False)
    q2, s2, _ = ops.fused_quantize_mx_wush_op(x, wm, "abs_max", False)
    assert torch.equal(q1, q2) and torch.equal(s1.view(torch.uint8), s2.view(torch.uint8))
    idx = torch.tensor([0, 1, 127, 128, 5000, 16383], device=dev)
    q3, s3, _ = ops.fused_quantize_mx_wush_op(x[idx].contiguous(), wm, "abs_max", False)
    assert torch.equal(q3, q1[idx])
    assert torch.equal(s3.view(torch.uint8)[: len(idx)], s1.view(torch.uint8)[idx])
    # oracle on a 64-row sample
    sample = torch.arange(0, rows, rows // 64, device=dev)[:64]
    ref = wo.fused_transform_quant(synth.bf16_to_f64(x[sample].cpu()), wm.cpu().to(torch.float64).numpy(), "mxfp4")
    assert mismatch_fraction(canon_codes(np_u8(q1[sample])), canon_codes(ref["e2m1"])) <= TIE_BUDGET
    assert mismatch_fraction(np_u8(s1)[sample.cpu().numpy()][:, : cols // 32], ref["scale_quant"]) <= TIE_BUDGET


def test_host_streamed_quantize_matches_single_launch():
    """Row-chunked, three-stream pass over pinned host buffers == one launch on the device (rows are
    independent), for a row count that is not a multiple of the chunk."""
    from wush_b200 import qutlass_ops as ops
    from wush_b200.host_stream import HostQuantizer
    dev = torch.device("cuda:0")
    rows, cols = 5 * 256 + 77, 1024
    x = synth.activations(rows, cols, seed=123)
    for fmt, g in (("mx", 32), ("nv", 16)):
        mat = synth.to_bf16_tensor(synth.wush_matrix(cols, g, seed=7)).to(dev)
        gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
        q_ref, sf_ref = ops._quantize(x.to(dev), mat, fmt, gs)
        xh = x.pin_memory()
        qh = torch.empty(rows, cols // 2, dtype=torch.uint8).pin_memory()
        sh = torch.empty(rows, cols // g, dtype=torch.uint8).pin_memory()
        hq = HostQuantizer(cols, mat, fmt, gs, chunk_rows=256)
        for _ in range(2):                      # second pass reuses the staging buffers
            qh.zero_(); sh.zero_()
            hq(xh, qh, sh)
            hq.synchronize()
            assert torch.equal(qh, q_ref.cpu())
            assert torch.equal(sh, sf_ref.view(torch.uint8)[:rows, : cols // g].cpu())
        assert hq.launches == 2 * 6


def test_pseudo_quant_wrappers_match_oracle_dequantization():
    """The Triton-wrapper-compatible entry points return dequant(quant(x @ H)) of the oracle."""
    from wush_b200 import pseudo_quant as pq
    dev = torch.device("cuda:0")
    x = synth.activations(96, 512, seed=321)
    for fmt, g in (("mxfp4", 32), ("nvfp4", 16)):
        hm = synth.to_bf16_tensor(synth.hadamard_matrix(g))
        want = wo.fused_transform_quant(synth.bf16_to_f64(x), synth.bf16_to_f64(hm), fmt)["fake_quant"]
        hm = hm.to(dev)
        if fmt == "mxfp4":
            got, mask = pq.mxfp4_forward_kernel_wrapper(x.to(dev).reshape(2, 48, 512), hm, return_clip_mask=True, quest=False)
            assert mask.dtype == torch.bool and bool(mask.all()) and mask.shape == got.shape
            with pytest.raises(NotImplementedError):
                pq.mxfp4_forward_kernel_wrapper(x.to(dev), hm)          # the defaults: quest with the abs-max constant 3/4
        else:
            got = pq.nvfp4_forward_kernel_wrapper(x.to(dev).reshape(2, 48, 512), hm, torch.tensor(10.0, device=dev))
        assert got.shape == (2, 48, 512) and got.dtype == torch.bfloat16
        want_bf16 = torch.from_numpy(want).to(torch.bfloat16).float().numpy().reshape(2, 48, 512)
        bad = np.mean(got.float().cpu().numpy() != want_bf16)
        assert bad <= 1e-4, bad
    y = pq.pseudoquantize_fp(x.to(dev), "mxfp4")
    assert y.shape == x.shape


@pytest.mark.parametrize("fmt", ["mx", "nv"])
@pytest.mark.parametrize("blocked", [True, False])
def test_column_shards_assemble_the_whole_operand(fmt, blocked):
    """Quantizing column shards one by one into a wider operand (codes with a row stride, scales at a group offset)
    gives the bytes of quantizing whole rows: what every GPU of a tensor-parallel layer does for its own columns."""
    ops = _ops()
    dev = torch.device("cuda:0")
    rows, cols, shards = 333, 1024 + 256, 5
    g = GROUP[fmt]
    x = synth.activations(rows, cols, seed=31).to(dev)
    mat = synth.to_bf16_tensor(synth.wush_matrix(cols, g, seed=5)).to(dev)
    gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
    layout = 1 if blocked else 0
    q_ref, sf_ref = ops._quantize(x, mat, fmt, gs, sf_layout=layout)
    q = torch.zeros_like(q_ref)
    sf = torch.zeros_like(sf_ref)
    per = cols // shards                                      # 256 columns: a multiple of 4 groups in both formats
    for s in range(shards):
        xs = x[:, s * per:(s + 1) * per]                      # a column slice: row stride = cols
        ops.fused_quantize_into(xs, mat[:, s * per:(s + 1) * per].contiguous(), fmt, gs, q, sf, col0=s * per, sf_layout=layout)
    assert torch.equal(q, q_ref)
    assert torch.equal(sf, sf_ref)


@pytest.mark.parametrize("fmt", ["mx", "nv"])
@pytest.mark.parametrize("rows,cols", [(77, 512), (1024, 4096)])
def test_rmsnorm_folded_into_the_quantizer_is_bit_identical_to_the_separate_steps(fmt, rows, cols):
    ops = _ops()
    dev = torch.device("cuda:0")
    g = GROUP[fmt]
    x = (synth.activations(rows, cols, seed=41).float() * 0.3).to(torch.bfloat16).to(dev)
    gamma = (1.0 + 0.2 * torch.randn(cols, generator=torch.Generator().manual_seed(2))).to(torch.bfloat16).to(dev)
    mat = synth.to_bf16_tensor(synth.wush_matrix(cols, g, seed=6)).to(dev)
    gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
    ssq = ops.row_sumsq(x)
    want_ssq = x.double().pow(2).sum(-1)
    assert float(((ssq.double() - want_ssq).abs() / want_ssq).max()) <= 1e-6
    rstd = torch.rsqrt(ssq / cols + 1e-5)
    normed = (x.float() * rstd[:, None]).to(torch.bfloat16) * gamma            # the separate steps, in torch
    q_ref, sf_ref = ops._quantize(normed, mat, fmt, gs, sf_layout=1)
    q, sf = torch.zeros_like(q_ref), torch.zeros_like(sf_ref)
    ops.fused_quantize_into(x, mat, fmt, gs, q, sf, row_scale=rstd, col_scale=gamma)
    assert torch.equal(q, q_ref) and torch.equal(sf, sf_ref)


def test_swiglu_pass_matches_torch():
    ops = _ops()
    dev = torch.device("cuda:0")
    gu = (synth.activations(300, 2 * 1536, seed=9).float() * 0.5).to(torch.bfloat16).to(dev)
    gate, up = gu[:, :1536], gu[:, 1536:]                       # column halves of one tensor
    got = ops.swiglu(gate, up)
    want = torch.nn.functional.silu(gate) * up
    diff = (got.float() - want.float()).abs()
    ulp = want.float().abs() * 2.0 ** -7                        # one bf16 step at the value's magnitude, at most
    assert bool((diff <= ulp + 1e-30).all())
    assert float((diff > 0).float().mean()) <= 5e-3             # hardware exponential: a rare last-bit difference


# ---- "quest" scaling ---------------------------------------------------------------------------------------------

_TIES = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]


def _quest_check(x_bf16, mat_np, blocked=False):
    """Kernel (codes, scale bytes, packed clip mask) against the oracle's quest restatement applied to the float32
    transform.  Scale bytes: equal except where the fp32 sums, taken in another order, straddle a power of two
    (budget 1e-3 of the groups).  In groups with equal scales: clip flags equal, codes equal except on exact
    rounding boundaries, where the kernel rounds to the even code and the reference's ladder toward zero."""
    ops = _ops()
    dev = torch.device("cuda:0")
    rows, cols = x_bf16.shape
    mask = torch.zeros(rows, cols // 8, dtype=torch.uint8, device=dev)
    q, sf = ops._quantize(x_bf16.to(dev), synth.to_bf16_tensor(mat_np).to(dev), "mx", None,
                          sf_layout=1 if blocked else 0, quest=True, clip_mask=mask)
    torch.cuda.synchronize()
    q, sf, mask = np_u8(q), np_u8(sf), np_u8(mask)
    x64 = synth.bf16_to_f64(x_bf16)
    t = np.asarray(mat_np, dtype=np.float64)
    y = wo.block_transform(x64, wo.matrix_to_transform(t) if t.shape[1] != 32 else t.T).astype(np.float32)
    ref = wo.quest_mxfp4(y)
    want_sf = ref["scale_quant"]
    if blocked:
        assert mismatch_fraction(sf.reshape(-1), wo.to_blocked(want_sf).reshape(-1)) < 1e-3
        return
    sf_valid = sf[:rows, : cols // 32]
    same = sf_valid == want_sf
    assert same.mean() > 1 - 1e-3, same.mean()
    same_e = np.repeat(same, 32, axis=1)
    bits = ((mask[:, :, None] >> np.arange(8, dtype=np.uint8)) & 1).reshape(rows, cols).astype(bool)
    assert np.array_equal(bits[same_e], ref["clip_mask"][same_e])
    got = canon_codes(q)
    want = canon_codes(ref["e2m1"])
    tie = np.isin(np.abs(ref["scaled"]), _TIES)
    assert np.array_equal(got[same_e & ~tie], want[same_e & ~tie])
    # on a tie either neighbour is a nearest value: same distance from the scaled value
    vg, vw = wo.E2M1_VALUES[got], wo.E2M1_VALUES[want]
    sc = ref["scaled"].astype(np.float64)
    assert np.array_equal(np.abs(vg - sc)[same_e & tie], np.abs(vw - sc)[same_e & tie])
    assert 0.5 < ref["clip_mask"].mean() <= 1.0


@pytest.mark.parametrize("kind", ["identity", "hadamard"])
@pytest.mark.parametrize("rows,cols", [(64, 128), (333, 4096), (1, 32), (130, 4096 + 64)])
def test_quest_matches_oracle(kind, rows, cols):
    x = synth.activations(rows, cols, seed=rows + cols)
    _quest_check(x, _matrix(kind, "mx", cols))


def test_quest_blocked_scales():
    _quest_check(synth.activations(300, 1024, seed=4), _matrix("hadamard", "mx", 1024), blocked=True)


def test_quest_against_triton_golden():
    """The inputs of the committed vectors (outputs of the reference's Triton kernel) through the kernel and through
    the pseudo-quantization wrapper that mirrors the reference's."""
    import os
    from wush_b200 import pseudo_quant
    d = np.load(os.path.join(os.path.dirname(__file__), "golden", "quest_vectors.npz"))
    x = torch.from_numpy(d["x"]).to(torch.bfloat16)
    _quest_check(x, np.eye(32))
    _quest_check(x, d["hadamard"].astype(np.float64))
    dev = torch.device("cuda:0")
    for name, mat in (("identity", torch.eye(32)), ("hadamard", torch.from_numpy(d["hadamard"]))):
        out, clip = pseudo_quant.mxfp4_forward_kernel_wrapper(x.to(dev), mat.to(dev, torch.bfloat16), return_clip_mask=True,
                                                              quest=True, gaussian_scale=2.92247856 / 6.0)
        want = torch.from_numpy(d[f"{name}_quest_out"]).to(torch.bfloat16).float().numpy()
        got = out.float().cpu().numpy()
        assert out.dtype == torch.bfloat16 and out.shape == x.shape
        # identical except on rounding ties and where a group's scale moved (sum order): well under 2 % here
        assert np.mean(got != want) < 0.02, np.mean(got != want)
        assert np.mean(clip.cpu().numpy() != d[f"{name}_quest_clip"]) < 1e-3
    with pytest.raises(NotImplementedError):
        pseudo_quant.mxfp4_forward_kernel_wrapper(x.to(dev), torch.eye(32, device=dev), quest=True)   # 3/4 with quest


# ---- shared transforms wider than the scale group (hadamard_group_size 64 / 128; 32 for NVFP4) -------------------

def _sylvester(n):
    h = np.ones((1, 1))
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return synth.bf16_to_f64(synth.to_bf16_tensor(h / np.sqrt(n)))


@pytest.mark.parametrize("fmt,n", [("mx", 64), ("mx", 128), ("nv", 32), ("nv", 64), ("nv", 128)])
@pytest.mark.parametrize("rows,cols", [(64, 128), (333, 4096), (130, 4096 + 128), (1, 256)])
@pytest.mark.parametrize("blocked", [False, True])
def test_wide_shared_matrix_matches_oracle(fmt, n, rows, cols, blocked):
    """x_block @ H_n in fp32 by the kernel, in float64 (rounded once to float32) by the oracle, then the same
    quantizer: scale bytes and codes within the tie budget.  Also a dense random 'rotation' in place of the
    Hadamard matrix, since nothing in the kernel assumes +-c entries."""
    ops = _ops()
    dev = torch.device("cuda:0")
    x = synth.activations(rows, cols, seed=rows + cols + n)
    for mat in (_sylvester(n), synth.bf16_to_f64(synth.to_bf16_tensor(
            np.linalg.qr(np.random.default_rng(n).standard_normal((n, n)))[0]))):
        gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
        q, sf = ops._quantize(x.to(dev), synth.to_bf16_tensor(mat).to(dev), fmt, gs, sf_layout=1 if blocked else 0)
        torch.cuda.synchronize()
        y = wo.wide_transform(synth.bf16_to_f64(x), mat).astype(np.float32).astype(np.float64)
        ref = wo.rtn_xxfp4(y, FMT[fmt])
        g = GROUP[fmt]
        keep = ~np.isnan(ref["fake_quant"]).any(axis=1)
        if blocked:
            assert mismatch_fraction(np_u8(sf).reshape(-1), wo.to_blocked(ref["scale_quant"]).reshape(-1)) <= 1e-3
        else:
            assert mismatch_fraction(np_u8(sf)[:rows, : cols // g][keep], ref["scale_quant"][keep]) <= 1e-3
        # the fp32 sums of 64 / 128 terms differ from the float64 ones in the last bits: values that sit on a rounding
        # boundary or on a power of two of the group maximum move a code or a scale (budget 1e-3)
        assert mismatch_fraction(canon_codes(np_u8(q)[keep]), canon_codes(ref["e2m1"][keep])) <= 1e-3


def test_wide_matrix_against_triton_golden_and_quest():
    """hadamard_group_size 64 and 128 on the committed outputs of the reference's Triton kernel, both methods,
    through the wrapper that mirrors the reference's; and the op-level API with a 128-wide Hadamard."""
    import os
    from wush_b200 import pseudo_quant
    ops = _ops()
    d = np.load(os.path.join(os.path.dirname(__file__), "golden", "quest_vectors.npz"))
    dev = torch.device("cuda:0")
    x = torch.from_numpy(d["x"]).to(torch.bfloat16).to(dev)
    for name in ("hadamard64", "hadamard128"):
        mat = torch.from_numpy(d[name]).to(dev, torch.bfloat16)
        for quest, gsc in ((True, 2.92247856 / 6.0), (False, 0.75)):
            out, clip = pseudo_quant.mxfp4_forward_kernel_wrapper(x, mat, return_clip_mask=True, quest=quest, gaussian_scale=gsc)
            tag = f"{name}_{'quest' if quest else 'absmax'}"
            want = torch.from_numpy(d[tag + "_out"]).to(torch.bfloat16).float().numpy()
            got = out.float().cpu().numpy()
            assert np.mean(got != want) < 0.03, (tag, np.mean(got != want))        # ties + sum order
            assert np.mean(clip.cpu().numpy() != d[tag + "_clip"]) < 2e-3
    q, sf, mask = ops.fused_quantize_mx_op(x, torch.from_numpy(d["hadamard128"]).to(dev, torch.bfloat16), "quest", True)
    assert q.shape == (64, 64) and mask.shape == (64, 16)
    with pytest.raises(NotImplementedError):
        ops.fused_quantize_mx_op(x[:, :64], torch.from_numpy(d["hadamard128"]).to(dev, torch.bfloat16), "abs_max", False)
