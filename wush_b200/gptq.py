"""GPTQ / Babai column sweep with per-group WUSH transforms on the GPU: the replacement for
``quantize_layers`` / ``gptq_babai_outer`` / ``block_transform_gptq_babai_inner`` / ``get_transform`` /
``collate_xxfp4`` of the reference (src/quantization/wush_gptq.py:165-441).

Division of labour.  The large float64 matrices stay with cuSOLVER / cuBLAS through torch (damped Cholesky of the
Hessian, the Gram matrix of a block's targets, the update of the remaining targets).  The 32 x 32 algebra of a
block -- eigen-decomposition, WUSH transform, rounding, QR -- is one CTA (``wush_gptq_block_prepare``), and
everything per weight row -- rotation, triangular solve, scale choice, E2M1 rounding, the nearest-plane loop with
frozen scales, the coefficient product and the packing the reference does in ``collate_xxfp4`` -- is one launch
of ``wush_gptq_block_step``.

Round-to-nearest mode (``force_rtn=True``) has no dependency between blocks, so all blocks are handled by one
launch of each kernel.  GPTQ mode walks the blocks from last to first like the reference.

Differences from the reference, both inside its own numerical freedom:
* the singular vectors of the block targets come from the eigen-decomposition of the G x G Gram matrix
  y y^T instead of an SVD of the G x R matrix y (same subspaces; the sign of every vector is fixed by
  making its largest component positive, where LAPACK's and cuSOLVER's SVDs each have their own convention,
  so the reference's transforms differ between its own CPU and GPU runs in the same way);
* float64 summation orders (cuBLAS vs. the reference's device), which can move a value across a rounding
  boundary only at an exact tie.
"""
from __future__ import annotations

import torch
from torch import nn

from . import _lib

_FORMATS = {
    "mxfp4": dict(group=32, fmt=_lib.FORMAT_MXFP4, scale_dtype=torch.float8_e8m0fnu, global_scale=3.0),
    "nvfp4": dict(group=16, fmt=_lib.FORMAT_NVFP4, scale_dtype=torch.float8_e4m3fn, global_scale=10.0),
}


def _hadamard(n: int, device) -> torch.Tensor:
    """Normalized Sylvester Hadamard matrix (the reference takes it from scipy, wush_gptq.py:20)."""
    h = torch.ones(1, 1, dtype=torch.float64, device=device)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    if h.shape[0] != n:
        raise ValueError("transform size must be a power of two")
    return h * n ** -0.5


def damped_cholesky_upper(hessian: torch.Tensor, damp_ratio: float = 1e-2, max_try: int = 100) -> torch.Tensor:
    """Upper factor U, U^T U = H + damping, with the reference's retry loop (wush_gptq.py:196-208)."""
    h = hessian.to(dtype=torch.float64, copy=True)
    d = h.diagonal()
    d += damp_ratio * d.mean()
    for _ in range(max_try):
        u, info = torch.linalg.cholesky_ex(h, upper=True, check_errors=False)
        if not bool(info.any()):
            return u.contiguous()      # the kernels index it row-major (cholesky_ex may return a transposed view)
        d += damp_ratio * d.mean()
    raise AssertionError("Hessian decomposition failed. Please try using more samples or increasing damp_ratio.")


def get_transform(basis: torch.Tensor, y: torch.Tensor, transform_type: str = "identity",
                  transform_dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """Block transforms, batched over leading dimensions (wush_gptq.py:304-347).

    basis: (..., B, B) upper-triangular diagonal blocks of the Cholesky factor; y: (..., B, R) targets.
    'wush': T = Had . diag(s^1/2) . V^T . basis^-T with V, s the left singular vectors / values of y,
    s scaled by R^-1/2 and damped by 1 % of its mean.  Returns float64 values rounded to `transform_dtype`.
    """
    b = basis.shape[-1]
    dev = basis.device
    if transform_type == "identity":
        t = torch.eye(b, dtype=torch.float64, device=dev).expand(basis.shape).clone()
    elif transform_type == "hadamard":
        t = _hadamard(b, dev).expand(basis.shape).clone()
    elif transform_type in ("wush", "wus"):
        had = torch.eye(b, dtype=torch.float64, device=dev) if transform_type == "wus" else _hadamard(b, dev)
        gram = y @ y.transpose(-2, -1)
        evals, evecs = torch.linalg.eigh(gram)                       # ascending
        evals, v = evals.flip(-1), evecs.flip(-1)                    # singular values descending, like an SVD
        lead = v.gather(-2, v.abs().argmax(dim=-2, keepdim=True))    # largest component of every vector
        v = v * torch.where(lead < 0, -1.0, 1.0)
        s = evals.clamp_min(0).sqrt() * y.shape[-1] ** -0.5
        s = s + s.mean(dim=-1, keepdim=True) * 1e-2
        rhs = (had * s.sqrt().unsqueeze(-2)) @ v.transpose(-2, -1)
        t = torch.linalg.solve_triangular(basis.transpose(-2, -1), rhs, upper=False, left=False)
    else:
        raise NotImplementedError(transform_type)
    t = t.to(transform_dtype).to(torch.float64)
    if not bool(t.isfinite().all()):
        raise AssertionError("non-finite block transform")
    return t


def _prepare(gram, basis, ldb, basis_step, nblocks, fmt, transform, fake_f32, rows, tmat, rn, qt, status):
    lib = _lib.load()
    with torch.cuda.device(tmat.device):
        rc = lib.wush_gptq_block_prepare(gram.data_ptr() if gram is not None else None, basis.data_ptr(), ldb, basis_step,
                                         nblocks, fmt, _lib.TRANSFORMS[transform], _lib.SWEEP_FAKE_F32 if fake_f32 else 0,
                                         rows, tmat.data_ptr(), rn.data_ptr(), qt.data_ptr(), status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_gptq_block_prepare")


def _block_step(rn, y, qt, tmat, nblocks, col_block0, rows, codes, scales, fake, coef, fmt, rtn):
    lib = _lib.load()
    flags = (_lib.SWEEP_RTN_ONLY if rtn else 0) | (_lib.SWEEP_FAKE_F32 if fake.dtype == torch.float32 else 0)
    with torch.cuda.device(codes.device):
        rc = lib.wush_gptq_block_step(rn.data_ptr(), y.data_ptr(), qt.data_ptr(), tmat.data_ptr(), nblocks, col_block0,
                                      rows, codes.shape[1] * 2, fmt, flags, codes.data_ptr(), scales.data_ptr(),
                                      fake.data_ptr(), coef.data_ptr() if coef is not None else None,
                                      torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_gptq_block_step")


@torch.no_grad()
def gptq_babai_sweep(weight: torch.Tensor, hessian: torch.Tensor | None, quant_type: str, transform_class: str,
                     force_rtn: bool = False, transforms: torch.Tensor | None = None, group=None,
                     total_rows: int | None = None) -> dict:
    """Quantize one (concatenated) weight matrix: the work of gptq_babai_outer as quantize_layers drives it
    (wush_gptq.py:373-441: block size = group size, `force_rtn` for the outer and the inner loop, transforms
    rounded to the weight dtype).

    weight: (R, C) bf16 / fp32 on a CUDA device; hessian: (C, C) or None (identity).  `transforms`
    ((C/G, G, G), optional) overrides the computed block transforms.  Returns a dict with
    'fake_quant' (R, C) weight dtype, 'qweight' (R, C/2) uint8 packed E2M1, 'scale_quant' (R, C/G) float8,
    'transform_basis' (C/G, G, G) weight dtype and 'global_scale'.

    Per block the GPU runs: the Gram matrix of the targets (cuBLAS), `wush_gptq_block_prepare` (transform, QR),
    `wush_gptq_block_step` (everything per weight row) and the update of the remaining targets (cuBLAS) --
    four launches and no host synchronisation; round-to-nearest mode does all blocks with one launch of each.

    Row-sharded over GPUs (`group` given, `total_rows` = rows of the whole matrix): every rank passes ITS rows of
    the weight and the same Hessian.  The sweep is independent per weight row except for the block transforms,
    which depend on the Gram matrix of the targets of ALL rows: the per-rank G x G Gram matrices are summed with one
    all-reduce per block (one for all blocks in round-to-nearest mode) and everything else stays local, so every
    rank computes the same transforms and its own rows' codes; the results are the rows of the unsharded sweep.
    """
    if not weight.is_cuda:
        raise RuntimeError("wush_b200 runs on CUDA devices only")
    if weight.dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"weight dtype {weight.dtype}")
    if transform_class not in ("identity", "hadamard", "wush", "wus"):
        raise NotImplementedError(transform_class)
    f = _FORMATS[quant_type]
    g, fmt = f["group"], f["fmt"]
    rows, cols = weight.shape
    if cols % g:
        raise ValueError(f"in_features must be a multiple of {g}")
    sharded = group is not None or total_rows is not None
    if sharded:
        import torch.distributed as dist
        if total_rows is None:
            raise ValueError("a row-sharded sweep needs total_rows (the R^-1/2 factor of the transform uses all rows)")
    all_rows = total_rows if sharded else rows

    def all_ranks(gram_t):
        if sharded and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(gram_t, group=group)
        return gram_t
    dev, nb = weight.device, cols // g
    f32 = weight.dtype == torch.float32
    x = weight.t().to(torch.float64).contiguous()                                     # (C, R), :188
    h = torch.eye(cols, dtype=torch.float64, device=dev) if hessian is None else hessian.to(dev)
    u = damped_cholesky_upper(h)                                                      # :195-208
    del h
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(rows, nb, dtype=torch.uint8, device=dev)
    fake = torch.empty(rows, cols, dtype=weight.dtype, device=dev)
    tb = torch.empty(nb, g, g, dtype=torch.float64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    transform = transform_class
    if transforms is not None:
        tb.copy_(transforms.to(torch.float64))
        transform = "given"
    need_gram = transform in ("wush", "wus")
    diag_step = g * cols + g                      # from one diagonal block of u to the next

    if force_rtn:
        # no error feedback between blocks: the targets of block b are U_bb x_b (what :210-222 leave in y
        # when x is never updated), and every block is prepared and quantized at once
        idx = torch.arange(nb, device=dev)
        basis = u.view(nb, g, nb, g)[idx, :, idx, :].contiguous()                     # (nb, G, G) diagonal blocks
        yb = basis @ x.view(nb, g, rows)
        gram = all_ranks(yb @ yb.transpose(-2, -1)) if need_gram else None
        rn, qt = torch.empty_like(tb), torch.empty_like(tb)
        _prepare(gram, basis, g, g * g, nb, fmt, transform, f32, all_rows, tb, rn, qt, status)
        _block_step(rn, yb, qt, tb, nb, 0, rows, codes, scales, fake, None, fmt, True)
    else:
        y = u @ x                                                                     # :210
        rn = torch.empty(g, g, dtype=torch.float64, device=dev)
        qt = torch.empty_like(rn)
        gram = torch.empty_like(rn) if need_gram else None
        for b in range(nb - 1, -1, -1):                                               # :214
            i1, i2 = b * g, (b + 1) * g
            yb = y[i1:i2]
            if need_gram:
                torch.mm(yb, yb.t(), out=gram)
                all_ranks(gram)
            _prepare(gram, u[i1:i2, i1:i2], cols, diag_step, 1, fmt, transform, f32, all_rows, tb[b], rn, qt, status)
            # the coefficients go straight into x (:221), which the update of the remaining targets reads (:222)
            _block_step(rn, yb, qt, tb[b], 1, b, rows, codes, scales, fake, x[i1:i2], fmt, False)
            if i1:
                y[:i1].addmm_(u[:i1, i1:i2], x[i1:i2], alpha=-1.0)
    if int(status.item()):
        raise AssertionError("non-finite block transform")
    return {
        "fake_quant": fake,
        "qweight": codes,
        "scale_quant": scales.view(f["scale_dtype"]),
        "transform_basis": tb.to(weight.dtype),
        "global_scale": f["global_scale"],
    }


class BlockTransformQuantizer(nn.Module):
    """Activation side of a pseudo-quantized layer (src/utils/wush_utils.py:114-150): per-group transform,
    then FP4 fake quantization, here one launch of the fused quantize kernel (with the bf16 rounding the
    reference has between its einsum and its quantizer) followed by the dequantization of its output."""

    def __init__(self, transform: torch.Tensor | None, quant_type: str) -> None:
        super().__init__()
        if transform is not None:
            self.register_buffer("transform", transform, persistent=True)       # (C/G, G, G)
        else:
            self.transform = None
        self.quant_type = quant_type

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import qutlass_ops as ops
        f = _FORMATS[self.quant_type]
        g = f["group"]
        xf = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        if self.transform is not None:
            mat = self.transform.to(torch.bfloat16).reshape(-1, g).t().contiguous()  # [G, C]: column block n = T_n^T
        else:
            mat = torch.eye(g, dtype=torch.bfloat16, device=x.device)
        fmt = "mx" if self.quant_type == "mxfp4" else "nv"
        gs = torch.tensor([f["global_scale"]], dtype=torch.float32, device=x.device) if fmt == "nv" else None
        q, sf = ops._quantize(xf, mat, fmt, gs, round_bf16=True)
        return dequantize(q, sf[: xf.shape[0], : xf.shape[1] // g], self.quant_type).to(x.dtype).reshape(x.shape)


def dequantize(qweight: torch.Tensor, scale_quant: torch.Tensor, quant_type: str) -> torch.Tensor:
    """Packed E2M1 codes and per-group float8 scales -> float32 values (dequant_xxfp4, wush_gptq.py:141-162)."""
    f = _FORMATS[quant_type]
    lut = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.],
                       dtype=torch.float32, device=qweight.device)
    b = qweight.view(torch.uint8)
    vals = lut[torch.stack([b & 0xF, b >> 4], dim=-1).flatten(-2).long()]
    s = scale_quant.view(f["scale_dtype"]).to(torch.float32)
    out = vals.unflatten(-1, (-1, f["group"])) * s.unsqueeze(-1) / f["global_scale"]
    return out.flatten(-2)


class QuantLinear(nn.Module):
    """Pseudo-quantized linear layer (src/utils/wush_utils.py:100-112): dequantized transformed weights and
    an activation quantizer that applies the matching transform."""

    def __init__(self, weight: torch.Tensor, activation_quantizer: nn.Module | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(weight, requires_grad=False)
        self.activation_quantizer = activation_quantizer

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xq = self.activation_quantizer(x) if self.activation_quantizer is not None else x
        return xq @ self.weight.transpose(-2, -1)


@torch.no_grad()
def quantize_layers(*weights: torch.Tensor, hessian: torch.Tensor, quant_type: str, transform_class: str,
                    force_rtn: bool = False):
    """Drop-in for quantize_layers (wush_gptq.py:373-441): the weights that share an input (q/k/v, gate/up)
    are concatenated, swept once, and split again.  Returns (pseudo-quantized layers, per-layer dicts with
    'transform_basis', 'qweight', 'scale_quant', 'global_scale')."""
    weight = torch.cat(weights, dim=0)
    res = gptq_babai_sweep(weight, hessian, quant_type, transform_class, force_rtn)
    sizes = [w.size(0) for w in weights]
    tb = res["transform_basis"]
    layers = [QuantLinear(weight=w, activation_quantizer=BlockTransformQuantizer(transform=tb, quant_type=quant_type))
              .to(weight.device) for w in res["fake_quant"].split(sizes, dim=0)]
    qs, ss = res["qweight"].split(sizes, dim=0), res["scale_quant"].split(sizes, dim=0)
    results = [{"transform_basis": tb, "qweight": qs[i], "scale_quant": ss[i], "global_scale": res["global_scale"]}
               for i in range(len(weights))]
    return layers, results


def export_realquant(result: dict, quant_type: str, dtype: torch.dtype = torch.bfloat16) -> dict:
    """One layer's entry of the reference's 'realquant' checkpoint (wush_gptq.py:586-599) from a per-layer dict
    of quantize_layers(): the names and layouts FPQuantLinear loads (`load_quantized`).  The per-group transforms
    (C/G, G, G) become the (G, C) matrix whose column block n is T_n^T."""
    gs = _FORMATS[quant_type]["global_scale"]
    tb = result["transform_basis"].to(dtype)
    matrix = tb.reshape(-1, tb.shape[-1]).t().contiguous()
    scale = torch.tensor([gs], dtype=torch.float32)
    return {
        "qweight": result["qweight"].view(torch.uint8).cpu(),
        "scales": result["scale_quant"].view(torch.uint8).cpu(),
        "forward_hadamard_matrix": matrix.cpu(),
        "backward_hadamard_matrix": matrix.cpu().clone(),
        "weight_global_scale": scale.clone(),
        "act_global_scale": scale.clone(),
    }
