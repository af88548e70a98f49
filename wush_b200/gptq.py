"""GPTQ / Babai column sweep with per-group WUSH transforms on the GPU: the replacement for
``quantize_layers`` / ``gptq_babai_outer`` / ``block_transform_gptq_babai_inner`` / ``get_transform`` /
``collate_xxfp4`` of the reference (src/quantization/wush_gptq.py:165-441).

Division of labour.  The dense float64 linear algebra the reference does with torch stays with torch on the
GPU (cuSOLVER / cuBLAS: damped Cholesky of the Hessian, the per-block symmetric eigenproblem and QR, the
trailing update of the targets).  Everything per weight row -- triangular solve, scale choice, E2M1
rounding, the nearest-plane loop with frozen scales, the coefficient product and the packing the
reference does in ``collate_xxfp4`` -- is one launch of ``wush_gptq_block_step`` per block.

Round-to-nearest mode (``force_rtn=True``) has no dependency between blocks, so all blocks are factored in
batched calls and quantized by ONE kernel launch.  GPTQ mode walks the blocks from last to first like the
reference.

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
            return u
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


def _block_step(rn, ynew, tmat, col_block0, codes, scales, fake, coef, fmt, rtn):
    lib = _lib.load()
    nblocks, g, rows = ynew.shape
    flags = (_lib.SWEEP_RTN_ONLY if rtn else 0) | (_lib.SWEEP_FAKE_F32 if fake is not None and fake.dtype == torch.float32 else 0)
    for t in (rn, ynew, tmat):
        assert t.is_contiguous() and t.dtype == torch.float64
    with torch.cuda.device(ynew.device):
        rc = lib.wush_gptq_block_step(rn.data_ptr(), ynew.data_ptr(), tmat.data_ptr(), nblocks, col_block0, rows,
                                      codes.shape[1] * 2, fmt, flags, codes.data_ptr(), scales.data_ptr(),
                                      fake.data_ptr() if fake is not None else None,
                                      coef.data_ptr() if coef is not None else None,
                                      torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_gptq_block_step")


@torch.no_grad()
def gptq_babai_sweep(weight: torch.Tensor, hessian: torch.Tensor | None, quant_type: str, transform_class: str,
                     force_rtn: bool = False, transforms: torch.Tensor | None = None) -> dict:
    """Quantize one (concatenated) weight matrix: the work of gptq_babai_outer as quantize_layers drives it
    (wush_gptq.py:373-441: block size = group size, `force_rtn` for the outer and the inner loop, transforms
    rounded to the weight dtype).

    weight: (R, C) bf16 / fp32 on a CUDA device; hessian: (C, C) or None (identity).  `transforms`
    ((C/G, G, G), optional) overrides the computed block transforms.  Returns a dict with
    'fake_quant' (R, C) weight dtype, 'qweight' (R, C/2) uint8 packed E2M1, 'scale_quant' (R, C/G) float8,
    'transform_basis' (C/G, G, G) weight dtype and 'global_scale'.
    """
    if not weight.is_cuda:
        raise RuntimeError("wush_b200 runs on CUDA devices only")
    if weight.dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"weight dtype {weight.dtype}")
    f = _FORMATS[quant_type]
    g, fmt = f["group"], f["fmt"]
    rows, cols = weight.shape
    if cols % g:
        raise ValueError(f"in_features must be a multiple of {g}")
    dev, nb = weight.device, cols // g
    x = weight.t().to(torch.float64).contiguous()                                     # (C, R), :188
    h = torch.eye(cols, dtype=torch.float64, device=dev) if hessian is None else hessian.to(dev)
    u = damped_cholesky_upper(h)                                                      # :195-208
    del h
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(rows, nb, dtype=torch.uint8, device=dev)
    fake = torch.empty(rows, cols, dtype=weight.dtype, device=dev)
    tb = torch.empty(nb, g, g, dtype=torch.float64, device=dev)

    def factor(basis, yb, t):
        # QR of basis . T^T (:251); only R and Q^T y are needed (:252)
        q, rn = torch.linalg.qr(basis @ t.transpose(-2, -1), mode="reduced")
        return rn.contiguous(), (q.transpose(-2, -1) @ yb).contiguous()

    if force_rtn:
        # no error feedback between blocks: the targets of block b are U_bb x_b (what :210-222 leave in y
        # when x is never updated), and every block can be factored and quantized at once
        idx = torch.arange(nb, device=dev)
        ur = u.view(nb, g, nb, g)
        basis = ur[idx, :, idx, :].contiguous()                                       # (nb, G, G) diagonal blocks
        yb = basis @ x.view(nb, g, rows)
        t = transforms.to(torch.float64) if transforms is not None else get_transform(basis, yb, transform_class, weight.dtype)
        rn, ynew = factor(basis, yb, t)
        tb.copy_(t)
        _block_step(rn, ynew, tb, 0, codes, scales, fake, None, fmt, True)
    else:
        y = u @ x                                                                     # :210
        coef = torch.empty(1, g, rows, dtype=torch.float64, device=dev)
        for b in range(nb - 1, -1, -1):                                               # :214
            i1, i2 = b * g, (b + 1) * g
            basis, yb = u[i1:i2, i1:i2], y[i1:i2]
            t = (transforms[b].to(torch.float64) if transforms is not None
                 else get_transform(basis, yb, transform_class, weight.dtype))
            rn, ynew = factor(basis, yb, t)
            tb[b] = t
            _block_step(rn[None], ynew[None], tb[b:b + 1], b, codes, scales, fake, coef, fmt, False)
            x[i1:i2] = coef[0]                                                        # :221
            if i1:
                y[:i1].addmm_(u[:i1, i1:i2], coef[0], alpha=-1.0)                     # :222
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
