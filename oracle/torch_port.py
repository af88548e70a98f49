"""Multi-threaded torch-CPU restatement of the reference's quantizer path -- TEST/BENCH
INFRASTRUCTURE, used as the timed CPU baseline (the reference itself is pure Python/torch and
can only be imported from its own checkout).

Same operations, dtype (float64) and tensor-op granularity as the reference's
``block_transform`` (src/quantization/wush_gptq.py:350-370) followed by ``rtn_xxfp4``
(:91-138) / ``rtn_e2m1`` (:34-71), so its wall time stands for the reference's CPU path.
``tests/test_torch_port.py`` checks it bit for bit against the NumPy oracle.
"""
from __future__ import annotations

import torch

_F64 = torch.float64
_GRID = [-6., -4., -3., -2., -1.5, -1., -.5, -0., 0., .5, 1., 1.5, 2., 3., 4., 6.]
_CODE = [15, 14, 13, 12, 11, 10, 9, 8, 0, 1, 2, 3, 4, 5, 6, 7]
_FMT = {"mxfp4": (32, torch.float8_e8m0fnu, 4.0, 3.0), "nvfp4": (16, torch.float8_e4m3fn, 6.0, 10.0)}


def block_transform(x: torch.Tensor, mat: torch.Tensor) -> torch.Tensor:
    """x (T, C) any float, mat (G, C) per-group or (G, G) shared -> float64 (T, C)."""
    g = mat.shape[0]
    xr = x.to(_F64).unflatten(-1, (-1, 1, g))                       # (T, C/G, 1, G)
    if mat.shape[1] == g:
        m = mat.to(_F64)                                             # y = x @ mat
    else:
        m = mat.to(_F64).unflatten(-1, (-1, g)).transpose(0, 1)      # (C/G, G, G): [n][k][out]
    return (xr @ m).flatten(-3)


def rtn_e2m1(x: torch.Tensor):
    grid = torch.tensor(_GRID, dtype=_F64)
    code = torch.tensor(_CODE, dtype=torch.uint8)
    idx = torch.bucketize(x, grid, right=False)
    lo, hi = (idx - 1).clamp(0, 15), idx.clamp(0, 15)
    d_hi, d_lo = grid[hi] - x, x - grid[lo]
    up = (d_hi < d_lo) | ((d_hi == d_lo) & (code[hi] % 2 == 0))
    pick = torch.where(up, hi, lo)
    c = code[pick]
    return grid[pick], (c[..., 1::2] << 4) | c[..., 0::2]


def rtn_xxfp4(y: torch.Tensor, fmt: str) -> dict:
    g, sdtype, ss, gs = _FMT[fmt]
    yr = y.to(_F64).unflatten(-1, (-1, g))
    amax = yr.abs().amax(dim=-1, keepdim=True)
    sq = (amax * gs / ss).to(sdtype)
    sd = sq.to(_F64)
    vals, packed = rtn_e2m1(yr * gs / sd)
    return {"fake_quant": (vals * sd / gs).flatten(-2), "e2m1": packed.flatten(-2),
            "scale_quant": sq[..., 0].view(torch.uint8)}


def fused_transform_quant(x: torch.Tensor, mat: torch.Tensor, fmt: str) -> dict:
    """block transform (float64, rounded once to float32) then group quantization."""
    return rtn_xxfp4(block_transform(x, mat).to(torch.float32), fmt)


def hessian_update(h: torch.Tensor, n: int, x: torch.Tensor) -> int:
    """One WUSH.update step (src/quantization/wush_gptq.py:456-469) with the Triton launch
    replaced by the equivalent fp32 addmm: h <- h*n/(n+b) + (x/sqrt(n+b))^T (x/sqrt(n+b))."""
    x = x.flatten(end_dim=-2)
    b = x.size(0)
    h *= n / (n + b)
    xs = x.to(torch.float32) * (n + b) ** -.5
    h.addmm_(xs.t(), xs)
    return n + b


def fp4_gemm(a_q, a_s, b_q, b_s, alpha: float, fmt: str) -> torch.Tensor:
    """Dequantize both operands (src/quantization/wush_gptq.py:141-162 without the global-scale
    division, which alpha carries) and multiply in fp32; bf16 result."""
    g, sdtype, _, _ = _FMT[fmt]
    lut = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.], dtype=torch.float32)

    def deq(q, s):
        codes = torch.stack([q & 0xF, q >> 4], dim=-1).flatten(-2).long()
        v = lut[codes].unflatten(-1, (-1, g))
        return (v * s.view(sdtype).to(torch.float32)[..., None]).flatten(-2)

    return (alpha * (deq(a_q, a_s) @ deq(b_q, b_s).t())).to(torch.bfloat16)
