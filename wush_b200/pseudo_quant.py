"""Pseudo-quantization (quantize, then dequantize) with the call signatures of the reference's Triton wrappers
``mxfp4_forward_kernel_wrapper`` (inference_lib/src/fp_quant/module/triton/mxfp4.py:136-176) and
``nvfp4_forward_kernel_wrapper`` (.../triton/nvfp4.py:122-149), and ``pseudoquantize_fp``
(src/utils/wush_utils.py:6-53) on top of them.  The fused transform + quantize kernel produces codes and
scales; the values are rebuilt from them.

Differences from the Triton kernels: ties round to the even code (the reference's torch quantizer's rule; the
Triton kernels round ties toward zero), and the scale constant is not free: ``quest=False`` goes with
``gaussian_scale=3/4`` (abs-max scaling, what the WUSH pipeline uses) and ``quest=True`` with
``gaussian_scale=2.92247856/6``, the two pairs the reference's own caller passes (pseudoquant_linear_fns.py:20-26).
"""
from __future__ import annotations

import torch

from . import _lib
from . import qutlass_ops as ops
from .gptq import dequantize


QUEST_GAUSSIAN_SCALE = 2.92247856 / 6.0


def _flat(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()


def _values_times_scale(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """E2M1 values times their group's E8M0 scale, exactly (quest codes carry no global factor)."""
    lut = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.],
                       dtype=torch.float32, device=q.device)
    vals = lut[torch.stack([q & 0xF, q >> 4], dim=-1).flatten(-2).long()]
    scale = sf.contiguous().view(torch.float8_e8m0fnu).to(torch.float32)
    return (vals.unflatten(-1, (-1, 32)) * scale.unsqueeze(-1)).flatten(-2)


def mxfp4_forward_kernel_wrapper(x: torch.Tensor, hadamard_matrix: torch.Tensor, return_clip_mask: bool = False,
                                 gaussian_scale: float = 3 / 4, quest: bool = True):
    """(dequantized tensor like x, clip mask | None).  x @ hadamard_matrix per 32-element group, E8M0 scale, E2M1
    values.  quest=False: abs-max scale, which never clips, so the mask is all True.  quest=True: the scale follows
    the group's standard deviation and the mask marks the values inside +-6 scales."""
    if hadamard_matrix.shape[-1] not in (32, 64, 128) or hadamard_matrix.shape[0] != hadamard_matrix.shape[-1]:
        raise NotImplementedError("the transform must be square, 32, 64 or 128 wide")
    xf = _flat(x)
    mat = hadamard_matrix.to(device=x.device, dtype=torch.bfloat16)
    if quest:
        if abs(gaussian_scale - QUEST_GAUSSIAN_SCALE) > 1e-9:
            raise NotImplementedError("quest=True is implemented for gaussian_scale=2.92247856/6 only")
        packed = torch.empty(xf.shape[0], xf.shape[1] // 8, dtype=torch.uint8, device=xf.device) if return_clip_mask else None
        q, sf = ops._quantize(xf, mat, "mx", None, quest=True, clip_mask=packed)
        out = _values_times_scale(q, sf[: xf.shape[0], : xf.shape[1] // 32]).to(x.dtype).reshape(x.shape)
        mask = None
        if return_clip_mask:
            bits = (packed.unsqueeze(-1) >> torch.arange(8, device=xf.device, dtype=torch.uint8)) & 1
            mask = bits.reshape(xf.shape).to(torch.bool).reshape(x.shape)
        return out, mask
    if abs(gaussian_scale - 0.75) > 1e-12:
        raise NotImplementedError("quest=False is implemented for gaussian_scale=3/4 (abs-max scaling) only")
    q, sf = ops._quantize(xf, mat, "mx", None)
    out = dequantize(q, sf[: xf.shape[0], : xf.shape[1] // 32], "mxfp4").to(x.dtype).reshape(x.shape)
    return out, (torch.ones_like(x, dtype=torch.bool) if return_clip_mask else None)


def nvfp4_forward_kernel_wrapper(x: torch.Tensor, hadamard_matrix: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """Dequantized tensor like x: x @ hadamard_matrix per 16-element group, E4M3 scale of absmax * global_scale / 6,
    E2M1 values, divided by global_scale again."""
    if hadamard_matrix.shape[-1] not in (16, 32, 64, 128) or hadamard_matrix.shape[0] != hadamard_matrix.shape[-1]:
        raise NotImplementedError("the transform must be square, 16, 32, 64 or 128 wide")
    xf = _flat(x)
    gs = global_scale.to(device=x.device, dtype=torch.float32).reshape(-1)[:1]
    q, sf = ops._quantize(xf, hadamard_matrix.to(device=x.device, dtype=torch.bfloat16), "nv", gs)
    lut_vals = dequantize(q, sf[: xf.shape[0], : xf.shape[1] // 16], "nvfp4") * (10.0 / gs)   # dequantize() divides by 10
    return lut_vals.to(x.dtype).reshape(x.shape)


def pseudoquantize_fp(x: torch.Tensor, dtype: str) -> torch.Tensor:
    """src/utils/wush_utils.py:6-53: identity transform, abs-max scaling."""
    if dtype == "mxfp4":
        return mxfp4_forward_kernel_wrapper(x, torch.eye(32, dtype=x.dtype, device=x.device), return_clip_mask=True,
                                            quest=False, gaussian_scale=3.0 / 4.0)[0]
    if dtype == "nvfp4":
        return nvfp4_forward_kernel_wrapper(x, torch.eye(16, dtype=x.dtype, device=x.device),
                                            torch.as_tensor(10.0, dtype=x.dtype, device=x.device))
    raise ValueError(f"Unsupported forward dtype: {dtype}")
