"""Inference-time quantized linear layer on top of the fused quantize and FP4 GEMM kernels.

Mirrors the inference path of the reference's ``FPQuantLinear`` / ``FPQuant4x16NoMasterFn``
(inference_lib/src/fp_quant/module/linear.py:51-386, linear_fns.py:29-76, 494-539): same config
field names, buffer names and shapes (``qweight`` u8 [out, in/2], ``scales`` u8 [out, in/G],
``forward_hadamard_matrix`` [G, in] for WUSH or [G, G] shared, fp32 ``weight_global_scale`` /
``act_global_scale``), same ``pre_forward()`` / ``forward()`` protocol.  Training paths, master
weights, pseudo-quantization and MXFP8 are not part of this layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

import torch
from torch import nn

from . import _lib
from . import qutlass_ops as ops


class FPQuantDtype(Enum):
    MXFP4 = "mxfp4"
    NVFP4 = "nvfp4"
    BF16 = "bf16"


@dataclass
class FPQuantConfig:
    """Field names follow inference_lib/src/fp_quant/utils/config.py:17-26."""
    forward_dtype: FPQuantDtype = FPQuantDtype.MXFP4
    forward_method: str = "abs_max"
    backward_dtype: FPQuantDtype = FPQuantDtype.BF16
    store_master_weights: bool = False
    hadamard_group_size: int = 32
    pseudoquantization: bool = False
    transform_init: str = "hadamard"            # "hadamard" | "identity" | "wush"
    modules_to_not_convert: List[str] = field(default_factory=lambda: ["lm_head"])


def validate_config(config: FPQuantConfig) -> None:
    if config.forward_dtype not in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4):
        raise ValueError(f"Unsupported forward dtype: {config.forward_dtype}")
    if config.forward_method != "abs_max":
        raise NotImplementedError("only forward_method='abs_max' is implemented")
    want = 32 if config.forward_dtype == FPQuantDtype.MXFP4 else 16
    if config.hadamard_group_size != want:
        raise NotImplementedError(f"{config.forward_dtype.value} needs hadamard_group_size == {want} here")
    if config.store_master_weights or config.pseudoquantization or config.backward_dtype != FPQuantDtype.BF16:
        raise NotImplementedError("inference only: no master weights, pseudo-quantization or quantized backward")


def _fmt(dtype: FPQuantDtype) -> str:
    return "mx" if dtype == FPQuantDtype.MXFP4 else "nv"


def forward_quantize(x: torch.Tensor, hadamard_matrix: torch.Tensor, global_scale: torch.Tensor, dtype: FPQuantDtype,
                     forward_method: str, blocked: bool = False):
    """(codes u8, scales u8) of a 2-D bf16 tensor; reference: linear_fns.py:29-62.  With ``blocked`` the
    scales come out in the layout the GEMM consumes (no separate re-layout pass)."""
    if forward_method != "abs_max":
        raise NotImplementedError("only forward_method='abs_max' is implemented")
    layout = _lib.SF_BLOCKED if blocked else _lib.SF_ROW_MAJOR
    gs = global_scale.float() if dtype == FPQuantDtype.NVFP4 else None
    return ops._quantize(x.to(torch.bfloat16), hadamard_matrix.to(torch.bfloat16), _fmt(dtype), gs, sf_layout=layout)


def _hadamard(n: int, device, dtype) -> torch.Tensor:
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h * n ** -0.5).to(device=device, dtype=dtype)


class FPQuantLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, config: FPQuantConfig, bias: bool = True, device=None,
                 dtype: Optional[torch.dtype] = None):
        super().__init__()
        validate_config(config)
        kw = {"device": device, "dtype": dtype or torch.bfloat16}
        self.in_features, self.out_features, self.config = in_features, out_features, config
        g = config.hadamard_group_size
        if in_features % 128 != 0 or out_features % 8 != 0:
            raise ValueError("in_features must be a multiple of 128 and out_features of 8")
        self.weight = nn.Parameter(torch.empty((out_features, in_features), **kw), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(out_features, **kw), requires_grad=False) if bias else None
        self.register_buffer("qweight", torch.empty(out_features, in_features // 2, dtype=torch.uint8, device=device))
        self.register_buffer("scales", torch.empty(out_features, in_features // g, dtype=torch.uint8, device=device))
        gs = 3.0 if config.forward_dtype == FPQuantDtype.MXFP4 else 10.0    # linear.py:207-217, wush_gptq.py:588
        self.register_buffer("weight_global_scale", torch.tensor([gs], dtype=torch.float32, device=device))
        self.register_buffer("act_global_scale", torch.tensor([gs], dtype=torch.float32, device=device))
        cols = in_features if config.transform_init == "wush" else g
        self.register_buffer("forward_hadamard_matrix", torch.zeros(g, cols, **kw))
        self._scales_blocked: Optional[torch.Tensor] = None
        self._alpha: Optional[torch.Tensor] = None

    # -- weights ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def pre_forward(self) -> None:
        """Build the transform (unless it is a WUSH matrix, which is loaded) and quantize ``weight`` once
        (reference: linear.py:165-265)."""
        cfg, g = self.config, self.config.hadamard_group_size
        dev, dt = self.weight.device, self.weight.dtype
        if cfg.transform_init == "hadamard":
            self.forward_hadamard_matrix = _hadamard(g, dev, dt)
        elif cfg.transform_init == "identity":
            self.forward_hadamard_matrix = torch.eye(g, device=dev, dtype=dt)
        elif cfg.transform_init != "wush":
            raise ValueError(f"Invalid transform init: {cfg.transform_init}")
        if cfg.transform_init == "wush":
            return                      # weights and matrix arrive through load_quantized()
        q, s = forward_quantize(self.weight.data, self.forward_hadamard_matrix, self.weight_global_scale,
                                cfg.forward_dtype, cfg.forward_method)
        self.load_quantized(q, s[: self.out_features, : self.in_features // g], self.forward_hadamard_matrix)

    @torch.no_grad()
    def load_quantized(self, qweight: torch.Tensor, scales: torch.Tensor, matrix: torch.Tensor,
                       weight_global_scale: Optional[torch.Tensor] = None,
                       act_global_scale: Optional[torch.Tensor] = None) -> None:
        """Take the tensors of an exported realquant checkpoint (names as in wush_gptq.py:592-599)."""
        dev = self.qweight.device
        self.qweight = qweight.view(torch.uint8).to(dev).contiguous()
        self.scales = scales.view(torch.uint8).to(dev).contiguous()
        self.forward_hadamard_matrix = matrix.to(device=dev, dtype=torch.bfloat16).contiguous()
        if weight_global_scale is not None:
            self.weight_global_scale = weight_global_scale.to(device=dev, dtype=torch.float32).reshape(1)
        if act_global_scale is not None:
            self.act_global_scale = act_global_scale.to(device=dev, dtype=torch.float32).reshape(1)
        self._scales_blocked = ops.to_blocked(self.scales)          # once, not per call
        self._alpha = (1.0 / (self.weight_global_scale * self.act_global_scale)).float()
        self.weight = None

    # -- forward ---------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._scales_blocked is None:
            raise RuntimeError("call pre_forward() or load_quantized() first")
        cfg = self.config
        x_flat = x.contiguous().flatten(end_dim=-2)
        xq, xs = forward_quantize(x_flat, self.forward_hadamard_matrix, self.act_global_scale, cfg.forward_dtype,
                                  cfg.forward_method, blocked=True)
        y = ops.matmul_fp4_blocked(xq, self.qweight, xs.view(-1), self._scales_blocked.view(-1), self._alpha,
                                   _fmt(cfg.forward_dtype))
        y = y.unflatten(0, x.shape[:-1])
        if self.bias is not None:
            y = y + self.bias
        return y
