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
    transform_init: str = "hadamard"            # "hadamard" | "identity" | "gsr" | "wush"
    modules_to_not_convert: List[str] = field(default_factory=lambda: ["lm_head"])


def validate_config(config: FPQuantConfig) -> None:
    if config.forward_dtype not in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4):
        raise ValueError(f"Unsupported forward dtype: {config.forward_dtype}")
    if config.forward_method not in ("abs_max", "quest"):
        raise ValueError(f"Unsupported forward method: {config.forward_method}")
    if config.forward_method == "quest" and config.forward_dtype == FPQuantDtype.MXFP4 and config.transform_init == "wush":
        # the reference's per-group op ignores the method (qutlass_ops.py:110-125) while its layer sets the global
        # scales for it (linear.py:207-211): the two do not fit together there either
        raise NotImplementedError("forward_method='quest' needs a shared square transform (hadamard or identity)")
    # inference_lib/src/fp_quant/utils/config.py:35-50: 32 / 64 / 128 for MXFP4, also 16 for NVFP4; a per-group (WUSH)
    # matrix is always as wide as the quantization group
    want = (32, 64, 128) if config.forward_dtype == FPQuantDtype.MXFP4 else (16, 32, 64, 128)
    if config.hadamard_group_size not in want:
        raise ValueError(f"{config.forward_dtype.value} can only be used with hadamard_group_size in {list(want)}")
    if config.transform_init == "wush" and config.hadamard_group_size != want[0]:
        raise NotImplementedError(f"per-group WUSH matrices are {want[0]} wide for {config.forward_dtype.value}")
    if config.store_master_weights or config.pseudoquantization or config.backward_dtype != FPQuantDtype.BF16:
        raise NotImplementedError("inference only: no master weights, pseudo-quantization or quantized backward")


def _fmt(dtype: FPQuantDtype) -> str:
    return "mx" if dtype == FPQuantDtype.MXFP4 else "nv"


def forward_quantize(x: torch.Tensor, hadamard_matrix: torch.Tensor, global_scale: torch.Tensor, dtype: FPQuantDtype,
                     forward_method: str, blocked: bool = False):
    """(codes u8, scales u8) of a 2-D bf16 tensor; reference: linear_fns.py:29-62.  With ``blocked`` the
    scales come out in the layout the GEMM consumes (no separate re-layout pass).  As in the reference, the method
    only matters for MXFP4 with a shared square transform: "quest" scales by the group's standard deviation."""
    if forward_method not in ("abs_max", "quest"):
        raise ValueError(f"Unsupported forward method: {forward_method}")
    layout = _lib.SF_BLOCKED if blocked else _lib.SF_ROW_MAJOR
    gs = global_scale.float() if dtype == FPQuantDtype.NVFP4 else None
    quest = (forward_method == "quest" and dtype == FPQuantDtype.MXFP4
             and hadamard_matrix.shape[0] == hadamard_matrix.shape[1])
    return ops._quantize(x.to(torch.bfloat16), hadamard_matrix.to(torch.bfloat16), _fmt(dtype), gs, sf_layout=layout,
                         quest=quest)


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
        qg = 32 if config.forward_dtype == FPQuantDtype.MXFP4 else 16     # scale group, whatever the transform size
        if in_features % g != 0:
            raise ValueError(f"in_features must be divisible by the hadamard group size ({g})")
        self.register_buffer("scales", torch.empty(out_features, in_features // qg, dtype=torch.uint8, device=device))
        # 3.0 whenever the method is abs_max, for both formats, like the reference's pre_forward (linear.py:206-217:
        # its abs_max branch comes before the NVFP4 one); exported WUSH checkpoints carry their own value (10.0 for
        # NVFP4, wush_gptq.py:588) and overwrite it through the state dict.  Buffers in the module dtype, as there.
        # MXFP4 with the quest method: 1.0 (its codes carry no implicit factor); NVFP4 with quest: 10.0 (ibid.)
        if config.forward_method == "quest":
            gsv = 1.0 if config.forward_dtype == FPQuantDtype.MXFP4 else 10.0
        else:
            gsv = 3.0
        self.register_buffer("weight_global_scale", torch.tensor([gsv], **kw))
        self.register_buffer("act_global_scale", torch.tensor([gsv], **kw))
        cols = in_features if config.transform_init == "wush" else g
        self.register_buffer("forward_hadamard_matrix", torch.zeros(g, cols, **kw))
        self.register_buffer("backward_hadamard_matrix", torch.zeros(g, cols, **kw))
        # blocked weight scales and alpha are derived from the buffers on first use and whenever the buffers are
        # replaced or written (load_state_dict copies in place, .to() / .cuda() replace the tensors)
        self._derived_key = None
        self._scales_blocked: Optional[torch.Tensor] = None
        self._alpha: Optional[torch.Tensor] = None
        self._quantized = False

    # -- weights ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def pre_forward(self) -> None:
        """Build the transform (unless it is a WUSH matrix, which is loaded) and quantize ``weight`` once
        (reference: linear.py:165-265)."""
        cfg, g = self.config, self.config.hadamard_group_size
        if cfg.transform_init == "wush" or self.weight is None:
            # the matrix and the quantized weights come from the checkpoint (linear.py:183-186); they may already
            # have been copied into the buffers by load_state_dict
            self.weight = None
            self._quantized = True
            return
        dev, dt = self.weight.device, self.weight.dtype
        if cfg.transform_init == "hadamard":
            mat = _hadamard(g, dev, dt)
        elif cfg.transform_init == "identity":
            mat = torch.eye(g, device=dev, dtype=dt)
        elif cfg.transform_init == "gsr":
            # the Hadamard columns ordered by their number of sign changes (reference: get_gsr_matrix, linear.py:44-48)
            h = _hadamard(g, dev, dt)
            mat = h[:, torch.argsort(torch.diff(h, dim=0).ne(0).sum(dim=0))].contiguous()
        else:
            raise ValueError(f"Invalid transform init: {cfg.transform_init}")
        q, s = forward_quantize(self.weight.data, mat, self.weight_global_scale, cfg.forward_dtype, cfg.forward_method)
        qg = 32 if cfg.forward_dtype == FPQuantDtype.MXFP4 else 16
        self.load_quantized(q, s[: self.out_features, : self.in_features // qg], mat)

    @torch.no_grad()
    def load_quantized(self, qweight: torch.Tensor, scales: torch.Tensor, matrix: torch.Tensor,
                       weight_global_scale: Optional[torch.Tensor] = None,
                       act_global_scale: Optional[torch.Tensor] = None) -> None:
        """Take the tensors of an exported realquant checkpoint (names as in wush_gptq.py:592-599)."""
        dev = self.qweight.device
        dt = self.forward_hadamard_matrix.dtype
        self.qweight = qweight.view(torch.uint8).to(dev).contiguous()
        self.scales = scales.view(torch.uint8).to(dev).contiguous()
        self.forward_hadamard_matrix = matrix.to(device=dev, dtype=dt).contiguous()
        self.backward_hadamard_matrix = self.forward_hadamard_matrix.clone()
        if weight_global_scale is not None:
            self.weight_global_scale = weight_global_scale.to(device=dev, dtype=dt).reshape(1)
        if act_global_scale is not None:
            self.act_global_scale = act_global_scale.to(device=dev, dtype=dt).reshape(1)
        self.weight = None
        self._quantized = True

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        """A checkpoint that carries ``qweight`` is a quantized one: its tensors land in the buffers (a bf16
        ``weight`` is then neither expected nor kept), which is the reference's loading protocol."""
        if prefix + "qweight" in state_dict:
            if prefix + "weight" not in state_dict:
                self.weight = None
            self._quantized = True
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def _derived(self):
        """(blocked weight scales, alpha) for the buffers as they are now."""
        s, wg, ag = self.scales, self.weight_global_scale, self.act_global_scale
        key = (s.data_ptr(), s._version, s.device, wg.data_ptr(), wg._version, ag.data_ptr(), ag._version)
        if key != self._derived_key:
            self._scales_blocked = ops.to_blocked(s.contiguous())          # once per set of weights, not per call
            self._alpha = (1.0 / (wg.float() * ag.float())).reshape(1)
            self._derived_key = key
        return self._scales_blocked, self._alpha

    # -- forward ---------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y = x W^T (+ bias) (+ residual): quantize the activations with the layer's transform, multiply in FP4
        (reference: FPQuant4x16NoMasterFn.forward, linear_fns.py:494-539).  Bias and the optional residual
        are added in the GEMM's epilogue."""
        if not self._quantized:
            raise RuntimeError("call pre_forward() or load_quantized(), or load a quantized state dict, first")
        cfg = self.config
        scales_blocked, alpha = self._derived()
        x_flat = x.contiguous().flatten(end_dim=-2)
        xq, xs = forward_quantize(x_flat, self.forward_hadamard_matrix, self.act_global_scale, cfg.forward_dtype,
                                  cfg.forward_method, blocked=True)
        res = residual.contiguous().flatten(end_dim=-2) if residual is not None else None
        y = ops.matmul_fp4_blocked(xq, self.qweight, xs.view(-1), scales_blocked.view(-1), alpha,
                                   _fmt(cfg.forward_dtype), bias=self.bias, residual=res)
        return y.unflatten(0, x.shape[:-1])
