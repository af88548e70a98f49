"""Hessian accumulation for GPTQ/WUSH calibration, backed by the sm_100a tensor-core kernel.

``accumulate_hessian`` keeps the signature and in-place semantics of the reference's wrapper at
src/quantization/accumulate_hessian.py:112-148.
"""
from __future__ import annotations

import torch

from . import _lib


def accumulate_hessian(mat_hessian: torch.Tensor, mat_input: torch.Tensor, save_lower_only: bool = False,
                       compute_lower_only: bool = True) -> torch.Tensor:
    """In place ``mat_hessian += mat_input^T @ mat_input``; returns ``mat_hessian``.

    mat_hessian: ([meta,] hidden, hidden) fp32, contiguous, on a CUDA device.
    mat_input:   ([meta,] tokens, hidden) bf16, contiguous.
    save_lower_only: update only the lower triangle (incl. diagonal) and leave the rest untouched.
    compute_lower_only: kept for signature compatibility; the kernel always computes the lower
        triangle and mirrors it, which gives the same (symmetric) result.
    """
    assert compute_lower_only or not save_lower_only, "compute_lower_only must be True when save_lower_only is True"
    assert mat_hessian.is_contiguous() and mat_input.is_contiguous()
    if not (mat_hessian.is_cuda and mat_input.is_cuda):
        raise _lib.WushB200Error("accumulate_hessian needs CUDA tensors; there is no CPU fallback")
    if mat_hessian.dtype != torch.float32:
        raise ValueError("mat_hessian must be float32")
    if mat_input.dtype != torch.bfloat16:
        raise NotImplementedError(f"mat_input dtype {mat_input.dtype}: the kernel takes bfloat16 activations")
    *meta, tokens, hidden = mat_input.shape
    if tuple(mat_hessian.shape) != (*meta, hidden, hidden):
        raise ValueError(f"shape mismatch: hessian {tuple(mat_hessian.shape)} vs input {tuple(mat_input.shape)}")
    h3 = mat_hessian.view(-1, hidden, hidden)
    x3 = mat_input.view(-1, tokens, hidden)
    lib = _lib.load()
    flags = _lib.HESSIAN_LOWER_ONLY if save_lower_only else 0
    with torch.cuda.device(mat_input.device):
        stream = torch.cuda.current_stream().cuda_stream
        for b in range(h3.shape[0]):
            rc = lib.wush_hessian_accumulate(h3[b].data_ptr(), x3[b].data_ptr(), tokens, hidden, flags, None, stream)
            _lib.check(rc, "wush_hessian_accumulate")
    return mat_hessian
