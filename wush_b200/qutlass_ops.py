"""Operator surface of the quantized linear layer, backed by the sm_100a library.

Drop-in for ``inference_lib/src/fp_quant/module/qutlass_ops.py`` of the reference: the same
callable names, argument meaning, output shapes/dtypes (including the 128-row / 4-column padding
of the scale tensors) and fake (meta) implementations, so ``forward_quantize`` /
``forward_gemm`` in ``linear_fns.py`` work unchanged when they import from here.  The torch
custom ops live in the ``wush_b200`` namespace so that they can coexist with the reference's
``fp_quant`` namespace in one process.

Every op runs a hand-written CUDA kernel through the C ABI; a tensor that is not on a CUDA
device, or a missing library, raises.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

HAS_QUTLASS = True  # the reference gates its real-quant path on this name


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise _lib.WushB200Error("wush_b200 ops need CUDA tensors; there is no CPU fallback")


def _padded_scale_shape(rows: int, groups: int) -> Tuple[int, int]:
    return (rows + 127) // 128 * 128, (groups + 3) // 4 * 4


def _alloc_scales(rows: int, groups: int, device) -> torch.Tensor:
    pr, pc = _padded_scale_shape(rows, groups)
    if pr == rows and pc == groups:
        return torch.empty(pr, pc, dtype=torch.uint8, device=device)
    return torch.zeros(pr, pc, dtype=torch.uint8, device=device)  # the kernel skips the padding


def _quantize(x_flat: torch.Tensor, matrix: torch.Tensor, fmt: str, global_scale: Optional[torch.Tensor],
              sf_layout: int = _lib.SF_ROW_MAJOR, round_bf16: bool = False, quest: bool = False,
              clip_mask: Optional[torch.Tensor] = None):
    """quest (MXFP4 only): standard-deviation scale with clipping; clip_mask: u8 [rows, cols/8] the kernel fills."""
    _require_cuda(x_flat, matrix, global_scale)
    if quest and fmt != "mx":
        raise ValueError("the quest method exists for MXFP4 only")
    if x_flat.dim() != 2:
        raise ValueError("x_flat must be 2-D (tokens, channels)")
    if x_flat.dtype != torch.bfloat16 or matrix.dtype != torch.bfloat16:
        raise ValueError("x_flat and the transform matrix must be bfloat16")
    group = 32 if fmt == "mx" else 16
    rows, cols = x_flat.shape
    if cols % 32 != 0:
        raise ValueError(f"channels ({cols}) must be a multiple of 32")
    # a square matrix wider than the group: one Hadamard-type transform per block of n channels (n = 64, 128; 32 for nv)
    wide = matrix.dim() == 2 and matrix.shape[0] == matrix.shape[1] and matrix.shape[0] > group
    if wide:
        if matrix.shape[0] not in (32, 64, 128) or cols % matrix.shape[0] != 0 or round_bf16:
            raise NotImplementedError(
                f"shared transform of shape {tuple(matrix.shape)} on {cols} channels: the size must be 64 or 128 (32 for "
                f"nvfp4) and divide the channels; not with round_bf16")
    elif matrix.dim() != 2 or matrix.shape[0] != group or matrix.shape[1] not in (group, cols):
        raise NotImplementedError(
            f"transform matrix of shape {tuple(matrix.shape)}: supported are ({group}, {group}) shared, "
            f"({group}, {cols}) per-group and square shared matrices of 64 or 128 channels")
    x_flat = x_flat.contiguous()
    matrix = matrix.contiguous()
    q = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x_flat.device)
    sf = _alloc_scales(rows, cols // group, x_flat.device)
    lib = _lib.load()
    if rows == 0:
        return q, sf
    flags = (_lib.QUANT_ROUND_BF16 if round_bf16 else 0) | (_lib.QUANT_WIDE_MATRIX if wide else 0)
    with torch.cuda.device(x_flat.device):
        if quest:
            rc = lib.wush_fused_quantize_mx_quest(x_flat.data_ptr(), matrix.data_ptr(), matrix.shape[1], q.data_ptr(),
                                                  sf.data_ptr(), sf.shape[1], sf_layout,
                                                  clip_mask.data_ptr() if clip_mask is not None else None, rows, cols,
                                                  flags, _stream(x_flat))
        elif fmt == "mx":
            rc = lib.wush_fused_quantize_mx(x_flat.data_ptr(), matrix.data_ptr(), matrix.shape[1], q.data_ptr(),
                                            sf.data_ptr(), sf.shape[1], sf_layout, rows, cols, flags, _stream(x_flat))
        else:
            gs = global_scale.to(device=x_flat.device, dtype=torch.float32).reshape(-1)[:1].contiguous()
            rc = lib.wush_fused_quantize_nv(x_flat.data_ptr(), matrix.data_ptr(), matrix.shape[1], gs.data_ptr(),
                                            q.data_ptr(), sf.data_ptr(), sf.shape[1], sf_layout, rows, cols, flags,
                                            _stream(x_flat))
    _lib.check(rc, f"wush_fused_quantize_{fmt}{'_quest' if quest else ''}")
    return q, sf


def fused_quantize_into(x: torch.Tensor, matrix: torch.Tensor, fmt: str, global_scale: Optional[torch.Tensor],
                        q_out: torch.Tensor, sf_out: torch.Tensor, col0: int = 0, sf_layout: int = _lib.SF_BLOCKED,
                        round_bf16: bool = False, row_scale: Optional[torch.Tensor] = None,
                        col_scale: Optional[torch.Tensor] = None) -> None:
    """Transform + quantize the columns ``x`` holds and write them into a wider GEMM operand: codes into
    ``q_out[:, col0/2 : (col0 + cols)/2]`` and scales into the matching groups of ``sf_out`` (the scale tensor of the
    WHOLE operand: ``ceil(K/G/4)*4`` bytes per row, row-major 2-D or blocked).  ``x`` may be a column slice of a wider
    tensor.  This is how a layer whose input columns are spread over GPUs assembles its quantized operand: scale
    groups never straddle a shard, so every GPU quantizes what it holds.

    ``row_scale`` (fp32 [rows]) and ``col_scale`` (bf16 [cols]) fold an RMSNorm into the call: the kernel quantizes
    ``bf16(bf16(x * row_scale[:, None]) * col_scale)`` without that tensor ever being written."""
    _require_cuda(x, matrix, global_scale, q_out, sf_out, row_scale, col_scale)
    if (row_scale is None) != (col_scale is None):
        raise ValueError("row_scale and col_scale go together")
    if row_scale is not None:
        if row_scale.dtype != torch.float32 or row_scale.numel() != x.shape[0] or not row_scale.is_contiguous():
            raise ValueError("row_scale must be a contiguous float32 [rows] tensor")
        if col_scale.dtype != torch.bfloat16 or col_scale.numel() != x.shape[1] or not col_scale.is_contiguous():
            raise ValueError("col_scale must be a contiguous bfloat16 [cols] tensor")
    group = 32 if fmt == "mx" else 16
    rows, cols = x.shape
    if x.dtype != torch.bfloat16 or matrix.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise ValueError("x and the transform matrix must be bfloat16, x with unit column stride")
    if q_out.dtype != torch.uint8 or q_out.dim() != 2 or q_out.shape[0] < rows or q_out.stride(1) != 1:
        raise ValueError("q_out must be a uint8 [rows, K/2] tensor")
    k_total = q_out.shape[1] * 2
    if col0 % (4 * group) or col0 + cols > k_total:
        raise ValueError(f"col0 must be a multiple of {4 * group} and the slice must fit into the operand")
    sf_cols = (k_total // group + 3) // 4 * 4
    pr = (rows + 127) // 128 * 128
    if sf_out.numel() < (pr if sf_layout == _lib.SF_BLOCKED else rows) * sf_cols:
        raise ValueError("sf_out is smaller than the operand's scale tensor")
    matrix = matrix.contiguous()
    if rows == 0:
        return
    gs = None
    if fmt == "nv":
        gs = global_scale.to(device=x.device, dtype=torch.float32).reshape(-1)[:1].contiguous()
    with torch.cuda.device(x.device):
        rc = _lib.load().wush_fused_quantize_strided(
            _lib.FORMAT_MXFP4 if fmt == "mx" else _lib.FORMAT_NVFP4, x.data_ptr(), x.stride(0), matrix.data_ptr(),
            matrix.shape[1], gs.data_ptr() if gs is not None else None, q_out.data_ptr() + col0 // 2, q_out.stride(0),
            sf_out.data_ptr(), sf_cols, sf_layout, col0 // group, row_scale.data_ptr() if row_scale is not None else None,
            col_scale.data_ptr() if col_scale is not None else None, rows, cols,
            _lib.QUANT_ROUND_BF16 if round_bf16 else 0, _stream(x))
    _lib.check(rc, "wush_fused_quantize_strided")


def row_sumsq(x: torch.Tensor) -> torch.Tensor:
    """fp32 [rows]: sum of squares of every row of a bf16 matrix (rows may be strided)."""
    _require_cuda(x)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D bfloat16 tensor with unit column stride")
    out = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().wush_row_sumsq(x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], _stream(x))
    _lib.check(rc, "wush_row_sumsq")
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """bf16(silu(gate)) * up for two bf16 [rows, cols] tensors with a common row stride (e.g. column halves of one
    fused projection output)."""
    _require_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.dim() != 2 \
            or gate.stride() != up.stride() or gate.stride(1) != 1:
        raise ValueError("gate and up must be bfloat16 [rows, cols] tensors with the same strides")
    out = torch.empty(gate.shape, dtype=torch.bfloat16, device=gate.device)
    with torch.cuda.device(gate.device):
        rc = _lib.load().wush_swiglu(gate.data_ptr(), up.data_ptr(), gate.stride(0), out.data_ptr(), out.stride(0),
                                     gate.shape[0], gate.shape[1], _stream(gate))
    _lib.check(rc, "wush_swiglu")
    return out


# --------------------------------------------------------------------------------------------
# forward quantization (reference: qutlass_ops.py:37-143)
# --------------------------------------------------------------------------------------------

@torch.library.custom_op("wush_b200::fused_quantize_mx_op", mutates_args=())
def _fused_quantize_mx(x_flat: torch.Tensor, hadamard_matrix: torch.Tensor, forward_method: str,
                       return_mask: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if forward_method not in ("abs_max", "quest"):
        raise ValueError(f"Unsupported forward method: {forward_method}")
    rows, cols = x_flat.shape
    if forward_method == "quest":
        mask = torch.empty(rows, cols // 8 if return_mask else 0, dtype=torch.uint8, device=x_flat.device)
        q, sf = _quantize(x_flat, hadamard_matrix, "mx", None, quest=True, clip_mask=mask if return_mask else None)
    else:
        # the absolute-maximum scale never clips (|3 y / scale| < 6): every bit of the packed mask is set
        mask = torch.full((rows, cols // 8 if return_mask else 0), 0xFF, dtype=torch.uint8, device=x_flat.device)
        q, sf = _quantize(x_flat, hadamard_matrix, "mx", None)
    return q, sf.view(torch.float8_e8m0fnu), mask


@_fused_quantize_mx.register_fake
def _(x_flat, hadamard_matrix, forward_method, return_mask):
    rows, groups = x_flat.size(0), x_flat.size(1) // 32
    pr, pc = _padded_scale_shape(rows, groups)
    return (torch.empty(rows, x_flat.size(1) // 2, dtype=torch.uint8, device=x_flat.device),
            torch.empty(pr, pc, dtype=torch.float8_e8m0fnu, device=x_flat.device),
            torch.empty(rows, groups * 4 if return_mask else 0, dtype=torch.uint8, device=x_flat.device))


def fused_quantize_mx_op(x_flat: torch.Tensor, hadamard_matrix: torch.Tensor, forward_method: str,
                         return_mask: bool):
    """(e2m1 u8 [T, C/2], e8m0 [ceil(T/128)*128, ceil(C/32/4)*4], packed clip mask u8 [T, C/8] | None).
    forward_method "abs_max" or "quest".  Reference: qutlass_ops.py:37-72 (shared square transform)."""
    q, sf, mask = _fused_quantize_mx(x_flat, hadamard_matrix, forward_method, return_mask)
    return q, sf, (mask if return_mask else None)


def fused_quantize_mx_wush_op(x_flat: torch.Tensor, wush_matrix: torch.Tensor, forward_method: str,
                              return_mask: bool):
    """Per-group 32x32 transform given as a (32, C) matrix.  Like the reference's op (qutlass_ops.py:110-143, whose
    kernel takes no method), this one always uses the absolute-maximum scale whatever `forward_method` says."""
    q, sf, mask = _fused_quantize_mx(x_flat, wush_matrix, "abs_max", return_mask)
    return q, sf, (mask if return_mask else None)


@torch.library.custom_op("wush_b200::fused_quantize_nv_op", mutates_args=())
def fused_quantize_nv_op(x_flat: torch.Tensor, hadamard_matrix: torch.Tensor,
                         global_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e2m1 u8 [T, C/2], e4m3 [ceil(T/128)*128, ceil(C/16/4)*4]).  Reference: qutlass_ops.py:75-106.
    The matrix may be (16, 16) shared or, beyond the reference, (16, C) per-group WUSH."""
    q, sf = _quantize(x_flat, hadamard_matrix, "nv", global_scale)
    return q, sf.view(torch.float8_e4m3fn)


@fused_quantize_nv_op.register_fake
def _(x_flat, hadamard_matrix, global_scale):
    rows, groups = x_flat.size(0), x_flat.size(1) // 16
    pr, pc = _padded_scale_shape(rows, groups)
    return (torch.empty(rows, x_flat.size(1) // 2, dtype=torch.uint8, device=x_flat.device),
            torch.empty(pr, pc, dtype=torch.float8_e4m3fn, device=x_flat.device))


def fused_quantize_debug(x_flat: torch.Tensor, matrix: torch.Tensor, fmt: str,
                         global_scale: Optional[torch.Tensor] = None, round_bf16: bool = False,
                         sf_layout: int = _lib.SF_ROW_MAJOR):
    """Validation entry: (q, sf u8, transformed fp32 [T, C]) -- the quantize kernel with its
    transform output also written out."""
    _require_cuda(x_flat, matrix)
    group = 32 if fmt == "mx" else 16
    rows, cols = x_flat.shape
    x_flat, matrix = x_flat.contiguous(), matrix.contiguous()
    q = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x_flat.device)
    sf = _alloc_scales(rows, cols // group, x_flat.device)
    tr = torch.empty(rows, cols, dtype=torch.float32, device=x_flat.device)
    gs = None
    if fmt == "nv":
        gs = global_scale.to(device=x_flat.device, dtype=torch.float32).reshape(-1)[:1].contiguous()
    lib = _lib.load()
    with torch.cuda.device(x_flat.device):
        rc = lib.wush_fused_quantize_debug(0 if fmt == "mx" else 1, x_flat.data_ptr(), matrix.data_ptr(),
                                           matrix.shape[1], gs.data_ptr() if gs is not None else None, q.data_ptr(),
                                           sf.data_ptr(), sf.shape[1], sf_layout, tr.data_ptr(), rows, cols,
                                           _lib.QUANT_ROUND_BF16 if round_bf16 else 0, _stream(x_flat))
    _lib.check(rc, "wush_fused_quantize_debug")
    return q, sf, tr


# --------------------------------------------------------------------------------------------
# scale layout (reference: qutlass_ops.py:372-373)
# --------------------------------------------------------------------------------------------

def to_blocked(x: torch.Tensor) -> torch.Tensor:
    """Row-major scales (any 1-byte dtype) -> flat blocked layout, same dtype."""
    _require_cuda(x)
    if x.dim() != 2 or x.element_size() != 1:
        raise ValueError("to_blocked expects a 2-D tensor of 1-byte scales")
    x = x.contiguous()
    rows, cols = x.shape
    pr, pc = _padded_scale_shape(rows, cols)
    out = torch.empty(pr * pc, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().wush_sf_to_blocked(x.view(torch.uint8).data_ptr(), out.data_ptr(), rows, cols, _stream(x))
    _lib.check(rc, "wush_sf_to_blocked")
    return out.view(x.dtype)


# --------------------------------------------------------------------------------------------
# GEMMs (reference: qutlass_ops.py:149-206)
# --------------------------------------------------------------------------------------------

def matmul_fp4_blocked(x: torch.Tensor, w: torch.Tensor, xs_blocked: torch.Tensor, ws_blocked: torch.Tensor,
                       alpha: torch.Tensor, fmt: str, splits: int = 0, bias: Optional[torch.Tensor] = None,
                       residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                       rows: Optional[int] = None, scale_shard_bytes: int = 0) -> torch.Tensor:
    """y = alpha * deq(x) @ deq(w)^T in bf16 with scales ALREADY in the blocked layout (what
    ``to_blocked`` returns, or what the fused quantize kernel writes with ``sf_layout=SF_BLOCKED``).
    x: (..., K/2) u8, w: (N, K/2) u8; fmt 'mx' (E8M0 per 32) or 'nv' (E4M3 per 16).

    ``bias`` (bf16 [N]) and ``residual`` (bf16 [..., N], may be ``out``) are added inside the GEMM's epilogue
    with the roundings of the separate steps they replace (``y += bias`` after forward_gemm, linear_fns.py:523-525,
    and the decoder block's ``hidden = residual + y``).  ``out`` (bf16 [..., N], rows may be strided) receives the
    result instead of a new tensor.

    ``rows`` given: ``x`` is a STACK of K shards, uint8 [shards, rows_alloc, K/shards/2] (rows_alloc >= rows), and
    ``xs_blocked`` the stack of their blocked scale tensors -- activations whose columns were quantized in pieces
    (on different GPUs) and copied side by side; the first ``rows`` rows of every piece are multiplied.
    ``scale_shard_bytes`` is the distance between the scale tensors of two pieces when they are not densely stacked."""
    _require_cuda(x, w, xs_blocked, ws_blocked, alpha, bias, residual, out)
    if x.dtype != torch.uint8 or w.dtype != torch.uint8:
        raise ValueError("packed FP4 operands must be uint8")
    group = 32 if fmt == "mx" else 16
    w = w.contiguous()
    n = w.shape[0]
    a_shards, a_shard_rows = 1, 0
    if rows is not None:
        if x.dim() != 3 or not x.is_contiguous() or rows > x.shape[1]:
            raise ValueError("a stacked operand must be a contiguous [shards, rows_alloc, K/shards/2] tensor")
        a_shards, a_shard_rows, kb = x.shape[0], x.shape[1], x.shape[0] * x.shape[2]
        lead, x2, m = (rows,), x, rows
        if (x.shape[2] * 2) % 256:
            raise ValueError("every K shard must be a multiple of 256 columns")
        need_a = (a_shards - 1) * scale_shard_bytes + (rows + 127) // 128 * 128 * (x.shape[2] * 2 // group) \
            if scale_shard_bytes else a_shards * ((a_shard_rows + 127) // 128 * 128) * (x.shape[2] * 2 // group)
    else:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        m, kb = x2.shape
        need_a = (m + 127) // 128 * 128 * ((kb * 2 // group + 3) // 4 * 4)
    if w.shape[1] != kb:
        raise ValueError(f"K mismatch: x has {kb * 2}, w has {w.shape[1] * 2}")
    k = kb * 2
    if xs_blocked.numel() < need_a or ws_blocked.numel() < (n + 127) // 128 * 128 * ((k // group + 3) // 4 * 4):
        raise ValueError("blocked scale tensor smaller than ceil(rows/128)*128 x ceil(K/G/4)*4")

    def rows_2d(t: torch.Tensor, what: str) -> torch.Tensor:
        t2 = t.reshape(-1, t.shape[-1]) if t.dim() != 2 else t
        if t2.dtype != torch.bfloat16 or tuple(t2.shape) != (m, n) or (m > 0 and t2.stride(1) != 1):
            raise ValueError(f"{what} must be bfloat16 of shape (..., {n}) with unit column stride")
        return t2

    y = torch.empty(m, n, dtype=torch.bfloat16, device=x.device) if out is None else rows_2d(out, "out")
    if m == 0:
        return y.reshape(*lead, n)
    res2 = rows_2d(residual, "residual") if residual is not None else None
    if bias is not None and (bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,)):
        raise ValueError(f"bias must be bfloat16 of shape ({n},)")
    lib = _lib.load()
    al = alpha.to(device=x.device, dtype=torch.float32).reshape(-1)[:1].contiguous()
    with torch.cuda.device(x.device):
        ws_bytes = int(lib.wush_gemm_workspace_bytes(m, n, k, splits))
        work = _lib.gemm_workspace(x.device, ws_bytes) if ws_bytes else None
        rc = lib.wush_gemm_fp4_bf16_tn_fused(
            _lib.FORMAT_MXFP4 if fmt == "mx" else _lib.FORMAT_NVFP4, x2.data_ptr(), a_shards, a_shard_rows, scale_shard_bytes,
            w.data_ptr(),
            xs_blocked.data_ptr(),
            ws_blocked.data_ptr(), al.data_ptr(), bias.contiguous().data_ptr() if bias is not None else None,
            res2.data_ptr() if res2 is not None else None, res2.stride(0) if res2 is not None else 0, y.data_ptr(),
            y.stride(0), m, n, k, work.data_ptr() if work is not None else None, work.numel() if work is not None else 0,
            splits, _lib.status_word(x.device).data_ptr(), _stream(x))
    _lib.check(rc, f"wush_gemm_{fmt}f4_bf16_tn")
    if _lib.CHECK_EVERY_OP:
        _lib.check_status(x.device, "FP4 GEMM")
    return y.reshape(*lead, n) if out is None else out


@torch.library.custom_op("wush_b200::matmul_mxf4_bf16_tn_op", mutates_args=())
def matmul_mxf4_bf16_tn_op(x: torch.Tensor, w: torch.Tensor, xs: torch.Tensor, ws: torch.Tensor,
                           alpha: torch.Tensor) -> torch.Tensor:
    """Reference: qutlass_ops.py:149-163.  xs / ws are ROW-MAJOR scales (E8M0 bytes, any 1-byte dtype) as
    the fused quantize op returns them; they are re-laid into the blocked layout here, like the reference."""
    return matmul_fp4_blocked(x, w, to_blocked(xs.view(torch.uint8)), to_blocked(ws.view(torch.uint8)), alpha, "mx")


@matmul_mxf4_bf16_tn_op.register_fake
def _(x, w, xs, ws, alpha):
    return x.new_empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16)


@torch.library.custom_op("wush_b200::matmul_nvf4_bf16_tn_op", mutates_args=())
def matmul_nvf4_bf16_tn_op(x: torch.Tensor, w: torch.Tensor, xs: torch.Tensor, ws: torch.Tensor,
                           alpha: torch.Tensor) -> torch.Tensor:
    """Reference: qutlass_ops.py:187-201 (E4M3 scales per 16 elements)."""
    return matmul_fp4_blocked(x, w, to_blocked(xs.view(torch.uint8)), to_blocked(ws.view(torch.uint8)), alpha, "nv")


@matmul_nvf4_bf16_tn_op.register_fake
def _(x, w, xs, ws, alpha):
    return x.new_empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16)
