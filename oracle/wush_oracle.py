"""CPU oracle for the WUSH hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This module restates, in NumPy float64, the arithmetic of the reference's pure-torch
quantizer for the path the CUDA kernels replace.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it; the product package never
does (the product fails loudly when its CUDA library is missing).

Every function cites the reference file:line it follows (paths are relative to the
reference project root).  The restatement is pinned two ways:

* ``tests/golden/*.npz`` hold input/output vectors produced by importing and running
  the reference's own functions (generator: ``tests/golden/make_golden.py``);
  ``tests/test_oracle_golden.py`` checks this module against them bit for bit.
* when the reference checkout is present, ``oracle/check_against_reference.py``
  compares the two implementations directly on fresh seeded inputs.

The reference ships no golden vectors or numeric unit tests of its own, so those
fixtures (outputs of the reference's code executed on CPU) are the pin.

FP4 (E2M1) code convention: code = sign << 3 | index into [0, .5, 1, 1.5, 2, 3, 4, 6];
element 2i sits in the low nibble and element 2i+1 in the high nibble of byte i
(src/quantization/wush_gptq.py:48,70,84).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------
# formats
# ----------------------------------------------------------------------------------

#: Ascending signed E2M1 grid with both zeros, as the reference lays it out
#: (src/quantization/wush_gptq.py:47) and the matching 4-bit codes (:48, after & 0xF).
_GRID = np.array([-6., -4., -3., -2., -1.5, -1., -.5, -0., 0., .5, 1., 1.5, 2., 3., 4., 6.], dtype=np.float64)
_GRID_CODE = np.array([15, 14, 13, 12, 11, 10, 9, 8, 0, 1, 2, 3, 4, 5, 6, 7], dtype=np.uint8)
#: code -> value table used when unpacking (src/quantization/wush_gptq.py:84)
E2M1_VALUES = np.array([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.], dtype=np.float64)

#: quantizer constants (src/quantization/wush_gptq.py:388-407)
FORMATS = {
    "mxfp4": dict(group=32, scale="e8m0", scale_scale=4.0, global_scale=3.0),
    "nvfp4": dict(group=16, scale="e4m3", scale_scale=6.0, global_scale=10.0),
}


def _f32_bits(x64: np.ndarray) -> np.ndarray:
    """float64 -> float32 (round to nearest even) -> raw bits.  torch's float8 casts
    from float64 go through float32 first, which this mirrors."""
    with np.errstate(over="ignore", invalid="ignore"):
        return np.asarray(x64, dtype=np.float64).astype(np.float32).view(np.uint32)


def cast_e8m0(x64: np.ndarray) -> np.ndarray:
    """Scale cast ``tensor.to(torch.float8_e8m0fnu)`` used at
    src/quantization/wush_gptq.py:120 for MXFP4: returns the biased-exponent byte.

    Power-of-two rounding of a non-negative float32: keep the exponent field and add one
    when the top mantissa bit is set (round half up).  Byte 0 stands for 2**-127, so a
    float32 subnormal maps to byte 1 only when it lies strictly above 2**-127, and to byte
    0 otherwise (zero included) -- torch's behaviour, reproduced as observed.  Anything that rounds past 2**127, infinities and NaN
    give 0xFF.
    """
    b = _f32_bits(x64)
    exp = ((b >> 23) & 0xFF).astype(np.int64)
    half = ((b >> 22) & 1).astype(np.int64)
    out = exp + half
    out = np.where(exp == 0, ((b & 0x7FFFFF) > 0x400000).astype(np.int64), out)
    out = np.where(exp == 0xFF, 0xFF, out)
    return np.minimum(out, 0xFF).astype(np.uint8)


def e8m0_to_f64(byte: np.ndarray) -> np.ndarray:
    """Value of an E8M0 byte: 2**(byte-127); 0xFF is NaN."""
    byte = np.asarray(byte, dtype=np.uint8)
    v = np.ldexp(1.0, byte.astype(np.int64) - 127)
    return np.where(byte == 0xFF, np.nan, v)


def cast_e4m3(x64: np.ndarray) -> np.ndarray:
    """Scale cast ``tensor.to(torch.float8_e4m3fn)`` used at
    src/quantization/wush_gptq.py:120 for NVFP4: returns the raw byte.

    Round to nearest even onto 3 mantissa bits, exponent bias 7, subnormal step 2**-9,
    largest finite 448; no saturation -- a value that rounds above 448 becomes NaN
    (0x7F | sign), as in torch.
    """
    f = np.asarray(x64, dtype=np.float64).astype(np.float32).astype(np.float64)
    sign = np.signbit(f)
    a = np.abs(f)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, None)                       # subnormal range shares exponent -6
    step = np.ldexp(1.0, (e - 3).astype(np.int64))  # spacing of representable values
    q = np.rint(a / step) * step                   # np.rint is round-half-even
    # re-derive fields from the rounded magnitude
    with np.errstate(divide="ignore", invalid="ignore"):
        e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    e2 = np.clip(e2, -6, None)
    is_sub = q < 2.0 ** -6
    mant = np.where(is_sub, q / 2.0 ** -9, (q / np.ldexp(1.0, e2.astype(np.int64)) - 1.0) * 8.0)
    expf = np.where(is_sub, 0, e2 + 7)
    byte = (expf.astype(np.int64) << 3) | np.rint(mant).astype(np.int64)
    byte = np.where((q > 448.0) | ~np.isfinite(f), 0x7F, byte)
    byte = byte | (sign.astype(np.int64) << 7)
    return byte.astype(np.uint8)


def e4m3_to_f64(byte: np.ndarray) -> np.ndarray:
    """Value of an E4M3 (fn) byte; 0x7F / 0xFF are NaN."""
    byte = np.asarray(byte, dtype=np.uint8).astype(np.int64)
    s = np.where(byte & 0x80, -1.0, 1.0)
    e = (byte >> 3) & 0xF
    m = byte & 0x7
    v = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.ldexp(1.0, e - 7))
    v = np.where((byte & 0x7F) == 0x7F, np.nan, v)
    return s * v


# ----------------------------------------------------------------------------------
# a1: rtn_e2m1
# ----------------------------------------------------------------------------------

def rtn_e2m1(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Nearest E2M1 value of already-scaled numbers, ties to the even code.

    Follows src/quantization/wush_gptq.py:34-71 (mode='even'): locate x between two
    neighbours of the 16-entry signed grid (bucketize with right=False == searchsorted
    'left'), pick the nearer, and on an exact tie pick the upper neighbour iff its code
    is even.  Because the grid lists -0 before +0, an exact zero (and any x in
    (-0.25, 0]) gets code 8 (-0); NaN clamps to the last entry (code 7).

    Returns (values float64, codes uint8 in 0..15), same shape as x.
    """
    x = np.asarray(x, dtype=np.float64)
    inds = np.searchsorted(_GRID, x, side="left")          # NaN sorts last -> 16
    lo = np.clip(inds - 1, 0, 15)
    hi = np.clip(inds, 0, 15)
    g_lo, g_hi = _GRID[lo], _GRID[hi]
    # the reference tests the *signed int8* code for evenness; parity equals that of
    # the 4-bit code
    hi_even = (_GRID_CODE[hi] % 2) == 0
    with np.errstate(invalid="ignore"):
        d_hi, d_lo = g_hi - x, x - g_lo
        pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & hi_even)
    picked = np.where(pick_hi, hi, lo)
    return _GRID[picked], _GRID_CODE[picked]


def pack_e2m1(codes: np.ndarray) -> np.ndarray:
    """Two codes per byte, even element in the low nibble
    (src/quantization/wush_gptq.py:70)."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape[-1] % 2 == 0
    return ((codes[..., 1::2] & 0xF) << 4) | (codes[..., 0::2] & 0xF)


def unpack_e2m1_codes(packed: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_e2m1` (src/quantization/wush_gptq.py:85-86)."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """Packed bytes -> float64 values (src/quantization/wush_gptq.py:74-88)."""
    return E2M1_VALUES[unpack_e2m1_codes(packed)]


# ----------------------------------------------------------------------------------
# a2: rtn_xxfp4 / dequant_xxfp4
# ----------------------------------------------------------------------------------

def _scale_cast(scale64: np.ndarray, kind: str) -> tuple[np.ndarray, np.ndarray]:
    if kind == "e8m0":
        b = cast_e8m0(scale64)
        return b, e8m0_to_f64(b)
    if kind == "e4m3":
        b = cast_e4m3(scale64)
        return b, e4m3_to_f64(b)
    raise NotImplementedError(kind)


def rtn_xxfp4(x: np.ndarray, fmt: str, existing_scale: np.ndarray | None = None) -> dict:
    """Group-scaled FP4 round-to-nearest, src/quantization/wush_gptq.py:91-138 with the
    constants of :388-407.

    x: (..., C) any float dtype (values are taken exactly into float64).
    Returns dict with
      'fake_quant'  (..., C) float64 -- dequantized values (the reference casts this to
                    x.dtype; callers do that where they need it),
      'codes'       (..., C) uint8 unpacked E2M1 codes,
      'e2m1'        (..., C/2) uint8 packed,
      'scale_quant' (..., C/G) uint8 raw scale byte (E8M0 or E4M3),
      'global_scale' float.
    """
    f = FORMATS[fmt]
    g, gs, ss = f["group"], f["global_scale"], f["scale_scale"]
    x64 = np.asarray(x, dtype=np.float64)
    xr = x64.reshape(x64.shape[:-1] + (x64.shape[-1] // g, g))
    if existing_scale is None:
        absmax = np.abs(xr).max(axis=-1, keepdims=True)              # :118
        sbyte, sdeq = _scale_cast(absmax * gs / ss, f["scale"])      # :119-120,124
    else:
        sbyte = np.asarray(existing_scale, dtype=np.uint8)[..., None]  # :122
        sdeq = e8m0_to_f64(sbyte) if f["scale"] == "e8m0" else e4m3_to_f64(sbyte)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = xr * gs / sdeq                                      # :127
        vals, codes = rtn_e2m1(scaled)                               # :128
        deq = vals * sdeq / gs                                       # :129
    flat = lambda a: a.reshape(a.shape[:-2] + (-1,))
    codes = flat(codes)
    return {
        "fake_quant": flat(deq),
        "codes": codes,
        "e2m1": pack_e2m1(codes),
        "scale_quant": sbyte[..., 0],
        "global_scale": gs,
    }


def dequant_xxfp4(e2m1: np.ndarray, scale_quant: np.ndarray, fmt: str) -> np.ndarray:
    """Packed codes + scale bytes -> float64 values,
    src/quantization/wush_gptq.py:141-162."""
    f = FORMATS[fmt]
    g, gs = f["group"], f["global_scale"]
    vals = unpack_e2m1(e2m1)
    sdeq = e8m0_to_f64(scale_quant) if f["scale"] == "e8m0" else e4m3_to_f64(scale_quant)
    vr = vals.reshape(vals.shape[:-1] + (vals.shape[-1] // g, g))
    out = vr * sdeq[..., None] / gs
    return out.reshape(vals.shape)


# ----------------------------------------------------------------------------------
# a3 / a4: transforms
# ----------------------------------------------------------------------------------

def normalized_hadamard(n: int) -> np.ndarray:
    """Sylvester Hadamard matrix times n**-0.5 (src/quantization/wush_gptq.py:20; the
    reference takes it from scipy.linalg.hadamard, which is the same construction)."""
    h = np.array([[1.0]])
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    assert h.shape[0] == n, "size must be a power of two"
    return h * n ** -0.5


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float64 -> float32 -> bfloat16 (round to nearest even each time) -> float64, the
    effect of ``tensor.to(torch.bfloat16)`` on a float64 tensor."""
    b = np.asarray(x, dtype=np.float64).astype(np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    rounded = np.where(nan, b | 0x400000, rounded)
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64)


def get_transform(basis: np.ndarray, y: np.ndarray, transform_type: str, round_bf16: bool = True) -> np.ndarray:
    """Per-block transform, src/quantization/wush_gptq.py:304-347.

    basis: (B, B) upper-triangular Cholesky block; y: (B, R).  'wush':
    T = Had . diag(s^1/2) . V^T . basis^-T with y = V diag(s) U^H, s scaled by R^-1/2 and
    damped by 1 % of its mean (:331-341).  The result is rounded to the model dtype
    (bf16 here) and returned in float64 (:345).  Flipping the sign of one singular
    vector flips one rank-1 term of T, so T depends on the SVD library's sign convention
    (T basis^T (T basis^T)^T = Had diag(s) Had^T does not).  The SVD is therefore taken
    from torch's CPU LAPACK binding, the one the reference calls, and the golden test
    checks both the matrix and that sign-free product.
    """
    b = basis.shape[-1]
    if transform_type == "identity":
        t = np.eye(b)
    elif transform_type == "hadamard":
        t = normalized_hadamard(b)
    elif transform_type in ("wush", "wus"):
        had = np.eye(b) if transform_type == "wus" else normalized_hadamard(b)
        import torch
        v, s, _ = (a.numpy() for a in torch.linalg.svd(torch.from_numpy(np.ascontiguousarray(y)), full_matrices=False))
        s = s * y.shape[-1] ** -0.5
        s = s + s.mean() * 1e-2
        rhs = (had * np.sqrt(s)[None, :]) @ v.T
        # X . basis^T = rhs  <=>  basis . X^T = rhs^T
        t = np.linalg.solve(basis, rhs.T).T
    else:
        raise NotImplementedError(transform_type)
    if round_bf16:
        t = round_to_bf16(t)
    assert np.isfinite(t).all()
    return t


def block_transform(x: np.ndarray, transform: np.ndarray) -> np.ndarray:
    """y[..., n, :] = x[..., n, :] @ transform[n].T in float64,
    src/quantization/wush_gptq.py:350-370 (the caller applies the final cast).

    x: (..., C); transform: (C/B, B, B) or (B, B) shared.  Returns float64 (..., C).
    """
    x64 = np.asarray(x, dtype=np.float64)
    t = np.asarray(transform, dtype=np.float64)
    b = t.shape[-1]
    xr = x64.reshape(x64.shape[:-1] + (x64.shape[-1] // b, b))
    if t.ndim == 2:
        y = np.einsum("...ng,hg->...nh", xr, t)
    else:
        y = np.einsum("...ng,nhg->...nh", xr, t)
    return y.reshape(x64.shape)


def transform_to_matrix(transform: np.ndarray) -> np.ndarray:
    """(C/G, G, G) per-group transforms -> the (G, C) matrix the fused quantize op
    takes: column block n holds T_n^T, so y_n = x_n @ M[:, nG:(n+1)G]
    (src/quantization/wush_gptq.py:589-590)."""
    n, g, _ = transform.shape
    return np.ascontiguousarray(transform.reshape(n * g, g).T)


def matrix_to_transform(mat: np.ndarray) -> np.ndarray:
    """Inverse of :func:`transform_to_matrix`."""
    g, c = mat.shape
    return np.ascontiguousarray(mat.T.reshape(c // g, g, g))


def fused_transform_quant(x: np.ndarray, mat: np.ndarray, fmt: str, round_bf16: bool = False) -> dict:
    """What the fused kernel must produce: block transform in float64, rounded once to
    float32 (or to bfloat16 when round_bf16, which is what the reference's runtime
    module does between its einsum and its quantizer, src/utils/wush_utils.py:140-149),
    then :func:`rtn_xxfp4`.

    mat is (G, C) per-group (see :func:`transform_to_matrix`) or (G, G) shared.
    Adds 'transformed' (float64 view of the rounded transform output) to the dict.
    """
    g = FORMATS[fmt]["group"]
    t = matrix_to_transform(np.asarray(mat, dtype=np.float64)) if mat.shape[1] != g else np.asarray(mat, dtype=np.float64).T
    y = block_transform(x, t)
    y = round_to_bf16(y) if round_bf16 else y.astype(np.float32).astype(np.float64)
    out = rtn_xxfp4(y, fmt)
    out["transformed"] = y
    return out


def wide_transform(x: np.ndarray, mat: np.ndarray) -> np.ndarray:
    """y_block = x_block @ mat for consecutive blocks of n = mat.shape[0] channels, n any multiple of the scale group
    (the shared Hadamard sizes 64 / 128 of inference_lib/src/fp_quant/utils/config.py:35-50).  This is the first step of
    the reference's Triton kernels (inference_lib/src/fp_quant/module/triton/mxfp4.py:56-59: reshape to
    (-1, hadamard_dim), tl.dot with the matrix); the result is regrouped by 32 / 16 for the scales afterwards.
    float64 in, float64 out."""
    x = np.asarray(x, dtype=np.float64)
    n = mat.shape[0]
    return (x.reshape(-1, n) @ np.asarray(mat, dtype=np.float64)).reshape(x.shape)


#: Gaussian-optimal scale of the "quest" method (inference_lib/src/fp_quant/module/pseudoquant_linear_fns.py:21)
QUEST_GAUSSIAN_SCALE = 2.92247856 / 6.0


def quest_mxfp4(y: np.ndarray, gaussian_scale: float = QUEST_GAUSSIAN_SCALE) -> dict:
    """MXFP4 with the "quest" scale: the group's standard deviation, not its absolute maximum, sets the shared
    exponent, and values beyond +-6 clip.  Follows the quest branch of the reference's Triton kernel
    (inference_lib/src/fp_quant/module/triton/mxfp4.py:64-74 for the scale, :77-118 for the value ladder,
    :119-124 for the clip mask) in its float32 arithmetic, one operation at a time.

    y: transformed values [..., C], C a multiple of 32.  Returns 'fake_quant' (dequantized float32), 'scaled'
    (y / 2^e, float32), 'scale_quant' (E8M0 byte: biased exponent e + 127), 'e2m1' (codes, ties toward zero
    as the ladder's strict comparisons give; 0 quantizes to -0) and 'clip_mask' (|scaled| < 6).
    """
    shape = np.shape(y)
    g = np.asarray(y, dtype=np.float32).reshape(-1, 32)
    f32 = np.float32
    mean_sq = (g * g).sum(axis=-1, keepdims=True, dtype=f32) / f32(32)
    mean = g.sum(axis=-1, keepdims=True, dtype=f32) / f32(32)
    with np.errstate(invalid="ignore", divide="ignore"):
        std = np.sqrt(mean_sq - mean * mean)
        scales = f32(gaussian_scale) * std + f32(1e-8)
        exps = np.floor(np.log2(scales))
        shared = np.exp2(exps).astype(f32)
        scaled = (g / shared).astype(f32)
    a = np.abs(scaled)
    idx = ((a > 0.25).astype(np.uint8) + (a > 0.75) + (a > 1.25) + (a > 1.75) + (a > 2.5) + (a > 3.5) + (a > 5)).astype(np.uint8)
    neg = ~(scaled > 0)
    codes = (idx | (neg.astype(np.uint8) << 3)).astype(np.uint8)
    fake = (E2M1_VALUES[codes].astype(f32) * shared).astype(f32)
    with np.errstate(invalid="ignore"):
        byte = np.where(np.isfinite(exps), np.clip(exps + 127, 0, 254), 255).astype(np.uint8)
    return dict(fake_quant=fake.reshape(shape), scaled=scaled.reshape(shape), e2m1=pack_e2m1(codes.reshape(shape)),
                scale_quant=byte.reshape(shape[:-1] + (shape[-1] // 32,)), clip_mask=(a < 6).reshape(shape))


# ----------------------------------------------------------------------------------
# scale-factor layout consumed by the block-scaled MMA
# ----------------------------------------------------------------------------------

def pad_scales(scales: np.ndarray) -> np.ndarray:
    """Row-major scales padded to (ceil(rows/128)*128, ceil(cols/4)*4), the shape the
    reference's fused-quantize ops return
    (inference_lib/src/fp_quant/module/qutlass_ops.py:57-66)."""
    r, c = scales.shape
    pr, pc = -(-r // 128) * 128, -(-c // 4) * 4
    out = np.zeros((pr, pc), dtype=scales.dtype)
    out[:r, :c] = scales
    return out


def to_blocked(scales: np.ndarray) -> np.ndarray:
    """Row-major (rows, cols) scale bytes -> the 128x4-tile interleaved layout of
    block-scaled tensor-core GEMMs (what ``qutlass.utils.to_blocked`` produces at
    inference_lib/src/fp_quant/module/qutlass_ops.py:160-161).  Tiles are stored
    row-block major; inside a 512-byte tile, element (r, c) lives at
    (r % 32) * 16 + (r // 32) * 4 + c.  Returns a flat uint8 array."""
    p = pad_scales(np.asarray(scales))
    pr, pc = p.shape
    t = p.reshape(pr // 128, 4, 32, pc // 4, 4)      # rb, r//32, r%32, cb, c
    t = t.transpose(0, 3, 2, 1, 4)                    # rb, cb, r%32, r//32, c
    return np.ascontiguousarray(t).reshape(-1)


# ----------------------------------------------------------------------------------
# a8: GEMM oracle
# ----------------------------------------------------------------------------------

def fp4_gemm(a_e2m1, a_scales, b_e2m1, b_scales, alpha: float, fmt: str) -> np.ndarray:
    """Y = alpha * deq(A) . deq(B)^T in float64 with the E2M1 values multiplied by their
    raw group scales (no global-scale division: alpha carries 1/(w_gs*a_gs),
    inference_lib/src/fp_quant/module/linear_fns.py:514-521).  a: (M, K/2), b: (N, K/2)
    packed; scales (M, K/G), (N, K/G) raw bytes."""
    g = FORMATS[fmt]["group"]
    dq = e8m0_to_f64 if FORMATS[fmt]["scale"] == "e8m0" else e4m3_to_f64

    def deq(q, s):
        v = unpack_e2m1(q)
        return (v.reshape(v.shape[0], -1, g) * dq(s)[..., None]).reshape(v.shape)

    return alpha * (deq(a_e2m1, a_scales) @ deq(b_e2m1, b_scales).T)


# ----------------------------------------------------------------------------------
# a10 / a11: Hessian
# ----------------------------------------------------------------------------------

def hessian_xtx(x: np.ndarray) -> np.ndarray:
    """float64 X^T X -- what src/quantization/accumulate_hessian.py:26-109 adds to H
    (the kernel there uses TF32 products; float64 is the accuracy reference)."""
    x64 = np.asarray(x, dtype=np.float64)
    return x64.T @ x64


def wush_update_sequence(batches: list[np.ndarray]) -> np.ndarray:
    """The running mean kept by WUSH.update (src/quantization/wush_gptq.py:456-469):
    H <- H * n/(n+b) + (X (n+b)^-1/2)^T (X (n+b)^-1/2), n <- n + b; equals
    (1/N) sum x^T x.  float64 throughout."""
    h, n = None, 0
    for x in batches:
        x64 = np.asarray(x, dtype=np.float64).reshape(-1, x.shape[-1])
        b = x64.shape[0]
        if h is None:
            h = np.zeros((x64.shape[1], x64.shape[1]))
        h *= n / (n + b)
        xs = x64 * (n + b) ** -0.5
        h += xs.T @ xs
        n += b
    return h


# ----------------------------------------------------------------------------------
# a12: GPTQ / Babai column sweep
# ----------------------------------------------------------------------------------

def damped_cholesky_upper(hessian: np.ndarray, damp_ratio: float = 1e-2, max_try: int = 100) -> np.ndarray:
    """Upper Cholesky factor U (U^T U = H + damping) with the reference's retry loop,
    src/quantization/wush_gptq.py:196-208: add damp_ratio * mean(diag) to the diagonal,
    factor, and add the same amount again (of the already damped matrix) while it fails."""
    h = np.array(hessian, dtype=np.float64, copy=True)
    idx = np.arange(h.shape[-1])
    h[idx, idx] += damp_ratio * h.diagonal().mean()
    for _ in range(max_try):
        try:
            return np.linalg.cholesky(h).T.copy()
        except np.linalg.LinAlgError:
            h[idx, idx] += damp_ratio * h.diagonal().mean()
    raise AssertionError("Hessian decomposition failed")


def _solve_upper(u: np.ndarray, b: np.ndarray) -> np.ndarray:
    """x with u @ x = b for an upper-triangular u (back substitution, float64)."""
    n = u.shape[0]
    x = np.zeros_like(b, dtype=np.float64)
    for i in range(n - 1, -1, -1):
        x[i] = (b[i] - u[i, i + 1:] @ x[i + 1:]) / u[i, i]
    return x


def babai_inner(basis: np.ndarray, y: np.ndarray, fmt: str, transform: np.ndarray, force_rtn: bool) -> dict:
    """One block of the sweep, src/quantization/wush_gptq.py:228-277, for a given block transform
    (the reference computes it at :246 with get_transform; here the caller passes it so that a test can
    use the very matrix another implementation chose -- 'wush' transforms are unique only up to the
    sign convention of the SVD).

    basis: (B, B) upper triangular; y: (B, R); transform: (B, B) float64 (already rounded to the model
    dtype).  QR of basis @ transform^T (:251), rotate y (:252), solve (:254-260), quantize the rows
    of the solution's transpose (:262); then either keep the round-to-nearest values (:264-265) or run
    Babai's nearest-plane steps from the last coordinate to the first with the scales frozen
    (:266-272).  Returns codes (R, B) uint8, scale bytes (R,), the dequantized transformed values
    'fake_quant' (R, B) and 'coefficient' = transform^T @ x_transformed (B, R) (:274).
    """
    q, r = np.linalg.qr(basis @ transform.T)                    # :251
    y_new = q.T @ y                                             # :252
    x_t = _solve_upper(r, y_new)                                # :254-260
    res = rtn_xxfp4(x_t.T, fmt)                                 # :262
    if force_rtn:
        x_t = res["fake_quant"].T                               # :265
    else:
        for i in range(r.shape[0] - 1, -1, -1):                 # :267
            x_t[i] = y_new[i] / r[i, i]                         # :269
            res = rtn_xxfp4(x_t.T, fmt, existing_scale=res["scale_quant"])   # :270
            x_t = res["fake_quant"].T.copy()                    # :271
            y_new[:i] -= r[:i, i:i + 1] * x_t[i:i + 1]          # :272
    return {
        "codes": res["codes"], "e2m1": res["e2m1"], "scale_quant": res["scale_quant"][..., 0],
        "fake_quant": res["fake_quant"], "coefficient": transform.T @ x_t, "transform": transform,
    }


def gptq_babai_outer(weight: np.ndarray, hessian: np.ndarray | None, fmt: str, transform_type: str,
                     force_rtn: bool, transform_fn=None) -> dict:
    """Column sweep over blocks of one scale group, last block first,
    src/quantization/wush_gptq.py:165-225 as quantize_layers drives it (:373-441: block size = group
    size, force_rtn for both the outer and the inner loop, the transform rounded to the model dtype).

    weight: (R, C); hessian: (C, C) or None (identity).  `transform_fn(block_index, basis, y)` overrides
    get_transform.  Returns packed codes (R, C/2), scale bytes (R, C/G), 'fake_quant' (R, C) float64
    (the dequantized transformed weights, :293-296), 'transform_basis' (C/G, G, G) and the sweep's
    coefficient matrix 'x' (C, R).
    """
    g = FORMATS[fmt]["group"]
    w = np.asarray(weight, dtype=np.float64)
    n = w.shape[1]
    x = w.T.copy()                                              # :188
    h = np.eye(n) if hessian is None else hessian               # :191-194
    u = damped_cholesky_upper(h)                                # :195-208
    y = u @ x                                                   # :210
    blocks = {}
    for i1 in range((n - 1) // g * g, -1, -g):                  # :214
        i2 = i1 + g
        basis, yb = u[i1:i2, i1:i2], y[i1:i2].copy()
        t = transform_fn(i1 // g, basis, yb) if transform_fn is not None else get_transform(basis, yb, transform_type)
        res = babai_inner(basis, yb, fmt, t, force_rtn)         # :216-219
        blocks[i1 // g] = res
        if not force_rtn:
            x[i1:i2] = res["coefficient"]                       # :221
        y[:i1] -= u[:i1, i1:i2] @ x[i1:i2]                      # :222
    order = sorted(blocks)
    return {
        "e2m1": np.concatenate([blocks[b]["e2m1"] for b in order], axis=-1),
        "codes": np.concatenate([blocks[b]["codes"] for b in order], axis=-1),
        "scale_quant": np.stack([blocks[b]["scale_quant"] for b in order], axis=-1),
        "fake_quant": np.concatenate([blocks[b]["fake_quant"] for b in order], axis=-1),
        "transform_basis": np.stack([blocks[b]["transform"] for b in order]),
        "x": x,
    }
