"""ctypes binding of ``libwush_b200.so`` (the C ABI declared in ``include/wush_b200.h``).

There is no CPU or PyTorch fallback: if the library cannot be loaded, or a call returns a
non-zero status, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("WUSH_B200_LIB") or os.path.join(HERE, "libwush_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "wush_b200.h")

ERRORS = {
    -1: "null pointer", -2: "bad shape", -3: "bad alignment", -4: "bad flag or layout",
    -5: "workspace too small", -6: "device is not sm_100", -7: "device-side bounded wait timed out",
    -8: "problem exceeds a fixed capacity of the entry point",
}

SF_ROW_MAJOR, SF_BLOCKED = 0, 1
QUANT_ROUND_BF16 = 1
HESSIAN_LOWER_ONLY = 1
HESSIAN_INPUT_F32 = 2
FORMAT_MXFP4, FORMAT_NVFP4 = 0, 1
SWEEP_RTN_ONLY, SWEEP_FAKE_F32 = 1, 2
TRANSFORMS = {"identity": 0, "hadamard": 1, "wush": 2, "wus": 3, "given": 4}

_lib = None


class WushB200Error(RuntimeError):
    pass


def declared_symbols(header: str = HEADER_PATH) -> list[str]:
    """Names of every function the public header declares."""
    text = open(header).read()
    return sorted(set(re.findall(r"WUSH_API\s+[\w\s\*]+?\b(wush_\w+)\s*\(", text)))


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        # build on first use when a compiler is around; otherwise fail loudly
        from . import build as _build
        _build.build()
    if not os.path.exists(LIB_PATH):
        raise WushB200Error(f"{LIB_PATH} is missing and could not be built; there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    sigs = {
        "wush_b200_arch": [],
        "wush_fused_quantize_mx": [vp, vp, i64, vp, vp, i64, i32, i64, i64, i32, vp],
        "wush_fused_quantize_nv": [vp, vp, i64, vp, vp, vp, i64, i32, i64, i64, i32, vp],
        "wush_fused_quantize_debug": [i32, vp, vp, i64, vp, vp, vp, i64, i32, vp, i64, i64, i32, vp],
        "wush_sf_to_blocked": [vp, vp, i64, i64, vp],
        "wush_hessian_accumulate": [vp, vp, i64, i64, i32, vp, vp],
        "wush_hessian_accumulate_rows": [vp, vp, i64, i64, i64, i64, i32, vp, vp],
        "wush_hessian_finalize": [vp, i64, ctypes.c_float, vp],
        "wush_hessian_finalize_count": [vp, i64, vp, vp],
        "wush_hessian_peer_reduce": [vp, vp, i32, i32, i64, vp],
        "wush_gemm_mxf4_bf16_tn": [vp, vp, vp, vp, vp, vp, i64, i64, i64, vp, ctypes.c_size_t, i32, vp, vp],
        "wush_gemm_nvf4_bf16_tn": [vp, vp, vp, vp, vp, vp, i64, i64, i64, vp, ctypes.c_size_t, i32, vp, vp],
        "wush_gemm_fp4_bf16_tn_sharded": [i32, vp, vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, i64, i64, vp, vp],
        "wush_gptq_block_step": [vp, vp, vp, vp, i32, i32, i64, i64, i32, i32, vp, vp, vp, vp, vp],
        "wush_gptq_block_prepare": [vp, vp, i64, i64, i32, i32, i32, i32, i64, vp, vp, vp, vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    lib.wush_gemm_mxf4_bf16_tn_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, vp, vp]
    lib.wush_gemm_mxf4_bf16_tn_noalloc.restype = ctypes.c_int
    lib.wush_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    lib.wush_gemm_workspace_bytes.restype = ctypes.c_size_t
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise WushB200Error(f"{what}: rejected argument ({ERRORS.get(rc, rc)})")
    raise WushB200Error(f"{what}: CUDA error {rc}")
