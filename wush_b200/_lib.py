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
QUANT_WIDE_MATRIX = 2
HESSIAN_LOWER_ONLY = 1
HESSIAN_INPUT_F32 = 2
HESSIAN_OVERWRITE = 4
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
        "wush_fused_quantize_mx_quest": [vp, vp, i64, vp, vp, i64, i32, vp, i64, i64, i32, vp],
        "wush_fused_quantize_nv": [vp, vp, i64, vp, vp, vp, i64, i32, i64, i64, i32, vp],
        "wush_fused_quantize_debug": [i32, vp, vp, i64, vp, vp, vp, i64, i32, vp, i64, i64, i32, vp],
        "wush_fused_quantize_strided": [i32, vp, i64, vp, i64, vp, vp, i64, vp, i64, i32, i64, vp, vp, i64, i64, i32, vp],
        "wush_peer_broadcast": [vp, vp, vp, i32, i64, vp],
        "wush_row_sumsq": [vp, i64, vp, i64, i64, vp],
        "wush_swiglu": [vp, vp, i64, vp, i64, i64, i64, vp],
        "wush_sf_to_blocked": [vp, vp, i64, i64, vp],
        "wush_hessian_accumulate": [vp, vp, i64, i64, i32, vp, vp],
        "wush_hessian_accumulate_rows": [vp, vp, i64, i64, i64, i64, i32, vp, vp],
        "wush_hessian_finalize": [vp, i64, ctypes.c_float, vp],
        "wush_hessian_finalize_count": [vp, i64, vp, vp],
        "wush_hessian_peer_reduce": [vp, vp, vp, i32, i32, i64, i64, i64, vp, ctypes.c_uint32, vp, vp],
        "wush_hessian_accumulate_tiles": [vp, vp, i64, i64, i64, i64, i32, vp, vp],
        "wush_hessian_mirror_tiles": [vp, i64, i64, i64, i32, i32, vp, ctypes.c_uint32, vp, vp],
        "wush_hessian_tiles_per_wave": [],
        "wush_hessian_tile_coords": [i64, i64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
        "wush_gemm_cluster_capacity": [i32, i32],
        "wush_status_check": [vp, vp],
        "wush_selftest_bounded_wait": [vp, i32, vp],
        "wush_gemm_fp4_bf16_tn_fused": [i32, vp, i32, i64, i64, vp, vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, i64, vp,
                                        ctypes.c_size_t, i32, vp, vp],
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
    lib.wush_gemm_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.wush_gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.wush_hessian_tile_count.argtypes = [i64]
    lib.wush_hessian_tile_count.restype = ctypes.c_int64
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc in (-6, -7):
        raise WushB200Error(f"{what}: {ERRORS[rc]}")
    if rc < 0:
        raise WushB200Error(f"{what}: rejected argument ({ERRORS.get(rc, rc)})")
    raise WushB200Error(f"{what}: CUDA error {rc}")


# --------------------------------------------------------------------------------------------
# per-device state shared by the ops: the status word of the bounded waits, split-K workspaces
# --------------------------------------------------------------------------------------------
_status_words: dict = {}
_workspaces: dict = {}


def status_word(device):
    """The int32 device word every kernel launch of this process reports a run-out wait into (one per
    device, allocated on first use and never freed)."""
    import torch
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return w


def check_status(device, what: str = "kernel") -> None:
    """Synchronize the current stream of `device` and raise WushB200Error if any kernel launched so far reported
    a device-side timeout (its output is invalid).  Called at the points where the host waits anyway
    (HostQuantizer.synchronize, DistributedHessian.num_samples, the column sweep) and after every op when the
    environment variable WUSH_B200_CHECK_STATUS=1 is set."""
    import torch
    w = status_word(device)
    with torch.cuda.device(w.device):
        rc = load().wush_status_check(w.data_ptr(), torch.cuda.current_stream().cuda_stream)
    check(rc, what)


CHECK_EVERY_OP = os.environ.get("WUSH_B200_CHECK_STATUS", "0") == "1"


def gemm_workspace(device, nbytes: int):
    """Split-K scratch for the current stream of `device` (contents irrelevant): grown on demand and reused by
    later calls on that stream.  While the stream is being captured into a CUDA graph the scratch comes from the
    graph's own memory pool instead, so that it lives exactly as long as the graph."""
    import torch
    device = torch.device(device)
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        w = _workspaces[key] = torch.empty(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
    return w
