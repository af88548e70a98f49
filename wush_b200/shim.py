"""Make the reference run on these kernels without editing it.

The reference reaches its GPU kernels through three seams, all bound by name at import time:
  * ``from qutlass import fusedQuantizeMx, fusedQuantizeNv, fusedQuantizeWushMx, matmul_mxf4_bf16_tn, ...`` and
    ``from qutlass.utils import to_blocked`` in inference_lib/src/fp_quant/module/qutlass_ops.py:5-29 (QuTLASS, a
    separate CUDA package); its own ``fp_quant::*`` custom ops (:37-206) and everything above them
    (linear_fns.py:9-26, linear.py) call these functions;
  * ``from .accumulate_hessian import accumulate_hessian`` in src/quantization/wush_gptq.py:22 (Triton kernel);
  * ``mxfp4_forward_kernel_wrapper`` / ``nvfp4_forward_kernel_wrapper`` imported by src/utils/wush_utils.py:3-4
    (Triton kernels) for the pseudo-quantized layers the calibration loop evaluates.

``install()`` puts a module named ``qutlass`` (with ``qutlass.utils``) in ``sys.modules`` whose functions have
QuTLASS's names and call conventions and run the kernels of this library, and rebinds the other two seams in every
reference module that is already imported -- and, through an import hook, in those imported later.  Call it before
importing the reference (``model_quant.py`` then runs as it is), or after: both orders work.  Training-only entry
points of QuTLASS (MXFP8 GEMMs, backward quantizers) raise NotImplementedError.
"""
from __future__ import annotations

import importlib.abc
import importlib.machinery
import sys
import types

import torch

from . import qutlass_ops as ops

_INSTALLED = False


# ---- QuTLASS surface ------------------------------------------------------------------------------------------

def fusedQuantizeMx(x_flat, hadamard_matrix, method: str = "abs_max", return_mask: bool = False):
    q, sf, mask = ops.fused_quantize_mx_op(x_flat, hadamard_matrix, method, return_mask)
    return (q, sf, mask) if return_mask else (q, sf)


def fusedQuantizeWushMx(x_flat, wush_matrix, method: str = "abs_max", return_mask: bool = False):
    q, sf, mask = ops.fused_quantize_mx_wush_op(x_flat, wush_matrix, method, return_mask)
    return (q, sf, mask) if return_mask else (q, sf)


def fusedQuantizeNv(x_flat, hadamard_matrix, global_scale):
    return ops.fused_quantize_nv_op(x_flat, hadamard_matrix, global_scale)


def to_blocked(x, use_triton_kernel: bool = True):
    return ops.to_blocked(x)


def matmul_mxf4_bf16_tn(x, w, xs_blocked, ws_blocked, alpha):
    return ops.matmul_fp4_blocked(x, w, xs_blocked.view(torch.uint8).reshape(-1), ws_blocked.view(torch.uint8).reshape(-1),
                                  alpha, "mx")


def matmul_ada_mxf4_bf16_tn(x, w, xs, ws, alpha):
    """QuTLASS's small-M variant takes ROW-MAJOR scales (qutlass_ops.py:171-184); here every M runs one kernel
    family, so the scales are re-laid and the ordinary GEMM is called."""
    return matmul_mxf4_bf16_tn(x, w, ops.to_blocked(xs.view(torch.uint8)), ops.to_blocked(ws.view(torch.uint8)), alpha)


def matmul_nvf4_bf16_tn(x, w, xs_blocked, ws_blocked, alpha):
    return ops.matmul_fp4_blocked(x, w, xs_blocked.view(torch.uint8).reshape(-1), ws_blocked.view(torch.uint8).reshape(-1),
                                  alpha, "nv")


def _training_only(name):
    def fn(*_a, **_k):
        raise NotImplementedError(f"qutlass.{name}: training / MXFP8 entry points are not part of the inference path")
    fn.__name__ = name
    return fn


def _qutlass_modules():
    pkg = types.ModuleType("qutlass")
    pkg.__doc__ = "QuTLASS-compatible surface backed by wush_b200 (installed by wush_b200.shim.install)"
    pkg.__path__ = []                      # a package: `qutlass.utils` can be imported
    for fn in (fusedQuantizeMx, fusedQuantizeNv, fusedQuantizeWushMx, matmul_mxf4_bf16_tn, matmul_ada_mxf4_bf16_tn,
               matmul_nvf4_bf16_tn):
        setattr(pkg, fn.__name__, fn)
    for name in ("matmul_mxf8_bf16_tn", "matmul_mxf8_bf16_nn", "backward_t_bf16", "backward_qt_bf16",
                 "backward_bf16_square_double_mxfp8", "mxfp4_transpose_mxfp8"):
        setattr(pkg, name, _training_only(name))
    utils = types.ModuleType("qutlass.utils")
    utils.to_blocked = to_blocked
    pkg.utils = utils
    return pkg, utils


# ---- the other two seams ----------------------------------------------------------------------------------------

def _rebind(module) -> None:
    """Replace, inside one imported reference module, the names that are bound to the Triton paths."""
    from . import hessian, pseudo_quant
    name = module.__name__
    if name.endswith("quantization.accumulate_hessian") or name.endswith("quantization.wush_gptq"):
        if hasattr(module, "accumulate_hessian"):
            module.accumulate_hessian = hessian.accumulate_hessian
    if name.endswith("triton.mxfp4") or name.endswith("utils.wush_utils") or name.endswith("module.pseudoquant_linear_fns"):
        if hasattr(module, "mxfp4_forward_kernel_wrapper"):
            module.mxfp4_forward_kernel_wrapper = pseudo_quant.mxfp4_forward_kernel_wrapper
    if name.endswith("triton.nvfp4") or name.endswith("utils.wush_utils") or name.endswith("module.pseudoquant_linear_fns"):
        if hasattr(module, "nvfp4_forward_kernel_wrapper"):
            module.nvfp4_forward_kernel_wrapper = pseudo_quant.nvfp4_forward_kernel_wrapper


_SUFFIXES = ("quantization.accumulate_hessian", "quantization.wush_gptq", "triton.mxfp4", "triton.nvfp4",
             "utils.wush_utils", "module.pseudoquant_linear_fns")


class _RebindLoader(importlib.abc.Loader):
    def __init__(self, inner):
        self.inner = inner

    def create_module(self, spec):
        return self.inner.create_module(spec)

    def exec_module(self, module):
        self.inner.exec_module(module)
        _rebind(module)


class _RebindFinder(importlib.abc.MetaPathFinder):
    """Wraps the loader of the reference modules named above so that they are rebound right after they execute."""

    def find_spec(self, fullname, path, target=None):
        if not fullname.endswith(_SUFFIXES):
            return None
        for finder in sys.meta_path:
            if finder is self or not hasattr(finder, "find_spec"):
                continue
            spec = finder.find_spec(fullname, path, target)
            if spec is not None and spec.loader is not None and hasattr(spec.loader, "exec_module"):
                spec.loader = _RebindLoader(spec.loader)
                return spec
        return None


def install() -> None:
    """Idempotent.  See the module docstring."""
    global _INSTALLED
    pkg, utils = _qutlass_modules()
    if "qutlass" not in sys.modules or getattr(sys.modules["qutlass"], "__doc__", "") == pkg.__doc__:
        sys.modules["qutlass"], sys.modules["qutlass.utils"] = pkg, utils
    for name, module in list(sys.modules.items()):
        if module is None:
            continue
        if name.endswith("fp_quant.module.qutlass_ops"):
            # imported before install(): its `from qutlass import ...` failed; give it the functions now
            for attr in dir(pkg):
                if not attr.startswith("_") and attr != "utils":
                    setattr(module, attr, getattr(pkg, attr))
            module.to_blocked_qutlass = to_blocked
            module.HAS_QUTLASS = True
        if name.endswith(_SUFFIXES):
            _rebind(module)
    if not _INSTALLED:
        sys.meta_path.insert(0, _RebindFinder())
        _INSTALLED = True


def uninstall() -> None:
    """Remove the import hook and the stand-in ``qutlass`` modules (already rebound modules stay rebound)."""
    global _INSTALLED
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, _RebindFinder)]
    for name in ("qutlass", "qutlass.utils"):
        if getattr(sys.modules.get(name), "__doc__", None) == _qutlass_modules()[0].__doc__ or name == "qutlass.utils":
            sys.modules.pop(name, None)
    _INSTALLED = False
