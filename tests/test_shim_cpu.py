"""wush_b200.shim.install() against a checkout of the reference (skipped without one): after it, the reference's own
modules are bound to this library at all three seams, whichever is imported first.  No kernel is launched."""
import os
import subprocess
import sys

import pytest

from tests.util_reference import REF, needs_reference

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHECK = """
import inference_lib.src.fp_quant.module.qutlass_ops as q
import inference_lib.src.fp_quant.module.linear_fns as lf
import src.quantization.wush_gptq as wg
import src.quantization.accumulate_hessian as ah
import src.utils.wush_utils as wu
from wush_b200 import hessian, pseudo_quant, shim as s
assert q.HAS_QUTLASS is True
assert q.fusedQuantizeWushMx is s.fusedQuantizeWushMx and q.matmul_mxf4_bf16_tn is s.matmul_mxf4_bf16_tn
assert q.to_blocked_qutlass is s.to_blocked
assert lf.fused_quantize_mx_wush_op is q.fused_quantize_mx_wush_op        # the reference's own fp_quant:: op
assert wg.accumulate_hessian is hessian.accumulate_hessian and ah.accumulate_hessian is hessian.accumulate_hessian
assert wu.mxfp4_forward_kernel_wrapper is pseudo_quant.mxfp4_forward_kernel_wrapper
assert wu.nvfp4_forward_kernel_wrapper is pseudo_quant.nvfp4_forward_kernel_wrapper
import torch
try:
    q.fused_quantize_mx_wush_op(torch.zeros(4, 64, dtype=torch.bfloat16), torch.zeros(32, 64, dtype=torch.bfloat16), "abs_max", False)
    raise SystemExit("a CPU tensor must be refused: there is no fallback path")
except Exception as exc:
    assert "CUDA" in str(exc), exc
print("shim ok")
"""


@needs_reference
@pytest.mark.parametrize("order", ["install_first", "import_first"])
def test_install_binds_the_reference_to_this_library(order):
    pre = "from wush_b200 import shim; shim.install()\n"
    imp = "import inference_lib.src.fp_quant.module.qutlass_ops, src.quantization.wush_gptq, src.utils.wush_utils\n"
    body = (pre + CHECK) if order == "install_first" else (imp + pre + CHECK)
    code = f"import sys, os\nsys.path.insert(0, {ROOT!r}); sys.path.insert(0, {REF!r}); os.chdir({REF!r})\n" + body
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0 and "shim ok" in p.stdout, p.stdout + p.stderr
