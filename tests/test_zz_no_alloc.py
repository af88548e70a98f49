"""The allocation-free split-K GEMM entry point (wush_gemm_mxf4_bf16_tn_noalloc), called through the C ABI.

It exists for hosts that may not allocate device memory where the GEMM runs (fixed memory plans, foreign
stream-ordered pools, graph replay): its split-K scratch is a fixed array inside the library.  The test checks
it against the regular entry point (same forced split count, caller-supplied workspace) on two calls in a row with
different operands -- the second call reuses the array with the first call's leftovers in it -- and checks the size
limit.  Tolerance: the GEMM tests' 1e-2 relative Frobenius bound (the two paths run the same kernels, so the
outputs are in fact identical).  Collected last on purpose: a failure here cannot hide other tests under `-x`.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _operands(m, n, k, seed, dev):
    rng = np.random.default_rng(seed)
    a = wo.rtn_xxfp4(rng.standard_normal((m, k)), "mxfp4")
    b = wo.rtn_xxfp4(rng.standard_normal((n, k)) * 0.02, "mxfp4")
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(dev)
    from wush_b200 import qutlass_ops as ops
    return (t(a["e2m1"]), t(b["e2m1"]), ops.to_blocked(t(a["scale_quant"])), ops.to_blocked(t(b["scale_quant"])),
            wo.fp4_gemm(a["e2m1"], a["scale_quant"], b["e2m1"], b["scale_quant"], 1.0 / 9.0, "mxfp4"))


def test_noalloc_entry_matches_regular_entry_twice():
    from wush_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    alpha = torch.tensor([1.0 / 9.0], device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (m, n, k, splits) in enumerate([(16, 1024, 2048, 4), (48, 512, 1024, 2)]):
        aq, bq, sa, sb, want = _operands(m, n, k, 100 + call, dev)
        y_new = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        y_old = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        rc = lib.wush_gemm_mxf4_bf16_tn_noalloc(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(),
                                                alpha.data_ptr(), y_new.data_ptr(), m, n, k, splits, None, stream)
        assert rc == 0, rc
        work = torch.empty(splits * m * n, dtype=torch.float32, device=dev)
        rc = lib.wush_gemm_mxf4_bf16_tn(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(), alpha.data_ptr(),
                                        y_old.data_ptr(), m, n, k, work.data_ptr(), work.numel() * 4, splits, None, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        new, old = y_new.double().cpu().numpy(), y_old.double().cpu().numpy()
        assert np.isfinite(new).all()
        assert np.linalg.norm(new - old) <= TOL * np.linalg.norm(old)
        assert np.linalg.norm(new - want) <= TOL * np.linalg.norm(want)
    # automatic split choice also works and agrees
    aq, bq, sa, sb, want = _operands(16, 1024, 2048, 7, dev)
    y = torch.empty(16, 1024, dtype=torch.bfloat16, device=dev)
    assert lib.wush_gemm_mxf4_bf16_tn_noalloc(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(), alpha.data_ptr(),
                                              y.data_ptr(), 16, 1024, 2048, 0, None, stream) == 0
    torch.cuda.synchronize()
    got = y.double().cpu().numpy()
    assert np.linalg.norm(got - want) <= TOL * np.linalg.norm(want)


def test_noalloc_entry_rejects_what_does_not_fit():
    from wush_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_uint8 * 64)()
    p = (ctypes.addressof(buf) + 15) // 16 * 16
    # 4096 x 4096 outputs x 2 splits = 128 MiB of partial tiles: beyond the 16 MiB array
    assert lib.wush_gemm_mxf4_bf16_tn_noalloc(p, p, p, p, p, p, 4096, 4096, 4096, 2, None, None) == -8
    # K = 256 is a single k-block and cannot be split
    assert lib.wush_gemm_mxf4_bf16_tn_noalloc(p, p, p, p, p, p, 16, 256, 256, 0, None, None) == -4
