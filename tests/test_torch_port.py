"""The timed CPU baseline (oracle/torch_port.py) computes what the NumPy oracle computes."""
import numpy as np
import torch

from oracle import synth, torch_port
from oracle import wush_oracle as wo


def test_torch_port_matches_numpy_oracle():
    for fmt, g in (("mxfp4", 32), ("nvfp4", 16)):
        x = synth.activations(64, 256, seed=4)
        mat = synth.wush_matrix(256, g)
        want = wo.fused_transform_quant(synth.bf16_to_f64(x), mat, fmt)
        got = torch_port.fused_transform_quant(x, torch.from_numpy(mat).to(torch.bfloat16), fmt)
        assert np.array_equal(got["e2m1"].numpy(), want["e2m1"])
        assert np.array_equal(got["scale_quant"].numpy(), want["scale_quant"])
        h = synth.hadamard_matrix(g)
        want = wo.fused_transform_quant(synth.bf16_to_f64(x), h, fmt)
        got = torch_port.fused_transform_quant(x, torch.from_numpy(h).to(torch.bfloat16), fmt)
        assert np.array_equal(got["e2m1"].numpy(), want["e2m1"])


def test_torch_port_hessian_and_gemm():
    xs = [synth.activations(96, 64, seed=s) for s in (1, 2, 3)]
    h, n = torch.zeros(64, 64), 0
    for x in xs:
        n = torch_port.hessian_update(h, n, x[None])
    ref = wo.wush_update_sequence([synth.bf16_to_f64(x) for x in xs])
    assert np.abs(h.double().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    a = wo.rtn_xxfp4(np.random.default_rng(0).standard_normal((8, 64)), "mxfp4")
    b = wo.rtn_xxfp4(np.random.default_rng(1).standard_normal((16, 64)), "mxfp4")
    want = wo.fp4_gemm(a["e2m1"], a["scale_quant"], b["e2m1"], b["scale_quant"], 1 / 9, "mxfp4")
    got = torch_port.fp4_gemm(torch.from_numpy(a["e2m1"]), torch.from_numpy(a["scale_quant"]),
                              torch.from_numpy(b["e2m1"]), torch.from_numpy(b["scale_quant"]), 1 / 9, "mxfp4")
    assert np.allclose(got.double().numpy(), want, rtol=1e-2, atol=1e-3)
