"""Whole quantized-linear path on the GPU: calibration Hessian -> WUSH matrices -> weight codes (CPU oracle, the
reference's RTN recipe) -> FPQuantLinear.forward = fused transform+quantize + FP4 GEMM, against the CPU oracle of
the same pipeline (1e-2 relative Frobenius) and, as a sanity bound, against the unquantized bf16 product."""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import wush_oracle as wo

pytestmark = pytest.mark.gpu


def _wush_setup(hidden, rows_out, fmt, dev):
    from wush_b200.hessian import DistributedHessian
    g = wo.FORMATS[fmt]["group"]
    calib = [synth.activations(512, hidden, seed=80 + i) for i in range(2)]
    dh = DistributedHessian(hidden, dev)
    for c in calib:
        dh.update(c.to(dev))
    h = dh.finalize().double().cpu().numpy()
    h[np.diag_indices(hidden)] += 1e-2 * np.trace(h) / hidden            # wush_gptq.py:197-199
    basis = np.linalg.cholesky(h).T                                       # upper: basis^T basis = h
    w = synth.bf16_to_f64(synth.weights(rows_out, hidden, seed=5))
    y = basis @ w.T
    t = np.stack([wo.get_transform(basis[i:i + g, i:i + g], y[i:i + g], "wush") for i in range(0, hidden, g)])
    # weight side of the transform: W_n T_n^-1 per group, then RTN (force_rtn path of quantize_layers)
    wt = np.concatenate([w[:, n * g:(n + 1) * g] @ np.linalg.inv(t[n]) for n in range(hidden // g)], axis=1)
    wq = wo.rtn_xxfp4(wt, fmt)
    return w, t, wq


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_wush_linear_end_to_end(fmt):
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    hidden, rows_out, tokens = 1024, 512, 200
    g = wo.FORMATS[fmt]["group"]
    w, t, wq = _wush_setup(hidden, rows_out, fmt, dev)
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype(fmt), hadamard_group_size=g, transform_init="wush")
    layer = FPQuantLinear(hidden, rows_out, cfg, bias=True, device=dev)
    mat = wo.transform_to_matrix(t)
    gs = wo.FORMATS[fmt]["global_scale"]       # what exported checkpoints carry (wush_gptq.py:588)
    layer.load_quantized(torch.from_numpy(wq["e2m1"]), torch.from_numpy(wq["scale_quant"]), torch.from_numpy(mat),
                         torch.tensor([gs]), torch.tensor([gs]))
    bias = torch.linspace(-1, 1, rows_out, dtype=torch.bfloat16, device=dev)
    layer.bias.data.copy_(bias)
    x = synth.activations(tokens, hidden, seed=90)
    y = layer(x.to(dev).view(2, tokens // 2, hidden))
    torch.cuda.synchronize()
    assert y.shape == (2, tokens // 2, rows_out) and y.dtype == torch.bfloat16
    got = y.double().cpu().numpy().reshape(tokens, rows_out)
    xq = wo.fused_transform_quant(synth.bf16_to_f64(x), mat, fmt)
    want = wo.fp4_gemm(xq["e2m1"], xq["scale_quant"], wq["e2m1"], wq["scale_quant"], 1.0 / (gs * gs), fmt)
    want = want + bias.double().cpu().numpy()[None, :]
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
    exact = synth.bf16_to_f64(x) @ w.T + bias.double().cpu().numpy()[None, :]
    rel = np.linalg.norm(got - exact) / np.linalg.norm(exact)
    assert rel < 0.25, rel                      # W4A4 quantization error, not a kernel tolerance


def test_hadamard_linear_quantizes_its_own_weight():
    from wush_b200.linear import FPQuantConfig, FPQuantLinear
    dev = torch.device("cuda:0")
    layer = FPQuantLinear(512, 256, FPQuantConfig(), bias=False, device=dev)
    w = synth.weights(256, 512, seed=6)
    layer.weight.data.copy_(w.to(dev))
    layer.pre_forward()
    assert layer.weight is None and layer.qweight.shape == (256, 256) and layer.scales.shape == (256, 16)
    x = synth.activations(64, 512, seed=7)
    y = layer(x.to(dev)).double().cpu().numpy()
    exact = synth.bf16_to_f64(x) @ synth.bf16_to_f64(w).T
    assert np.linalg.norm(y - exact) / np.linalg.norm(exact) < 0.25
    with pytest.raises(NotImplementedError):       # the per-group transform has no quest variant (nor in the reference)
        FPQuantLinear(512, 256, FPQuantConfig(forward_method="quest", transform_init="wush"), device=dev)
    with pytest.raises(ValueError):
        FPQuantLinear(512, 256, FPQuantConfig(forward_method="median"), device=dev)


def test_quest_linear():
    """forward_method="quest": global scales 1.0, weights and activations scaled by their groups' standard deviation
    (with clipping); the layer output is the dequantized product of the two quantized operands."""
    from oracle import wush_oracle as wo
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    layer = FPQuantLinear(512, 256, FPQuantConfig(forward_method="quest"), bias=False, device=dev)
    assert float(layer.weight_global_scale) == 1.0 and float(layer.act_global_scale) == 1.0
    w = synth.weights(256, 512, seed=16)
    layer.weight.data.copy_(w.to(dev))
    layer.pre_forward()
    x = synth.activations(96, 512, seed=17)
    y = layer(x.to(dev)).double().cpu().numpy()
    had = synth.bf16_to_f64(layer.forward_hadamard_matrix.cpu())
    deq = lambda t: wo.quest_mxfp4(wo.block_transform(synth.bf16_to_f64(t), had.T).astype(np.float32))["fake_quant"].astype(np.float64)
    want = deq(x) @ deq(w).T
    assert np.linalg.norm(y - want) <= 2e-2 * np.linalg.norm(want)          # ties and bf16 output rounding
    exact = synth.bf16_to_f64(x) @ synth.bf16_to_f64(w).T
    assert np.linalg.norm(y - exact) / np.linalg.norm(exact) < 0.3
    nv = FPQuantLinear(512, 256, FPQuantConfig(forward_dtype=FPQuantDtype.NVFP4, forward_method="quest", hadamard_group_size=16),
                       bias=False, device=dev)
    assert float(nv.weight_global_scale) == 10.0


@pytest.mark.parametrize("fmt,rtn", [("mxfp4", False), ("nvfp4", True)])
def test_calibrate_sweep_export_load_forward(fmt, rtn):
    """The whole pipeline on the GPU: Hessian from calibration activations -> column sweep (quantize_layers, two
    layers sharing the input) -> realquant checkpoint entries -> FPQuantLinear.  The real-quant layer (fused
    quantize + FP4 GEMM) must agree with the pseudo-quantized layer the sweep returned (same codes, same
    transforms; the two differ only in where values are rounded to bf16)."""
    from wush_b200 import gptq
    from wush_b200.hessian import DistributedHessian
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    hidden, tokens = 512, 256
    g = wo.FORMATS[fmt]["group"]
    dh = DistributedHessian(hidden, dev)
    for i in range(3):
        dh.update(synth.activations(700, hidden, seed=40 + i).to(dev))
    h = dh.finalize()
    w1, w2 = synth.weights(256, hidden, seed=6).to(dev), synth.weights(128, hidden, seed=7).to(dev)
    pseudo, results = gptq.quantize_layers(w1, w2, hessian=h, quant_type=fmt, transform_class="wush", force_rtn=rtn)
    x = synth.activations(tokens, hidden, seed=50).to(dev)
    for layer_p, res, w in zip(pseudo, results, (w1, w2)):
        entry = gptq.export_realquant(res, fmt)
        assert entry["qweight"].dtype == torch.uint8 and entry["forward_hadamard_matrix"].shape == (g, hidden)
        cfg = FPQuantConfig(forward_dtype=FPQuantDtype(fmt), hadamard_group_size=g, transform_init="wush")
        real = FPQuantLinear(hidden, w.shape[0], cfg, bias=False, device=dev)
        real.load_quantized(entry["qweight"], entry["scales"], entry["forward_hadamard_matrix"],
                            entry["weight_global_scale"], entry["act_global_scale"])
        y_real, y_pseudo = real(x).float(), layer_p(x).float()
        rel = float((y_real - y_pseudo).norm() / y_pseudo.norm())
        assert rel < 2e-2, rel
        exact = x.float() @ w.float().T
        assert float((y_real - exact).norm() / exact.norm()) < 0.25


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_state_dict_loading_matches_load_quantized(fmt):
    """The reference's checkpoint protocol copies qweight / scales / matrices / global scales into the module's
    buffers through load_state_dict; the layer must then behave exactly like one filled by load_quantized(),
    also after a second, different state dict (nothing derived from the old buffers may survive) and after
    pre_forward(), which the loader calls on every layer."""
    from wush_b200 import gptq
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    hidden, rows_out = 512, 256
    g = wo.FORMATS[fmt]["group"]
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype(fmt), hadamard_group_size=g, transform_init="wush")
    x = synth.activations(96, hidden, seed=3).to(dev)
    entries = []
    for seed in (11, 12):
        w = synth.weights(rows_out, hidden, seed=seed).to(dev)
        _, results = gptq.quantize_layers(w, hessian=None, quant_type=fmt, transform_class="hadamard", force_rtn=True)
        entries.append(gptq.export_realquant(results[0], fmt))
    ref_layers = []
    for e in entries:
        ref = FPQuantLinear(hidden, rows_out, cfg, bias=False, device=dev)
        ref.load_quantized(e["qweight"], e["scales"], e["forward_hadamard_matrix"], e["weight_global_scale"],
                           e["act_global_scale"])
        ref_layers.append(ref)
    layer = FPQuantLinear(hidden, rows_out, cfg, bias=False, device=dev)
    for e, ref in zip(entries, ref_layers):
        missing = layer.load_state_dict(e, strict=False)
        assert not missing.unexpected_keys
        layer.pre_forward()
        assert layer.weight is None
        assert torch.equal(layer(x), ref(x))
    assert not torch.equal(ref_layers[0](x), ref_layers[1](x))


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("tokens", [8, 300])
def test_bias_and_residual_in_the_gemm_epilogue_are_bit_identical_to_separate_adds(fmt, tokens):
    """tokens = 8 runs the split-K kernel (the CTAs of a cluster add their partial tiles through shared memory and
    finish the output), 300 the CTA-pair kernel."""
    from wush_b200 import qutlass_ops as ops
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    hidden, rows_out = 1024, 384
    g = wo.FORMATS[fmt]["group"]
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype(fmt), hadamard_group_size=g, transform_init="hadamard")
    layer = FPQuantLinear(hidden, rows_out, cfg, bias=True, device=dev)
    layer.weight.data.copy_(synth.weights(rows_out, hidden, seed=21).to(dev))
    layer.bias.data.copy_(torch.randn(rows_out, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16))
    layer.pre_forward()
    x = synth.activations(tokens, hidden, seed=22).to(dev)
    res = synth.activations(tokens, rows_out, seed=23).to(dev)
    fused = layer(x, residual=res)
    scales_blocked, alpha = layer._derived()
    xq, xs = ops._quantize(x, layer.forward_hadamard_matrix, "mx" if fmt == "mxfp4" else "nv",
                           layer.act_global_scale.float() if fmt == "nvfp4" else None, sf_layout=1)
    plain = ops.matmul_fp4_blocked(xq, layer.qweight, xs.view(-1), scales_blocked.view(-1), alpha,
                                   "mx" if fmt == "mxfp4" else "nv")
    want = plain + layer.bias           # bf16 tensor arithmetic: one rounding per step, as in the reference
    want = want + res
    assert torch.equal(fused, want)
    # in place: the residual buffer receives the result
    buf = res.clone()
    ops.matmul_fp4_blocked(xq, layer.qweight, xs.view(-1), scales_blocked.view(-1), alpha,
                           "mx" if fmt == "mxfp4" else "nv", bias=layer.bias, residual=buf, out=buf)
    assert torch.equal(buf, want)


def test_single_layer_pipeline_at_4096_through_a_checkpoint_file(tmp_path):
    """One 4096 x 4096 layer end to end at the size of the reference's CPU-runnable case: second moment from 16 x 2048
    calibration tokens, MXFP4 round-to-nearest sweep with WUSH transforms, checkpoint written to disk and read
    back, real-quant forward of 2048 tokens.  The layer loaded from the file must give the bits of the layer filled in
    memory, and both must agree with the CPU pseudo-quantizer (oracle sweep on sampled weight rows with the transforms
    the GPU chose, oracle activation quantizer, float64 product) within 1e-2."""
    from wush_b200 import checkpoint, gptq
    from wush_b200.hessian import DistributedHessian
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    hidden, tokens = 4096, 2048
    dh = DistributedHessian(hidden, dev)
    for i in range(16):
        dh.update(synth.activations(2048, hidden, seed=500 + i).to(dev)[None])
    h = dh.finalize()
    assert dh.num_samples == 16 * 2048
    w = synth.weights(hidden, hidden, seed=520)
    res = gptq.gptq_babai_sweep(w.to(dev), h, "mxfp4", "wush", force_rtn=True)
    entry = gptq.export_realquant({"transform_basis": res["transform_basis"], "qweight": res["qweight"],
                                   "scale_quant": res["scale_quant"], "global_scale": res["global_scale"]}, "mxfp4")
    name = "model.layers.0.self_attn.q_proj"
    checkpoint.export_quantized_model(str(tmp_path), {name: entry}, None, {"hidden_size": hidden}, hadamard_group_size=32,
                                      format="mxfp", transform_class="wush")
    from_file = checkpoint.load_quantized_layers(str(tmp_path), device=dev)[name]
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, hadamard_group_size=32, transform_init="wush")
    in_memory = FPQuantLinear(hidden, hidden, cfg, bias=False, device=dev)
    in_memory.load_quantized(entry["qweight"], entry["scales"], entry["forward_hadamard_matrix"],
                             entry["weight_global_scale"], entry["act_global_scale"])
    x = synth.activations(tokens, hidden, seed=530)
    y_file, y_mem = from_file(x.to(dev)), in_memory(x.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(y_file, y_mem)
    # CPU pseudo-quantizer on sampled output features
    rows = np.sort(np.random.default_rng(0).choice(hidden, size=64, replace=False))
    t = res["transform_basis"].double().cpu().numpy()
    h64 = h.double().cpu().numpy()
    ref_w = wo.gptq_babai_outer(synth.bf16_to_f64(w)[rows], h64, "mxfp4", "wush", True, transform_fn=lambda b, basis, y: t[b])
    got_scales = res["scale_quant"].view(torch.uint8).cpu().numpy()[rows]
    got_codes = wo.unpack_e2m1_codes(res["qweight"].cpu().numpy()[rows])
    assert np.array_equal(got_scales, ref_w["scale_quant"])
    assert np.mean(got_codes != ref_w["codes"]) <= 1e-3
    mat = wo.transform_to_matrix(t)
    ref_x = wo.fused_transform_quant(synth.bf16_to_f64(x), mat, "mxfp4")["fake_quant"]
    want = ref_x @ ref_w["fake_quant"].T
    got = y_mem.double().cpu().numpy()[:, rows]
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)


@pytest.mark.parametrize("fmt,size,init", [("mxfp4", 128, "hadamard"), ("mxfp4", 64, "gsr"), ("nvfp4", 64, "hadamard")])
def test_layer_with_a_transform_wider_than_the_scale_group(fmt, size, init):
    """hadamard_group_size 64 / 128 (and the sequency-ordered "gsr" columns): the layer quantizes its weight and its
    activations with one shared square matrix per block of that many channels; scales stay per 32 / 16 channels.
    The output equals the product of the two dequantized operands (rotations cancel: H H^T = I up to bf16)."""
    from oracle import wush_oracle as wo
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    dev = torch.device("cuda:0")
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype(fmt), hadamard_group_size=size, transform_init=init)
    layer = FPQuantLinear(1024, 256, cfg, bias=False, device=dev)
    w = synth.weights(256, 1024, seed=26)
    layer.weight.data.copy_(w.to(dev))
    if fmt == "nvfp4":                     # the oracle's NVFP4 quantizer is the exported one: tensor scale 10
        layer.weight_global_scale.fill_(10.0)
        layer.act_global_scale.fill_(10.0)
    layer.pre_forward()
    group = 32 if fmt == "mxfp4" else 16
    assert layer.forward_hadamard_matrix.shape == (size, size) and layer.scales.shape == (256, 1024 // group)
    mat = synth.bf16_to_f64(layer.forward_hadamard_matrix.cpu())
    assert np.allclose(mat @ mat.T, np.eye(size), atol=2e-2)
    if init == "gsr":                      # column j changes sign j times
        assert np.array_equal((np.diff(np.sign(mat), axis=0) != 0).sum(axis=0), np.arange(size))
    x = synth.activations(96, 1024, seed=27)
    y = layer(x.to(dev)).double().cpu().numpy()
    deq = lambda t: wo.rtn_xxfp4(wo.wide_transform(synth.bf16_to_f64(t), mat).astype(np.float32).astype(np.float64),
                                 fmt)["fake_quant"]
    want = deq(x) @ deq(w).T
    assert np.linalg.norm(y - want) <= 1e-2 * np.linalg.norm(want)
    exact = synth.bf16_to_f64(x) @ synth.bf16_to_f64(w).T
    assert np.linalg.norm(y - exact) / np.linalg.norm(exact) < 0.25
