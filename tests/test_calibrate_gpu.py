"""The calibration driver (wush_b200/calibrate.py) on the GPU with the real kernels: a two-block toy model is
calibrated and quantized (MXFP4, WUSH transforms, round-to-nearest); the block outputs of the quantized model stay
close to the original, the export entries load into FPQuantLinear layers whose real-quant forward agrees with the
pseudo-quantized layers the driver left in the model, and the shared second moments are what a float64 accumulation
of the layer inputs gives."""
import types

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_toy_model_end_to_end():
    from tests.test_calibrate_cpu import _Model, VOCAB
    from wush_b200 import calibrate
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    import tests.test_calibrate_cpu as toy
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    # the kernels want in_features % 128 == 0: widen the toy model
    toy.HID, toy.FFN = 256, 384
    try:
        model = _Model().to(dev).to(torch.bfloat16)
    finally:
        toy.HID, toy.FFN = 64, 96
    g = torch.Generator().manual_seed(3)
    data = [torch.randint(0, VOCAB, (1, 64), generator=g) for _ in range(6)]
    ref_out = [model(d.to(dev)).float() for d in data]
    args = types.SimpleNamespace(format="mxfp", gptq=False, transform_class="wush", export_quantized_model="realquant",
                                 cpu_offload_activations=False, cpu_offload_modules=False, dtype="auto")
    seen = []
    qsd, _ = calibrate.wush_quantization_gptq(model, data, args, dev, log=lambda s: seen.append(s))
    assert len(qsd) == 14 and any("l2_loss" in s for s in seen)
    q_out = [model(d.to(dev)).float() for d in data]
    rel = max(float((a - b).norm() / b.norm()) for a, b in zip(q_out, ref_out))
    assert rel < 0.3, rel                                       # W4A4 error of a random toy model, not a kernel tolerance
    # real-quant layers from the export entries agree with the pseudo-quantized layers left in the model
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, hadamard_group_size=32, transform_init="wush")
    x = torch.randn(40, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    for name in ("model.layers.0.self_attn.q_proj", "model.layers.1.mlp.gate_proj"):
        e = qsd[name]
        real = FPQuantLinear(256, e["qweight"].shape[0], cfg, bias=False, device=dev)
        real.load_state_dict(e, strict=False)
        real.pre_forward()
        pseudo = model.get_submodule(name.replace("model.layers.", "model.layers."))
        yr, yp = real(x).float(), pseudo(x).float()
        assert float((yr - yp).norm() / yp.norm()) < 2e-2
