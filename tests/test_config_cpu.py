"""FPQuantConfig validation and the layer's buffers on CPU (no kernel runs): the accepted transform sizes and methods
are those of the reference's validate_config (inference_lib/src/fp_quant/utils/config.py:29-50) minus training."""
import pytest
import torch

from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear, validate_config


@pytest.mark.parametrize("dtype,sizes", [(FPQuantDtype.MXFP4, (32, 64, 128)), (FPQuantDtype.NVFP4, (16, 32, 64, 128))])
def test_hadamard_group_sizes(dtype, sizes):
    for n in sizes:
        validate_config(FPQuantConfig(forward_dtype=dtype, hadamard_group_size=n))
    for n in (8, 48, 256) + ((16,) if dtype == FPQuantDtype.MXFP4 else ()):
        with pytest.raises(ValueError):
            validate_config(FPQuantConfig(forward_dtype=dtype, hadamard_group_size=n))
    with pytest.raises(NotImplementedError):        # a per-group matrix is as wide as the scale group
        validate_config(FPQuantConfig(forward_dtype=dtype, hadamard_group_size=sizes[1], transform_init="wush"))


def test_methods_and_global_scales():
    for method, dtype, size, want in (("abs_max", FPQuantDtype.MXFP4, 32, 3.0), ("quest", FPQuantDtype.MXFP4, 32, 1.0),
                                      ("abs_max", FPQuantDtype.NVFP4, 16, 3.0), ("quest", FPQuantDtype.NVFP4, 16, 10.0)):
        layer = FPQuantLinear(256, 64, FPQuantConfig(forward_dtype=dtype, forward_method=method, hadamard_group_size=size),
                              bias=False, device="cpu")
        assert float(layer.weight_global_scale) == want and float(layer.act_global_scale) == want
        assert layer.weight_global_scale.dtype == torch.bfloat16
    with pytest.raises(ValueError):
        validate_config(FPQuantConfig(forward_method="median"))
    with pytest.raises(NotImplementedError):
        validate_config(FPQuantConfig(forward_method="quest", transform_init="wush"))
    with pytest.raises(NotImplementedError):
        validate_config(FPQuantConfig(pseudoquantization=True))


def test_buffer_shapes_follow_the_scale_group_not_the_transform_size():
    layer = FPQuantLinear(512, 64, FPQuantConfig(hadamard_group_size=128), bias=True, device="cpu")
    assert layer.scales.shape == (64, 16) and layer.qweight.shape == (64, 256)
    assert layer.forward_hadamard_matrix.shape == (128, 128)
    nv = FPQuantLinear(512, 64, FPQuantConfig(forward_dtype=FPQuantDtype.NVFP4, hadamard_group_size=64), device="cpu")
    assert nv.scales.shape == (64, 32) and nv.forward_hadamard_matrix.shape == (64, 64)
    wush = FPQuantLinear(512, 64, FPQuantConfig(transform_init="wush"), device="cpu")
    assert wush.forward_hadamard_matrix.shape == (32, 512)
    with pytest.raises(ValueError):                 # the GEMM needs K % 128 == 0
        FPQuantLinear(96, 64, FPQuantConfig(), device="cpu")
