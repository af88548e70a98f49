"""The C-ABI library loads and exports every symbol the public header declares (CPU-only:
no kernel is launched), and argument validation works without a device."""
import ctypes

from wush_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _lib.declared_symbols()
    assert "wush_fused_quantize_mx" in names and len(names) >= 5
    for n in names:
        assert hasattr(lib, n), n
    assert lib.wush_b200_arch() == 100


def test_argument_validation_needs_no_device():
    lib = _lib.load()
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 15) // 16 * 16
    assert lib.wush_fused_quantize_mx(None, p, 32, p, p, 4, 0, 1, 32, 0, None) == -1
    assert lib.wush_fused_quantize_mx(p, p, 32, p, p, 4, 0, 1, 48, 0, None) == -2      # cols % 32
    assert lib.wush_fused_quantize_mx(p, p, 64, p, p, 4, 0, 1, 128, 0, None) == -2     # matrix width
    assert lib.wush_fused_quantize_mx(p, p, 32, p, p, 3, 0, 1, 32, 0, None) == -2      # sf_cols % 4
    assert lib.wush_fused_quantize_mx(p, p, 32, p, p, 4, 7, 1, 32, 0, None) == -4      # layout
    assert lib.wush_fused_quantize_mx(p + 2, p, 32, p, p, 4, 0, 1, 32, 0, None) == -3  # alignment
    assert lib.wush_fused_quantize_mx(p, p, 32, p, p, 4, 0, 0, 32, 0, None) == 0       # empty input
    assert lib.wush_fused_quantize_nv(p, p, 16, None, p, p, 4, 0, 1, 32, 0, None) == -1
    assert lib.wush_sf_to_blocked(p, p, 0, 0, None) == 0
