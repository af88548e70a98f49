"""Compare the NumPy oracle with the reference's torch code on fresh seeded inputs.

TEST INFRASTRUCTURE.  Run by hand, or by tests/test_oracle_vs_reference.py when a
reference checkout is present:

    python oracle/check_against_reference.py /path/to/WUSH

Exits non-zero on the first byte that differs.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(ref_root: str, seeds=(11, 12, 13)) -> int:
    sys.dont_write_bytecode = True
    sys.path.insert(0, ROOT)
    from oracle import wush_oracle as wo
    cwd = os.getcwd()
    os.chdir(ref_root)
    sys.path.insert(0, ref_root)
    try:
        from src.quantization import wush_gptq as ref
    finally:
        os.chdir(cwd)
    kws = dict(mxfp4=dict(group_size=32, scale_dtype=torch.float8_e8m0fnu, scale_scale=4., global_scale=3.),
               nvfp4=dict(group_size=16, scale_dtype=torch.float8_e4m3fn, scale_scale=6., global_scale=10.))
    checked = 0
    for seed in seeds:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(64, 512, generator=g)
        x[:, torch.randperm(512, generator=g)[:3]] *= 50.0
        for xi in (x, x.to(torch.bfloat16), x * 1e-3, x.to(torch.bfloat16) * 2.0 ** -100):
            for fmt, kw in kws.items():
                r = ref.rtn_xxfp4(xi, fp4_rounding_mode="even", **kw)
                o = wo.rtn_xxfp4(xi.to(torch.float64).numpy(), fmt)
                assert np.array_equal(o["e2m1"], r["e2m1"].view(torch.uint8).numpy()), (seed, fmt, "codes")
                assert np.array_equal(o["scale_quant"], r["scale_quant"].view(torch.uint8).numpy()), (seed, fmt, "scales")
                checked += o["e2m1"].size
        t = torch.randn(16, 32, 32, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
        xb = x.to(torch.bfloat16)
        got = wo.block_transform(xb.to(torch.float64).numpy(), t.numpy())
        want = ref.block_transform(xb.to(torch.float32), t).to(torch.float64).numpy()
        assert np.array_equal(got.astype(np.float32).astype(np.float64), want), (seed, "block_transform")
    print(f"oracle == reference on {checked} packed bytes and {len(seeds)} transforms")
    return 0


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("WUSH_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: check_against_reference.py <reference checkout>   (or set WUSH_REFERENCE_ROOT)")
    sys.exit(run(root))
