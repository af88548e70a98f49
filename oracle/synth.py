"""Seeded synthetic inputs for tests and benchmarks -- TEST INFRASTRUCTURE.

The reference calibrates on web text through real checkpoints; neither exists offline,
so tensors with the benchmark configurations' shapes and value distributions stand in:
activations N(0,1) in bf16 with a seeded 0.5 % of channels multiplied by 50, weights
N(0, 0.02^2) in bf16, per-group WUSH matrices built by the reference's own recipe
(src/quantization/wush_gptq.py:304-347) from a synthetic second moment.

All generators use torch CPU generators so the same seed gives the same bits on any
machine with the same torch build.
"""
from __future__ import annotations

import numpy as np
import torch

from . import wush_oracle as wo

SEED_DATA, SEED_OUTLIER, SEED_WEIGHT, SEED_SPD = 0, 1, 2, 3


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def outlier_channels(hidden: int, seed: int = SEED_OUTLIER) -> torch.Tensor:
    k = max(1, int(0.005 * hidden))
    return torch.randperm(hidden, generator=_gen(seed))[:k]


def activations(tokens: int, hidden: int, seed: int = SEED_DATA, outlier_seed: int = SEED_OUTLIER,
                dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """(tokens, hidden) activations: N(0,1), outlier channels x50, rounded to dtype."""
    x = torch.randn(tokens, hidden, generator=_gen(seed), dtype=torch.float32)
    x[:, outlier_channels(hidden, outlier_seed)] *= 50.0
    return x.to(dtype)


def weights(rows: int, cols: int, seed: int = SEED_WEIGHT, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return (torch.randn(rows, cols, generator=_gen(seed), dtype=torch.float32) * 0.02).to(dtype)


def bf16_to_f64(x: torch.Tensor) -> np.ndarray:
    return x.to(torch.float64).numpy()


def wush_matrix(hidden: int, group: int, seed: int = SEED_SPD, calib_tokens: int = 256, rows: int = 64) -> np.ndarray:
    """(group, hidden) per-group WUSH matrix in bf16-representable float64.

    For every group of channels: second moment of a small synthetic calibration batch,
    damped like the reference (1 % of the mean diagonal), upper Cholesky factor ->
    'basis'; a random (group, rows) block stands for the weight-side 'y'.  Those go
    through :func:`oracle.wush_oracle.get_transform` ('wush').  Block-diagonal second
    moments keep this cheap for hidden = 14336; the kernels only see the matrix.
    """
    g = _gen(seed)
    n = hidden // group
    xc = torch.randn(calib_tokens, hidden, generator=g, dtype=torch.float64)
    xc[:, outlier_channels(hidden)] *= 50.0
    yb = torch.randn(n, group, rows, generator=g, dtype=torch.float64).numpy() * 0.02
    xc = xc.numpy().reshape(calib_tokens, n, group)
    t = np.empty((n, group, group))
    for i in range(n):
        h = xc[:, i, :].T @ xc[:, i, :] / calib_tokens
        h[np.diag_indices(group)] += 1e-2 * np.trace(h) / group
        basis = np.linalg.cholesky(h).T          # upper: basis.T @ basis = h
        t[i] = wo.get_transform(basis, basis @ yb[i], "wush", round_bf16=True)
    return wo.transform_to_matrix(t)


def hadamard_matrix(group: int) -> np.ndarray:
    """(group, group) shared normalized Hadamard, bf16-representable."""
    return wo.round_to_bf16(wo.normalized_hadamard(group))


def to_bf16_tensor(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16)
