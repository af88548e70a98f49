"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import wush_oracle as wo


def canon_codes(packed: np.ndarray) -> np.ndarray:
    """Unpacked E2M1 codes with -0 folded onto +0 (both dequantize to zero)."""
    c = wo.unpack_e2m1_codes(np.asarray(packed, dtype=np.uint8))
    return np.where(c == 8, 0, c)


def mismatch_fraction(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.mean(a != b)) if a.size else 0.0


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).cpu().numpy()
