"""Shared helpers for the test-suite: golden-fixture loading, bit-pattern conversions, tolerances."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

F16, F32, BF16 = 12, 13, 19
TORCH_DTYPE = {F16: torch.float16, F32: torch.float32, BF16: torch.bfloat16}

# Parity tolerances of the decode path: fp16 atol 2e-3 / rtol 2e-3, bf16 atol 1e-2 / rtol 1e-2.
ATTN_TOL = {F16: (2e-3, 2e-3), BF16: (1e-2, 1e-2), torch.float16: (2e-3, 2e-3), torch.bfloat16: (1e-2, 1e-2)}


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


def golden_names(prefix: str):
    return sorted(p.stem for p in GOLDEN.glob(f"{prefix}*.npz"))


def bits_to_float(a: np.ndarray, dtype_code: int) -> np.ndarray:
    """uint16 bit patterns (or float32 values) -> float64 values."""
    if dtype_code == F32:
        return a.astype(np.float64)
    t = torch.from_numpy(a.view(np.int16).copy()).view(TORCH_DTYPE[dtype_code])
    return t.to(torch.float64).numpy()


def bits_to_torch(a: np.ndarray, dtype_code: int) -> torch.Tensor:
    if dtype_code == F32:
        return torch.from_numpy(a.copy())
    return torch.from_numpy(a.view(np.int16).copy()).view(TORCH_DTYPE[dtype_code])


def torch_to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def assert_close(actual: np.ndarray, expected: np.ndarray, atol: float, rtol: float, what: str = ""):
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    err = np.abs(actual - expected)
    bound = atol + rtol * np.abs(expected)
    bad = err > bound
    if bad.any() or np.isnan(actual).any():
        worst = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {err.size} elements outside atol={atol} rtol={rtol}; "
            f"worst at {worst}: got {actual[worst]!r}, want {expected[worst]!r}; max abs err {err.max():.3e}")
