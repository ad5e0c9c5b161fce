"""Shared helpers for the parity tests."""

from __future__ import annotations

import torch

# Acceptance tolerances of this path, stated once:
#   loss: |new - oracle| / |oracle| <= 1e-3
#   dX, dW (16-bit inputs): max|new - oracle| / max|oracle| <= 2e-2
#   fp32 inputs: rtol = atol = 1e-5 on gradients (the reference's own fp32 tolerance,
#   tests/_utils.py:14-17 of the reference), which rules out TF32.
LOSS_RTOL = 1e-3
GRAD_RTOL_16BIT = 2e-2
FP32_TOL = 1e-5


def rel_loss_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    return float(((got - ref).abs() / ref.abs().clamp_min(1e-30)).max())


def scaled_max_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def reference_tolerances(dtype: torch.dtype, accumulated: bool = False) -> tuple[float, float]:
    """(rtol, atol) the reference's tests use (its tests/_utils.py:14-29)."""
    if dtype == torch.float32:
        return 1e-5, 1e-5
    return (3e-2, 3e-2) if accumulated else (2e-2, 2e-2)
