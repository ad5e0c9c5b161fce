"""``matmul`` / ``matmul_vec`` of the reference (tritium/ops/matmul.py:336-347) on the GEMM cores of the
fused loss: tcgen05 for 16-bit inputs, CUDA cores for fp32 (which must match fp32 torch to 1e-5).

Same signatures, validation messages (:130-185) and autograd contract (:310-333) as the reference. Inputs
may be any 2-D views with one unit stride (``weight.T`` is the common case, tests :24-34): the layout goes
to the kernel as a flag instead of being copied; anything else is made contiguous first.
"""

from __future__ import annotations

from typing import Any

import torch

from . import _lib
from .ops import FLOAT_DTYPES, _DTYPE_CODE, _need_cuda, _need_dtype, _on_device, _path_flags, _stream, _workspace


def _check_matmul_inputs(a: torch.Tensor, b: torch.Tensor) -> tuple[int, int, int]:
    _need_cuda("a", a)
    _need_cuda("b", b)
    _need_dtype("a", a, FLOAT_DTYPES)
    _need_dtype("b", b, FLOAT_DTYPES)
    if a.dim() != 2:
        raise ValueError("a must be a 2D tensor shaped (M, K).")
    if b.dim() != 2:
        raise ValueError("b must be a 2D tensor shaped (K, N).")
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError(f"Shape mismatch: a has shape {tuple(a.shape)}, b has shape {tuple(b.shape)}.")
    if a.dtype != b.dtype:
        raise ValueError(f"Dtype mismatch: a has dtype {a.dtype}, b has dtype {b.dtype}.")
    if a.device != b.device:
        raise ValueError(f"Device mismatch: a is on {a.device}, b is on {b.device}.")
    return m, n, k


def _layout(t: torch.Tensor) -> tuple[torch.Tensor, bool, int]:
    """(tensor, rows_are_contiguous_dim?, pitch): a [R, C] view as "element (r, c) at r * pitch + c"
    (False) or "at c * pitch + r" (True)."""
    rows, cols = t.shape
    if t.stride(1) == 1 and (rows == 1 or t.stride(0) >= cols):
        return t, False, max(t.stride(0), cols) if rows > 1 else max(cols, 1)
    if t.stride(0) == 1 and (cols == 1 or t.stride(1) >= rows):
        return t, True, max(t.stride(1), rows) if cols > 1 else max(rows, 1)
    t = t.contiguous()
    return t, False, max(cols, 1)


def _product(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    m, n, k = _check_matmul_inputs(a, b)
    c = torch.empty((m, n), device=a.device, dtype=a.dtype)
    if m == 0 or n == 0:
        return c
    if k == 0:
        return c.zero_()
    a, a_t, lda = _layout(a)       # a_t: stored as [K, M]
    b, b_t, ldb = _layout(b)       # b_t: stored as [N, K]
    dev = a.device
    L = _lib.lib()
    dtype = _DTYPE_CODE[a.dtype]
    flags = _path_flags() & ~_lib.FLAG_FORCE_TC  # "tc" stays a preference here: fp32 has no tensor-core path
    ws = _workspace(L.lce_matmul_workspace_bytes(m, n, k, dtype, flags), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_matmul(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, int(a_t), lda, int(not b_t), ldb, n, dtype,
                         ws.data_ptr(), ws.numel(), flags, _stream(dev)),
            "lce_matmul",
        )
    return c


class _MatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, a, b):
        ctx.save_for_backward(a, b)
        return _product(a, b)

    @staticmethod
    def backward(ctx: Any, *grad_outputs):
        dc = grad_outputs[0]
        a, b = ctx.saved_tensors
        da = _product(dc, b.t()) if ctx.needs_input_grad[0] else None   # [M, N] x [N, K]
        db = _product(a.t(), dc) if ctx.needs_input_grad[1] else None   # [K, M] x [M, N]
        return da, db


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Return the matrix product ``a @ b`` with autograd support (reference :336-340)."""
    if not (torch.is_grad_enabled() and (a.requires_grad or b.requires_grad)):
        return _product(a, b)
    return _MatMul.apply(a, b)


def matmul_vec(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Return the vector-matrix product ``a @ b`` for ``a`` shaped ``(K,)`` (reference :343-347)."""
    _need_cuda("a", a)
    _need_cuda("b", b)
    _need_dtype("a", a, FLOAT_DTYPES)
    _need_dtype("b", b, FLOAT_DTYPES)
    if a.dim() != 1:
        raise ValueError("a must be a 1D tensor shaped (K,).")
    if b.dim() != 2:
        raise ValueError("b must be a 2D tensor shaped (K, N).")
    if a.shape[0] != b.shape[0]:
        raise ValueError(f"Shape mismatch: a has shape {tuple(a.shape)}, b has shape {tuple(b.shape)}.")
    if a.dtype != b.dtype:
        raise ValueError(f"Dtype mismatch: a has dtype {a.dtype}, b has dtype {b.dtype}.")
    if a.device != b.device:
        raise ValueError(f"Device mismatch: a is on {a.device}, b is on {b.device}.")
    return matmul(a.unsqueeze(0), b).squeeze(0)
