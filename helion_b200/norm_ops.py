"""RMSNorm and residual-add RMSNorm: the reference's ``tritium.rmsnorm``, ``tritium.residual_rmsnorm`` and
``tritium.rmsnorm_backward`` (tritium/ops/rmsnorm.py:577-613, :737-778) over the C ABI. This is the op that
produces the hidden states the fused linear-cross-entropy head consumes.

Same positional signatures, validation order and messages as the reference (:283-317, :577-597,
:663-676), including its refusal of hidden sizes whose next power of two exceeds 65536. What differs
is underneath: one pass over ``dy`` and ``x`` in the backward (the reference reads them twice to form
``dweight``) and a ``dweight`` summed in a fixed order for every shape (the reference uses atomics
below hidden = 512).
"""

from __future__ import annotations

from typing import Any

import torch

from . import _lib
from .ops import FLOAT_DTYPES, _DTYPE_CODE, _need_cuda, _need_dtype, _on_device, _stream, _workspace

MAX_RMSNORM_HIDDEN_NEXT_POW2 = 65536


def _next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def _need_contiguous(name: str, t: torch.Tensor, op: str) -> None:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous for tritium.{op}.")


def check_inputs(x: torch.Tensor, weight: torch.Tensor) -> int:
    """The reference's _check_rmsnorm_inputs (tritium/ops/rmsnorm.py:283-317)."""
    _need_cuda("x", x)
    _need_cuda("weight", weight)
    _need_dtype("x", x, FLOAT_DTYPES)
    _need_dtype("weight", weight, FLOAT_DTYPES)
    if x.dim() < 1:
        raise ValueError("x must have at least 1 dimension.")
    hidden = x.shape[-1]
    if tuple(weight.shape) != (hidden,):
        raise ValueError(f"Shape mismatch: weight has shape {tuple(weight.shape)}, expected ({hidden},).")
    if weight.dtype != x.dtype:
        raise ValueError(f"Dtype mismatch: weight has dtype {weight.dtype}, x has dtype {x.dtype}.")
    if weight.device != x.device:
        raise ValueError(f"Device mismatch: weight is on {weight.device}, x is on {x.device}.")
    if _next_pow2(hidden) > MAX_RMSNORM_HIDDEN_NEXT_POW2:
        raise ValueError(f"Unsupported hidden size: next_power_of_2({hidden}) exceeds {MAX_RMSNORM_HIDDEN_NEXT_POW2}.")
    _need_contiguous("x", x, "rmsnorm")
    _need_contiguous("weight", weight, "rmsnorm")
    return hidden


def _rows(x: torch.Tensor) -> int:
    return x.numel() // x.shape[-1] if x.shape[-1] else 0


def _forward(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, want_rstd: bool):
    """(out, residual_out or None, rstd or None); inputs already validated."""
    hidden = x.shape[-1]
    n_rows = _rows(x)
    out = torch.empty_like(x)
    res_out = torch.empty_like(x) if residual is not None else None
    rstd = torch.empty((n_rows,), dtype=torch.float32, device=x.device) if want_rstd else None
    if n_rows == 0 or hidden == 0:
        return out, res_out, rstd
    L = _lib.lib()
    with _on_device(x.device):
        _lib.check(
            L.lce_rmsnorm_forward(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                  weight.data_ptr(), out.data_ptr(),
                                  res_out.data_ptr() if res_out is not None else None,
                                  rstd.data_ptr() if rstd is not None else None, n_rows, hidden, float(eps),
                                  _DTYPE_CODE[x.dtype], _stream(x.device)),
            "lce_rmsnorm_forward",
        )
    return out, res_out, rstd


def _backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor | None,
              dresidual: torch.Tensor | None, eps: float, want_dweight: bool):
    """(dx, dweight or None) for contiguous ``dy`` / ``x`` of equal shape."""
    hidden = x.shape[-1]
    n_rows = _rows(x)
    dx = torch.empty_like(x)
    dweight = torch.empty_like(weight) if want_dweight else None
    if hidden == 0:
        return dx, dweight
    L = _lib.lib()
    code = _DTYPE_CODE[x.dtype]
    ws = _workspace(L.lce_rmsnorm_backward_workspace_bytes(n_rows, hidden, code) if want_dweight else 0, x.device)
    with _on_device(x.device):
        _lib.check(
            L.lce_rmsnorm_backward(dy.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                   rstd.data_ptr() if rstd is not None else None,
                                   dresidual.data_ptr() if dresidual is not None else None, dx.data_ptr(),
                                   dweight.data_ptr() if dweight is not None else None, n_rows, hidden, float(eps),
                                   code, ws.data_ptr(), ws.numel(), _stream(x.device)),
            "lce_rmsnorm_backward",
        )
    return dx, dweight


def rmsnorm_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """``(dx, dweight)`` of ``rmsnorm``, recomputing rstd from ``x`` (reference :577-613)."""
    check_inputs(x, weight)
    _need_cuda("dy", dy)
    if dy.shape != x.shape:
        raise ValueError(f"Shape mismatch: dy has shape {tuple(dy.shape)}, x has shape {tuple(x.shape)}.")
    if dy.dtype != x.dtype:
        raise ValueError(f"Dtype mismatch: dy has dtype {dy.dtype}, x has dtype {x.dtype}.")
    if dy.device != x.device:
        raise ValueError(f"Device mismatch: dy is on {dy.device}, x is on {x.device}.")
    _need_contiguous("dy", dy, "rmsnorm_backward")
    dx, dweight = _backward(dy, x, weight, None, None, eps, True)
    return dx, dweight


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x, weight, eps):
        out, _, rstd = _forward(x, None, weight, eps, True)
        ctx.save_for_backward(x, weight, rstd)
        return out

    @staticmethod
    def backward(ctx: Any, *grad_outputs):
        if not ctx.needs_input_grad[0] and not ctx.needs_input_grad[1]:
            return None, None, None
        x, weight, rstd = ctx.saved_tensors
        dy = grad_outputs[0].contiguous()
        dx, dweight = _backward(dy, x, weight, rstd, None, 0.0, ctx.needs_input_grad[1])
        return (dx if ctx.needs_input_grad[0] else None), dweight, None


class _ResidualRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x, residual, weight, eps):
        out, res_out, rstd = _forward(x, residual, weight, eps, True)
        ctx.save_for_backward(res_out, weight, rstd)
        return out, res_out

    @staticmethod
    def backward(ctx: Any, *grad_outputs):
        if not any(ctx.needs_input_grad[:3]):
            return None, None, None, None
        res_out, weight, rstd = ctx.saved_tensors
        dy = grad_outputs[0].contiguous()
        dres = grad_outputs[1].contiguous()
        # dz = d(out)/dz + d(residual_out): the add rides in the same pass
        dz, dweight = _backward(dy, res_out, weight, rstd, dres, 0.0, ctx.needs_input_grad[2])
        return (dz if ctx.needs_input_grad[0] else None), (dz if ctx.needs_input_grad[1] else None), dweight, None


def _autograd(*tensors: torch.Tensor) -> bool:
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x**2) + eps) * weight`` over the last dimension (reference :737-746)."""
    check_inputs(x, weight)
    if not _autograd(x, weight):
        return _forward(x, None, weight, eps, False)[0]
    return _RMSNorm.apply(x, weight, eps)


def _check_residual(x: torch.Tensor, residual: torch.Tensor) -> None:
    _need_cuda("residual", residual)
    if residual.shape != x.shape:
        raise ValueError(f"Shape mismatch: residual has shape {tuple(residual.shape)}, x has shape {tuple(x.shape)}.")
    if residual.dtype != x.dtype:
        raise ValueError(f"Dtype mismatch: residual has dtype {residual.dtype}, x has dtype {x.dtype}.")
    if residual.device != x.device:
        raise ValueError(f"Device mismatch: residual is on {residual.device}, x is on {x.device}.")
    _need_contiguous("residual", residual, "residual_rmsnorm")


def residual_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """``(rmsnorm(x + residual), x + residual)`` in one pass (reference :749-778)."""
    check_inputs(x, weight)
    _check_residual(x, residual)
    if not _autograd(x, residual, weight):
        out, res_out, _ = _forward(x, residual, weight, eps, False)
        return out, res_out
    return _ResidualRMSNorm.apply(x, residual, weight, eps)
