"""The consumers of the LM-head gradient: ``adamw_step`` (the reference's ``tritium.adamw_step``,
tritium/ops/adamw.py:113-151) and gradient clipping (``helion.clip_grad_norm``, helion/training.py:36-49)
on streaming kernels of the C ABI.

``adamw_step`` keeps the reference's signature, checks and messages. ``clip_grad_norm`` returns the same
pre-clip total norm, but computes it with a deterministic sum of squares and, instead of rescaling every
gradient in place with a host-side ``if`` (which makes the reference synchronise with the device), returns the
coefficient as a device scalar that ``adamw_step(..., grad_scale=...)`` multiplies into the gradient.
"""

from __future__ import annotations

import torch

from . import _lib, grad_norm
from .ops import FLOAT_DTYPES, _DTYPE_CODE, _need_cuda, _need_dtype, _on_device, _stream, _workspace


def _check_adamw_inputs(param, grad, exp_avg, exp_avg_sq) -> None:
    for name, t in (("param", param), ("grad", grad), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
        _need_cuda(name, t)
    _need_dtype("param", param, FLOAT_DTYPES)
    _need_dtype("grad", grad, FLOAT_DTYPES)
    if param.shape != grad.shape:
        raise ValueError(f"Shape mismatch: param has shape {tuple(param.shape)}, grad has shape {tuple(grad.shape)}.")
    if exp_avg.shape != param.shape:
        raise ValueError(f"Shape mismatch: exp_avg has shape {tuple(exp_avg.shape)}, expected {tuple(param.shape)}.")
    if exp_avg_sq.shape != param.shape:
        raise ValueError(
            f"Shape mismatch: exp_avg_sq has shape {tuple(exp_avg_sq.shape)}, expected {tuple(param.shape)}.")
    if grad.dtype != param.dtype:
        raise ValueError(f"Dtype mismatch: grad has dtype {grad.dtype}, param has dtype {param.dtype}.")
    if exp_avg.dtype != torch.float32:
        raise ValueError(f"exp_avg must have dtype float32, got {exp_avg.dtype}.")
    if exp_avg_sq.dtype != torch.float32:
        raise ValueError(f"exp_avg_sq must have dtype float32, got {exp_avg_sq.dtype}.")
    for name, t in (("grad", grad), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
        if t.device != param.device:
            raise ValueError(f"Device mismatch: {name} is on {t.device}, param is on {param.device}.")
    for name, t in (("param", param), ("grad", grad), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous for tritium.adamw_step.")


def adamw_step(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, *,
               lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
               step: int = 1, grad_scale: torch.Tensor | None = None) -> None:
    """Update ``param`` in-place with AdamW using fp32 moments (reference :113-151).

    ``grad_scale`` (extension): a 0-dim float32 device tensor multiplied into the gradient first."""
    _check_adamw_inputs(param, grad, exp_avg, exp_avg_sq)
    n = param.numel()
    if n == 0:
        return
    dev = param.device
    with _on_device(dev):
        _lib.check(
            _lib.lib().lce_adamw_step(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), n,
                                      _DTYPE_CODE[param.dtype], lr, beta1, beta2, eps, weight_decay, int(step),
                                      None if grad_scale is None else grad_scale.data_ptr(), _stream(dev)),
            "lce_adamw_step",
        )


def grad_sumsq(tensors: list[torch.Tensor]) -> torch.Tensor:
    """Sum of squares of all elements of ``tensors`` as a 0-dim float32 device tensor (fixed summation order).
    A gradient whose producing kernel already summed its squares (``grad_norm``: the LM-head gradient of the
    fused loss, when enabled) is not read again; its remembered sum is added instead."""
    dev = tensors[0].device
    L = _lib.lib()
    out = torch.empty((), dtype=torch.float32, device=dev)
    ws = _workspace(L.lce_sumsq_workspace_bytes(), dev)
    known = []
    started = False
    with _on_device(dev):
        for t in tensors:
            if t.dtype not in _DTYPE_CODE or not t.is_contiguous():
                raise ValueError("grad_sumsq needs contiguous float16 / bfloat16 / float32 CUDA tensors.")
            have = grad_norm.lookup(t)
            if have is not None:
                known.append(have)
                continue
            _lib.check(L.lce_sumsq(t.data_ptr(), t.numel(), _DTYPE_CODE[t.dtype], out.data_ptr(), int(started),
                                   ws.data_ptr(), ws.numel(), _stream(dev)), "lce_sumsq")
            started = True
    if not started:
        out.zero_()
    for have in known:  # device scalars, added in list order
        out = out + have
    return out


def clip_grad_norm(params, max_norm: float) -> tuple[torch.Tensor, torch.Tensor]:
    """(pre-clip total norm, clip coefficient), both 0-dim float32 device tensors; nothing is rescaled and the
    host never waits. The coefficient is ``min(1, max_norm / (norm + 1e-6))`` (reference :45-48): pass it to
    ``adamw_step(..., grad_scale=coef)``."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        zero = torch.tensor(0.0)
        return zero, torch.tensor(1.0)
    total_norm = grad_sumsq(grads).sqrt()
    coef = (max_norm / (total_norm + 1e-6)).clamp(max=1.0)
    return total_norm, coef
