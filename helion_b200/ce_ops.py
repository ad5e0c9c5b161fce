"""Cross-entropy on materialised logits: the reference's ``tritium.cross_entropy`` and
``tritium.cross_entropy_backward`` (tritium/ops/cross_entropy.py:708-713, :792-799) over the C ABI.

Same positional signatures, validation order and messages as the reference (:383-428, :734-775);
``reduction`` and ``ignore_index`` are keyword-only extensions with torch semantics, as for the fused
op. One difference on purpose: the reference refuses vocabularies whose next power of two exceeds
131072 (it keeps a whole row in one Triton program); these kernels chunk the row and accept any size.
"""

from __future__ import annotations

from typing import Any

import torch

from . import _lib
from .ops import (FLOAT_DTYPES, INDEX_DTYPES, _DTYPE_CODE, _check_reduction, _need_cuda, _need_dtype, _on_device,
                  _stream, _workspace)

_OP = "for tritium.cross_entropy"


def check_inputs(logits: torch.Tensor, target: torch.Tensor) -> tuple[int, int]:
    _need_cuda("logits", logits)
    _need_cuda("target", target)
    _need_dtype("logits", logits, FLOAT_DTYPES)
    _need_dtype("target", target, INDEX_DTYPES)
    if logits.dim() != 2:
        raise ValueError("logits must be a 2D tensor shaped (n_rows, vocab_size).")
    if target.dim() != 1:
        raise ValueError("target must be a 1D tensor.")
    n_rows, vocab_size = logits.shape
    if target.shape != (n_rows,):
        raise ValueError(f"Shape mismatch: target has shape {tuple(target.shape)}, expected ({n_rows},).")
    if target.device != logits.device:
        raise ValueError(f"Device mismatch: target is on {target.device}, logits is on {logits.device}.")
    if vocab_size <= 0:
        raise ValueError("vocab_size must be positive.")
    if not logits.is_contiguous():
        raise ValueError(f"logits must be contiguous {_OP}.")
    if not target.is_contiguous():
        raise ValueError(f"target must be contiguous {_OP}.")
    return n_rows, vocab_size


def _forward(logits: torch.Tensor, target: torch.Tensor, reduction: str, ignore_index: int):
    n_rows, vocab_size = check_inputs(logits, target)
    red = _check_reduction(reduction)
    dev = logits.device
    lse = torch.empty((n_rows,), dtype=torch.float32, device=dev)
    if logits.numel() == 0:
        # reference: zero loss when there is nothing to reduce (tritium/ops/cross_entropy.py:540-544)
        return torch.zeros((n_rows,) if red == _lib.REDUCTION_NONE else (), dtype=torch.float32, device=dev), lse
    L = _lib.lib()
    loss = torch.empty((n_rows,) if red == _lib.REDUCTION_NONE else (), dtype=torch.float32, device=dev)
    ws = _workspace(L.lce_ce_workspace_bytes(n_rows, vocab_size, _DTYPE_CODE[logits.dtype]), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_ce_forward(logits.data_ptr(), target.data_ptr(), int(target.dtype == torch.int64), n_rows, vocab_size,
                             _DTYPE_CODE[logits.dtype], ignore_index, red, lse.data_ptr(), loss.data_ptr(), None,
                             ws.data_ptr(), ws.numel(), _stream(dev)),
            "lce_ce_forward",
        )
    return loss, lse


def cross_entropy_backward(grad_out: torch.Tensor, logits: torch.Tensor, target: torch.Tensor,
                           logsumexp: torch.Tensor, *, reduction: str = "mean",
                           ignore_index: int = -100) -> torch.Tensor:
    """``dlogits`` from saved per-row logsumexp values (reference :792-799); ``grad_out`` stays on the device."""
    n_rows, vocab_size = check_inputs(logits, target)
    red = _check_reduction(reduction)
    _need_cuda("grad_out", grad_out)
    _need_cuda("logsumexp", logsumexp)
    grad_shape = (n_rows,) if red == _lib.REDUCTION_NONE else ()
    if tuple(grad_out.shape) != grad_shape:
        raise ValueError(f"Shape mismatch: grad_out has shape {tuple(grad_out.shape)}, expected {grad_shape}.")
    if tuple(logsumexp.shape) != (n_rows,):
        raise ValueError(f"Shape mismatch: logsumexp has shape {tuple(logsumexp.shape)}, expected ({n_rows},).")
    if grad_out.device != logits.device:
        raise ValueError(f"Device mismatch: grad_out is on {grad_out.device}, logits is on {logits.device}.")
    if logsumexp.device != logits.device:
        raise ValueError(f"Device mismatch: logsumexp is on {logsumexp.device}, logits is on {logits.device}.")
    if logsumexp.dtype != torch.float32:
        raise ValueError(f"Dtype mismatch: logsumexp has dtype {logsumexp.dtype}, expected float32.")
    if not logsumexp.is_contiguous():
        raise ValueError(f"logsumexp must be contiguous {_OP}.")
    dlogits = torch.empty_like(logits)
    if logits.numel() == 0:
        return dlogits
    dev = logits.device
    L = _lib.lib()
    go = grad_out if grad_out.dtype == torch.float32 else grad_out.float()
    go = go.contiguous()
    ws = _workspace(L.lce_ce_workspace_bytes(n_rows, vocab_size, _DTYPE_CODE[logits.dtype]), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_ce_backward(logits.data_ptr(), target.data_ptr(), int(target.dtype == torch.int64), logsumexp.data_ptr(),
                              go.data_ptr(), n_rows, vocab_size, _DTYPE_CODE[logits.dtype], ignore_index, red,
                              dlogits.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)),
            "lce_ce_backward",
        )
    return dlogits


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, logits, target, reduction, ignore_index):
        loss, lse = _forward(logits, target, reduction, ignore_index)
        ctx.opts = (reduction, ignore_index)
        ctx.save_for_backward(logits, target, lse)
        return loss

    @staticmethod
    def backward(ctx: Any, *grad_outputs):
        if not ctx.needs_input_grad[0]:
            return None, None, None, None
        logits, target, lse = ctx.saved_tensors
        reduction, ignore_index = ctx.opts
        return cross_entropy_backward(grad_outputs[0], logits, target, lse, reduction=reduction,
                                      ignore_index=ignore_index), None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, *, reduction: str = "mean",
                  ignore_index: int = -100) -> torch.Tensor:
    """Cross-entropy of 2-D ``logits[N, V]`` against ``target[N]`` without a materialised softmax
    (reference :708-713): 0-dim float32 mean by default."""
    if not (torch.is_grad_enabled() and logits.requires_grad):
        loss, _ = _forward(logits, target, reduction, ignore_index)
        return loss
    return _CrossEntropy.apply(logits, target, reduction, ignore_index)
