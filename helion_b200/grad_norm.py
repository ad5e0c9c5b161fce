"""Sum of squares of a gradient that its producing kernel already added up.

``helion.clip_grad_norm`` (helion/training.py:36-49 of the reference) reads every gradient once more to form
the total norm; for the LM head that is a V x H tensor, 1 GB at the Llama-3 head. The dW GEMM of the fused
loss can add up the squares of the values it stores while it stores them. This module is the hand-over: the
backward ``remember``s the device scalar next to the gradient tensor it belongs to, and
``optim_ops.grad_sumsq`` ``lookup``s a gradient before it launches a reduction over it.

A remembered sum is used only for a tensor that IS that gradient: same storage object (checked through a weak
reference to the storage, which also keeps the storage's identity from being reused while the sum is on
record, without keeping the memory alive), same address, shape and dtype, and not written since
(``Tensor._version``). Autograd hands the gradient of a leaf to ``.grad`` without a copy when it can - holding
the tensor itself here would prevent exactly that; when it accumulates into an existing ``.grad`` instead, the
lookup simply misses. Off by default (one small extra launch per backward); ``enable()`` switches it on for
the process.
"""

from __future__ import annotations

import torch

KEEP = 4
_enabled = False
# (weak storage handle, storage identity, address, shape, dtype, version, sum of squares)
_known: list[tuple[int, int, int, tuple, torch.dtype, int, torch.Tensor]] = []


def _drop(entries) -> None:
    for e in entries:
        torch.UntypedStorage._free_weak_ref(e[0])


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)
    if not on:
        _drop(_known)
        _known.clear()


def enabled() -> bool:
    return _enabled


def remember(grad: torch.Tensor, sumsq: torch.Tensor) -> None:
    storage = grad.untyped_storage()
    keep = [e for e in _known if e[1] != storage._cdata and not torch.UntypedStorage._expired(e[0])][-(KEEP - 1):]
    _drop([e for e in _known if e not in keep])
    _known[:] = keep
    _known.append((storage._weak_ref(), storage._cdata, grad.data_ptr(), tuple(grad.shape), grad.dtype,
                   grad._version, sumsq))


def lookup(grad: torch.Tensor) -> torch.Tensor | None:
    cdata = grad.untyped_storage()._cdata
    for handle, known_cdata, ptr, shape, dtype, version, sumsq in _known:
        if (known_cdata == cdata and not torch.UntypedStorage._expired(handle) and ptr == grad.data_ptr()
                and shape == tuple(grad.shape) and dtype == grad.dtype and grad.is_contiguous()
                and grad._version == version):
            return sumsq
    return None
