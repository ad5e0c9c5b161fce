"""Sum of squares of a gradient that its producing kernel already added up.

``helion.clip_grad_norm`` (helion/training.py:36-49 of the reference) reads every gradient once more to form
the total norm; for the LM head that is a V x H tensor, 1 GB at the Llama-3 head. The dW GEMM of the fused
loss can add up the squares of the values it stores while it stores them. This module is the hand-over: the
backward ``remember``s the device scalar next to the gradient tensor it belongs to, and
``optim_ops.grad_sumsq`` ``lookup``s a gradient before it launches a reduction over it.

A remembered sum is used only for the very tensor object it was computed for, and only while that tensor has
not been written since (``Tensor._version``): autograd hands the gradient of a leaf to ``.grad`` without a
copy when it can, otherwise it accumulates into a different tensor and the lookup simply misses. Off by
default (one small extra launch per backward); ``enable()`` switches it on for the process.
"""

from __future__ import annotations

import weakref

import torch

_enabled = False
_known: dict[int, tuple[weakref.ref, int, torch.Tensor]] = {}


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)
    if not on:
        _known.clear()


def enabled() -> bool:
    return _enabled


def remember(grad: torch.Tensor, sumsq: torch.Tensor) -> None:
    key = id(grad)
    _known[key] = (weakref.ref(grad, lambda _ref, key=key: _known.pop(key, None)), grad._version, sumsq)


def lookup(grad: torch.Tensor) -> torch.Tensor | None:
    entry = _known.get(id(grad))
    if entry is None:
        return None
    ref, version, sumsq = entry
    if ref() is grad and grad._version == version:
        return sumsq
    return None
