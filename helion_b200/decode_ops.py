"""Greedy decoding head: ``argmax_v hidden . weight[v]`` and its log-probability without the logits.

The reference's decode step forms the logits with ``tritium.matmul`` / ``matmul_vec`` on
``lm_head.T.contiguous()`` (examples/common.py:127-131, :380-384: a V x H transpose copy and an N x V
write per step) and picks the token from them. For greedy sampling nothing but the largest logit and the
row's logsumexp is needed, and those are what the forward of the fused linear-cross-entropy already
reduces to per vocabulary tile: this op runs that forward with an argmax epilogue. It takes the LM-head
weight as it is stored (``[V, H]``) and returns ``(token, logprob)`` shaped like ``hidden.shape[:-1]``.
No counterpart in the reference (new entry point; ``install()`` does not rebind anything to it).

With ``process_group`` the weight is this rank's contiguous vocabulary shard (as for the fused loss): every
rank reduces its shard, one all-gather of 16 bytes per row follows, and all ranks merge to the same result.
"""

from __future__ import annotations

import torch

from . import _lib, parallel
from .ops import FLOAT_DTYPES, _DTYPE_CODE, _need_contiguous, _need_cuda, _need_dtype, _on_device, _path_flags, _stream, \
    _workspace


def greedy_head(hidden: torch.Tensor, weight: torch.Tensor, *, vocab_start: int | None = None,
                return_logsumexp: bool = False, process_group=None):
    """``(token, logprob)`` - int64 index of the largest logit of every row (lowest index on ties, offset by
    ``vocab_start``) and float32 ``log_softmax`` at it; with ``return_logsumexp`` also the row's logsumexp.
    ``vocab_start`` defaults to 0, or with a ``process_group`` to the sum of the lower ranks' shard heights."""
    _need_cuda("hidden", hidden)
    _need_cuda("weight", weight)
    _need_dtype("hidden", hidden, FLOAT_DTYPES)
    _need_dtype("weight", weight, FLOAT_DTYPES)
    if hidden.dim() < 1:
        raise ValueError("hidden must have at least 1 dimension shaped (..., hidden_size).")
    if weight.dim() != 2:
        raise ValueError("weight must be a 2D tensor shaped (vocab_size, hidden_size).")
    vocab_size, hidden_size = weight.shape
    if hidden.shape[-1] != hidden_size:
        raise ValueError(f"Shape mismatch: hidden has last dimension {hidden.shape[-1]}, weight expects {hidden_size}.")
    if weight.dtype != hidden.dtype:
        raise ValueError(f"Dtype mismatch: weight has dtype {weight.dtype}, hidden has dtype {hidden.dtype}.")
    if weight.device != hidden.device:
        raise ValueError(f"Device mismatch: weight is on {weight.device}, hidden is on {hidden.device}.")
    if hidden_size <= 0:
        raise ValueError("hidden_size must be positive.")
    if vocab_size <= 0:
        raise ValueError("vocab_size must be positive.")
    _need_contiguous("hidden", hidden)
    _need_contiguous("weight", weight)
    shape = tuple(hidden.shape[:-1])
    n_rows = hidden.numel() // hidden_size
    dev = hidden.device
    rank, world = parallel.group_rank_size(process_group)
    if vocab_start is None:
        vocab_start = parallel.shard_start(process_group, vocab_size, hidden.device)
    token = torch.empty(shape, dtype=torch.int64, device=dev)
    logprob = torch.empty(shape, dtype=torch.float32, device=dev)
    lse = torch.empty(shape, dtype=torch.float32, device=dev) if return_logsumexp or world > 1 else None
    if n_rows:
        L = _lib.lib()
        flags = _path_flags()
        code = _DTYPE_CODE[hidden.dtype]
        ws = _workspace(L.lce_forward_workspace_bytes(n_rows, hidden_size, vocab_size, code, flags), dev)
        with _on_device(dev):
            _lib.check(
                L.lce_greedy_head(hidden.data_ptr(), weight.data_ptr(), n_rows, hidden_size, vocab_size, int(vocab_start),
                                  code, token.data_ptr(), logprob.data_ptr(), lse.data_ptr() if lse is not None else None,
                                  ws.data_ptr(), ws.numel(), flags, _stream(dev)),
                "lce_greedy_head",
            )
    if world > 1:
        merged = parallel.merge_greedy(parallel.gather_stats(parallel.pack_greedy(token, logprob, lse), process_group))
        token, logprob, lse = (t.reshape(shape) for t in merged)
    return (token, logprob, lse) if return_logsumexp else (token, logprob)
