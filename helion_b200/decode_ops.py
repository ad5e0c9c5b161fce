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


TOPK_MAX = 64


def _check_head_inputs(hidden: torch.Tensor, weight: torch.Tensor) -> tuple[int, int, int]:
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
    if hidden_size <= 0 or vocab_size <= 0:
        raise ValueError("hidden_size and vocab_size must be positive.")
    _need_contiguous("hidden", hidden)
    _need_contiguous("weight", weight)
    return hidden.numel() // hidden_size, hidden_size, vocab_size


def topk_head(hidden: torch.Tensor, weight: torch.Tensor, k: int, *, temperature: float = 1.0,
              vocab_start: int | None = None, process_group=None):
    """``(values, indices, logsumexp)`` of the ``k`` (1..64) largest logits of every row of
    ``hidden @ weight.T / temperature``, without the logits: float32 ``[..., k]`` values (largest first, the
    lower index first among equal values), int64 ``[..., k]`` vocabulary indices and the float32 logsumexp of
    the scaled logits over the whole vocabulary, so that ``exp(values - logsumexp)`` are the tokens' true
    probabilities. Where the vocabulary has fewer than ``k`` entries the tail is ``-inf`` / ``-1``.

    New entry point (``install()`` rebinds nothing to it): the reference's decode step materialises all
    logits and runs ``torch.topk`` / ``torch.sort`` on them (examples/common.py:288-301, 380-396). With a
    ``process_group`` the weight is this rank's vocabulary shard: every rank selects its shard's best ``k``,
    one all-gather of ``k`` pairs per row follows, and all ranks merge to the same result."""
    n_rows, hidden_size, vocab_size = _check_head_inputs(hidden, weight)
    if not 1 <= int(k) <= TOPK_MAX:
        raise ValueError(f"k must be between 1 and {TOPK_MAX}.")
    if not temperature > 0:
        raise ValueError("temperature must be > 0")
    k = int(k)
    shape = tuple(hidden.shape[:-1])
    dev = hidden.device
    rank, world = parallel.group_rank_size(process_group)
    if vocab_start is None:
        vocab_start = parallel.shard_start(process_group, vocab_size, dev)
    values = torch.empty(shape + (k,), dtype=torch.float32, device=dev)
    indices = torch.empty(shape + (k,), dtype=torch.int64, device=dev)
    lse = torch.empty(shape, dtype=torch.float32, device=dev)
    if n_rows:
        L = _lib.lib()
        flags = _path_flags()
        code = _DTYPE_CODE[hidden.dtype]
        ws = _workspace(L.lce_topk_workspace_bytes(n_rows, hidden_size, vocab_size, code, flags), dev)
        with _on_device(dev):
            _lib.check(
                L.lce_topk_head(hidden.data_ptr(), weight.data_ptr(), n_rows, hidden_size, vocab_size, int(vocab_start),
                                code, k, 1.0 / float(temperature), values.data_ptr(), indices.data_ptr(),
                                lse.data_ptr(), ws.data_ptr(), ws.numel(), flags, _stream(dev)),
                "lce_topk_head",
            )
    if world > 1:
        values, indices, lse = merge_topk_shards(values, indices, lse, k, process_group)
    return values, indices, lse


def merge_topk_shards(values: torch.Tensor, indices: torch.Tensor, lse: torch.Tensor, k: int, process_group):
    """Merge every rank's best ``k`` into the best ``k`` of the whole vocabulary (one all-gather). Ties resolve
    to the lower index: shards are contiguous and ascending by rank, each shard's list puts the lower index
    first among equals, and the sort is stable."""
    import torch.distributed as dist

    rank, world = parallel.group_rank_size(process_group)
    shape = tuple(lse.shape)
    n = lse.numel()
    packed = torch.empty((n, 3 * k + 1), dtype=torch.float32, device=values.device)
    packed[:, :k] = values.reshape(n, k)
    packed[:, k:3 * k] = indices.reshape(n, k).view(torch.float32)  # int64 bits as two floats each
    packed[:, 3 * k] = lse.reshape(n)
    everyone = torch.empty((world, n, 3 * k + 1), dtype=torch.float32, device=values.device)
    dist.all_gather_into_tensor(everyone.view(world * n, 3 * k + 1), packed, group=process_group)
    vals = everyone[:, :, :k].permute(1, 0, 2).reshape(n, world * k)
    idx = everyone[:, :, k:3 * k].contiguous().view(torch.int64).permute(1, 0, 2).reshape(n, world * k)
    order = torch.sort(vals, dim=1, descending=True, stable=True).indices[:, :k]
    merged_lse = torch.logsumexp(everyone[:, :, 3 * k], dim=0)
    return (vals.gather(1, order).reshape(shape + (k,)), idx.gather(1, order).reshape(shape + (k,)),
            merged_lse.reshape(shape))


def sample_head(hidden: torch.Tensor, weight: torch.Tensor, *, temperature: float = 0.8, top_k: int = 0,
                top_p: float = 1.0, repetition_penalty: float = 1.0, seen_token_ids=None,
                generator: torch.Generator | None = None, process_group=None, vocab_start: int | None = None,
                max_candidates: int = TOPK_MAX) -> torch.Tensor:
    """One sampled token per row of ``hidden`` (int64, shaped like ``hidden.shape[:-1]``): a multinomial draw
    from ``sampling_distribution`` (same arguments), as the reference's ``sample_next_token`` ends with."""
    idx, probs = sampling_distribution(hidden, weight, temperature=temperature, top_k=top_k, top_p=top_p,
                                       repetition_penalty=repetition_penalty, seen_token_ids=seen_token_ids,
                                       process_group=process_group, vocab_start=vocab_start,
                                       max_candidates=max_candidates)
    flat = probs.reshape(-1, probs.shape[-1])
    choice = torch.multinomial(flat, num_samples=1, generator=generator)
    return idx.reshape(-1, idx.shape[-1]).gather(1, choice).reshape(tuple(hidden.shape[:-1]))


def sampling_distribution(hidden: torch.Tensor, weight: torch.Tensor, *, temperature: float = 0.8, top_k: int = 0,
                          top_p: float = 1.0, repetition_penalty: float = 1.0, seen_token_ids=None,
                          process_group=None, vocab_start: int | None = None,
                          max_candidates: int = TOPK_MAX) -> tuple[torch.Tensor, torch.Tensor]:
    """``(indices, probs)``, each ``[..., m]``: the tokens that can be drawn for every row and their probabilities
    (0 for masked ones; ``-1`` indices only carry probability 0) under the reference's
    sampling rule - repetition penalty, temperature, top-k, nucleus (top-p), multinomial draw
    (``sample_next_token``, examples/common.py:263-306) - computed from at most ``max_candidates`` (<= 64)
    candidates per row that ``topk_head`` selects, instead of from ``V`` materialised logits.

    What makes that exact: with ``top_k`` in 1..64 only the ``top_k`` best survive the reference's mask, so
    the draw needs nothing else; their order can only change through the repetition penalty, which for a
    penalty >= 1 only lowers seen tokens, so fetching ``top_k + len(seen)`` candidates covers every token
    that can enter. Nucleus sampling keeps the shortest prefix of the sorted tokens whose probability
    exceeds ``top_p``; without top-k the probabilities come from the full-vocabulary logsumexp the head
    returns, so the prefix is exact whenever it fits in the fetched candidates.
    Raises ``ValueError`` where the rule cannot be evaluated from the candidates: ``top_k == 0`` with
    ``top_p == 1`` (a draw from the whole vocabulary), a penalty < 1, a penalty together with
    ``top_k == 0`` (the normaliser would need every seen token's logit), more candidates needed than
    ``max_candidates``, or a nucleus that does not fit - callers then use the logits path.
    ``seen_token_ids`` is one list of ids for all rows (the reference decodes one sequence)."""
    if temperature <= 0:
        raise ValueError("temperature must be > 0")
    if top_k < 0:
        raise ValueError("top_k must be >= 0")
    if not 0.0 < top_p <= 1.0:
        raise ValueError("top_p must satisfy 0 < top_p <= 1")
    if repetition_penalty <= 0:
        raise ValueError("repetition_penalty must be > 0")
    if repetition_penalty < 1.0:
        raise ValueError("sample_head needs repetition_penalty >= 1 (a boost can lift any token into the top k)")
    if top_k == 0 and top_p >= 1.0:
        raise ValueError("sample_head needs top_k > 0 or top_p < 1: a draw from the whole vocabulary needs all logits")
    seen = sorted(set(int(i) for i in (seen_token_ids or []))) if repetition_penalty != 1.0 else []
    if seen and top_k == 0:
        raise ValueError("sample_head applies a repetition penalty only together with top_k > 0")
    vocab_total = weight.shape[0] if process_group is None else None
    fetch = max_candidates if top_k == 0 else top_k + len(seen)
    if vocab_total is not None:
        fetch = min(fetch, vocab_total)
    if fetch > min(max_candidates, TOPK_MAX):
        raise ValueError(f"sampling needs {fetch} candidates per row, more than max_candidates={max_candidates}")
    values, indices, lse = topk_head(hidden, weight, fetch, temperature=temperature, process_group=process_group,
                                     vocab_start=vocab_start)
    shape = tuple(lse.shape)
    vals = values.reshape(-1, fetch).clone()
    idx = indices.reshape(-1, fetch)
    lse = lse.reshape(-1).clone()
    if seen:
        # the penalty acts on the unscaled logit: z / p for z >= 0, z * p for z < 0; values hold y = z / T
        seen_t = torch.tensor(seen, device=vals.device)
        hit = (idx[:, :, None] == seen_t[None, None, :]).any(dim=-1) & (idx >= 0)
        penalised = torch.where(vals < 0, vals * repetition_penalty, vals / repetition_penalty)
        vals = torch.where(hit, penalised, vals)
        order = torch.sort(vals, dim=1, descending=True, stable=True).indices
        vals, idx = vals.gather(1, order), idx.gather(1, order)
    if top_k > 0:
        keep = min(top_k, fetch)
        vals, idx = vals[:, :keep], idx[:, :keep]
    vals = vals.masked_fill(idx < 0, float("-inf"))
    if top_p < 1.0:
        # the reference renormalises over what survived top-k before it accumulates probabilities
        norm = torch.logsumexp(vals, dim=1) if top_k > 0 else lse
        probs = torch.exp(vals - norm[:, None])
        cumulative = probs.cumsum(dim=1)
        if top_k == 0 and bool((cumulative[:, -1] <= top_p).any()):
            raise ValueError("the nucleus does not fit in the fetched candidates; use the logits path")
        remove = cumulative > top_p
        remove[:, 1:] = remove[:, :-1].clone()
        remove[:, 0] = False
        vals = vals.masked_fill(remove, float("-inf"))
    probs = torch.softmax(vals, dim=1)
    return idx.reshape(shape + (idx.shape[1],)), probs.reshape(shape + (probs.shape[1],))
