"""Host side of the fused linear-cross-entropy op: the reference's Python interface over the C ABI.

Mirrors ``tritium/ops/cross_entropy.py`` of the reference for this one path:

* ``linear_cross_entropy(hidden, weight, target)``            (reference :716-725)
* ``linear_cross_entropy_backward(grad_out, hidden, weight, target, logsumexp)``   (:863-959)
* the autograd wrapper                                         (:663-705)
* input validation with the same checks, order and messages   (:431-494, :871-907,
  ``tritium/ops/_utils.py:25-46``)

The positional signatures are the reference's. ``reduction``, ``ignore_index`` and
``process_group`` are keyword-only extensions: the reference always takes the mean over all rows
and has no ignored label, which is what the defaults give when no target equals ``-100``.
All GPU work happens in libhelion_lce.so; nothing here computes on the CPU or through torch ops.
"""

from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from . import _lib, grad_norm, parallel

FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
INDEX_DTYPES = (torch.int32, torch.int64)
_DTYPE_CODE = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16, torch.float32: _lib.DTYPE_F32}

_OP = "for tritium.linear_cross_entropy"


# ----------------------------------------------------------------------------------------------
# validation (same order and wording as the reference so its tests match on substrings)
# ----------------------------------------------------------------------------------------------
def _dtype_names(dtypes) -> str:
    return ", ".join(str(d).replace("torch.", "") for d in dtypes)


def _need_cuda(name: str, t: torch.Tensor) -> None:
    if t.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor.")


def _need_dtype(name: str, t: torch.Tensor, allowed) -> None:
    if t.dtype not in allowed:
        raise ValueError(f"{name} must have one of these dtypes: {_dtype_names(allowed)}.")


def _need_contiguous(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous {_OP}.")


def check_inputs(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor) -> tuple[int, int, int]:
    """Validate (hidden, weight, target); returns (n_rows, hidden_size, vocab_size)."""
    _need_cuda("hidden", hidden)
    _need_cuda("weight", weight)
    _need_cuda("target", target)
    _need_dtype("hidden", hidden, FLOAT_DTYPES)
    _need_dtype("weight", weight, FLOAT_DTYPES)
    _need_dtype("target", target, INDEX_DTYPES)
    if hidden.dim() < 2:
        raise ValueError("hidden must have at least 2 dimensions shaped (..., hidden_size).")
    if weight.dim() != 2:
        raise ValueError("weight must be a 2D tensor shaped (vocab_size, hidden_size).")
    vocab_size, hidden_size = weight.shape
    if hidden.shape[-1] != hidden_size:
        raise ValueError(
            f"Shape mismatch: hidden has last dimension {hidden.shape[-1]}, weight expects {hidden_size}."
        )
    if target.shape != hidden.shape[:-1]:
        raise ValueError(
            f"Shape mismatch: target has shape {tuple(target.shape)}, expected {tuple(hidden.shape[:-1])}."
        )
    if weight.dtype != hidden.dtype:
        raise ValueError(f"Dtype mismatch: weight has dtype {weight.dtype}, hidden has dtype {hidden.dtype}.")
    if weight.device != hidden.device:
        raise ValueError(f"Device mismatch: weight is on {weight.device}, hidden is on {hidden.device}.")
    if target.device != hidden.device:
        raise ValueError(f"Device mismatch: target is on {target.device}, hidden is on {hidden.device}.")
    if hidden_size <= 0:
        raise ValueError("hidden_size must be positive.")
    if vocab_size <= 0:
        raise ValueError("vocab_size must be positive.")
    _need_contiguous("hidden", hidden)
    _need_contiguous("weight", weight)
    _need_contiguous("target", target)
    return target.numel(), hidden_size, vocab_size


def check_backward_inputs(grad_out: torch.Tensor, hidden: torch.Tensor, logsumexp: torch.Tensor, n_rows: int,
                          grad_shape: tuple[int, ...]) -> None:
    _need_cuda("grad_out", grad_out)
    _need_cuda("logsumexp", logsumexp)
    if tuple(grad_out.shape) != grad_shape:
        raise ValueError(
            f"Shape mismatch: grad_out has shape {tuple(grad_out.shape)}, expected {grad_shape}."
        )
    if tuple(logsumexp.shape) != (n_rows,):
        raise ValueError(
            f"Shape mismatch: logsumexp has shape {tuple(logsumexp.shape)}, expected ({n_rows},)."
        )
    if grad_out.device != hidden.device:
        raise ValueError(f"Device mismatch: grad_out is on {grad_out.device}, hidden is on {hidden.device}.")
    if logsumexp.device != hidden.device:
        raise ValueError(f"Device mismatch: logsumexp is on {logsumexp.device}, hidden is on {hidden.device}.")
    if logsumexp.dtype != torch.float32:
        raise ValueError(f"Dtype mismatch: logsumexp has dtype {logsumexp.dtype}, expected float32.")
    if not logsumexp.is_contiguous():
        raise ValueError(f"logsumexp must be contiguous {_OP}.")


def _check_reduction(reduction: str) -> int:
    if reduction not in _lib.REDUCTIONS:
        raise ValueError(f"reduction must be one of 'none', 'mean', 'sum'; got {reduction!r}.")
    return _lib.REDUCTIONS[reduction]


# ----------------------------------------------------------------------------------------------
# knobs (debug / tests)
# ----------------------------------------------------------------------------------------------
def _path_flags() -> int:
    force = os.environ.get("HELION_B200_FORCE", "")
    if force == "simt":
        return _lib.FLAG_FORCE_SIMT
    if force == "tc":
        return _lib.FLAG_FORCE_TC
    if force == "tc1":  # tensor-core path on single CTAs (cta_group::1) instead of CTA pairs
        return _lib.FLAG_FORCE_TC | _lib.FLAG_ONE_CTA
    return 0


def _block_bytes() -> int:
    return int(os.environ.get("HELION_B200_BLOCK_BYTES", "0"))


def _stream(device: torch.device) -> int:
    """Raw handle of torch's current stream on ``device`` (the stream every launch is enqueued on)."""
    try:
        return torch._C._cuda_getCurrentRawStream(device.index if device.index is not None else
                                                  torch.cuda.current_device())
    except AttributeError:  # older / newer torch without the private fast path
        return torch.cuda.current_stream(device).cuda_stream


class _on_device:
    """Makes ``device`` current for the duration of a C-ABI call, at no cost when it already is."""

    __slots__ = ("guard",)

    def __init__(self, device: torch.device):
        self.guard = None
        if device.index is not None and device.index != torch.cuda.current_device():
            self.guard = torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_WS_CACHE_MAX = 32 << 20
_ws_cache: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Scratch for one C-ABI call. Small requests (latency-bound problems, where an allocation is a visible
    share of the call) reuse one buffer per (device, stream): calls on one stream run in order, so they may
    share scratch; calls on different streams get different buffers. Large requests are allocated per call and
    go back to torch's caching allocator afterwards."""
    nbytes = max(int(nbytes), 256)
    if nbytes > _WS_CACHE_MAX:
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        if len(_ws_cache) >= 64:  # streams come and go: do not let the cache grow without bound
            _ws_cache.clear()
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _resolve_vocab_start(vocab_start: int | None, process_group: Any, v_local: int, device: torch.device) -> int:
    """Where this rank's shard begins: what the caller says, else the sum of the lower ranks' shard heights
    (``rank * v_local`` for equal shards; uneven shards, as ``parallel.shard_weight`` cuts them, differ)."""
    if vocab_start is not None:
        return int(vocab_start)
    return parallel.shard_start(process_group, v_local, device)


# ----------------------------------------------------------------------------------------------
# forward
# ----------------------------------------------------------------------------------------------
def local_stats(hidden2d: torch.Tensor, weight: torch.Tensor, target1d: torch.Tensor, vocab_start: int,
                flags: int = 0) -> torch.Tensor:
    """Per-row (max, sum-exp, target-logit) of the local vocabulary shard, float32 ``[3, N]``."""
    n_rows, hidden_size = hidden2d.shape
    v_local = weight.shape[0]
    dev = hidden2d.device
    L = _lib.lib()
    stats = torch.empty((3, n_rows), dtype=torch.float32, device=dev)
    dtype = _DTYPE_CODE[hidden2d.dtype]
    ws = _workspace(L.lce_forward_workspace_bytes(n_rows, hidden_size, v_local, dtype, flags), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_forward_stats(hidden2d.data_ptr(), weight.data_ptr(), target1d.data_ptr(),
                                int(target1d.dtype == torch.int64), n_rows, hidden_size, v_local, vocab_start,
                                dtype, stats.data_ptr(), ws.data_ptr(), ws.numel(), flags, _stream(dev)),
            "lce_forward_stats",
        )
    return stats


def finalize(stats: torch.Tensor, target1d: torch.Tensor, reduction: str, ignore_index: int,
             want_count: bool = False) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """Merge ``[R, 3, N]`` shard statistics into (loss, logsumexp[N], valid_count or None)."""
    red = _check_reduction(reduction)
    n_shards, _, n_rows = stats.shape
    dev = stats.device
    L = _lib.lib()
    lse = torch.empty((n_rows,), dtype=torch.float32, device=dev)
    loss = torch.empty((n_rows,) if red == _lib.REDUCTION_NONE else (), dtype=torch.float32, device=dev)
    count = torch.empty((), dtype=torch.float32, device=dev) if want_count else None
    ws = _workspace(L.lce_finalize_workspace_bytes(n_rows), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_finalize(stats.data_ptr(), n_shards, target1d.data_ptr(), int(target1d.dtype == torch.int64),
                           n_rows, ignore_index, red, lse.data_ptr(), loss.data_ptr(), _ptr(count),
                           ws.data_ptr(), ws.numel(), _stream(dev)),
            "lce_finalize",
        )
    return loss, lse, count


def _forward_single(hidden2d: torch.Tensor, weight: torch.Tensor, target1d: torch.Tensor, target_shape,
                    red: int, ignore_index: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Unsharded forward in one C-ABI call (GEMM + statistics, fused merge/finalize, loss reduction)."""
    n_rows, hidden_size = hidden2d.shape
    v = weight.shape[0]
    dev = hidden2d.device
    L = _lib.lib()
    dtype = _DTYPE_CODE[hidden2d.dtype]
    flags = _path_flags()
    lse = torch.empty((n_rows,), dtype=torch.float32, device=dev)
    loss = torch.empty(tuple(target_shape) if red == _lib.REDUCTION_NONE else (), dtype=torch.float32, device=dev)
    ws = _workspace(L.lce_forward_loss_workspace_bytes(n_rows, hidden_size, v, dtype, flags), dev)
    with _on_device(dev):
        _lib.check(
            L.lce_forward_loss(hidden2d.data_ptr(), weight.data_ptr(), target1d.data_ptr(),
                               int(target1d.dtype == torch.int64), n_rows, hidden_size, v, dtype, ignore_index, red,
                               lse.data_ptr(), loss.data_ptr(), None, ws.data_ptr(), ws.numel(), flags, _stream(dev)),
            "lce_forward_loss",
        )
    return loss, lse


def _forward(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, reduction: str,
             ignore_index: int, process_group: Any, vocab_start: int | None) -> tuple[torch.Tensor, torch.Tensor]:
    n_rows, hidden_size, v_local = check_inputs(hidden, weight, target)
    red = _check_reduction(reduction)
    dev = hidden.device
    if n_rows == 0:
        # reference: zero loss and an empty logsumexp (tritium/ops/cross_entropy.py:576-581)
        shape = tuple(target.shape) if red == _lib.REDUCTION_NONE else ()
        return (torch.zeros(shape, dtype=torch.float32, device=dev),
                torch.empty((0,), dtype=torch.float32, device=dev))
    rank, world = parallel.group_rank_size(process_group)
    hidden2d = hidden.view(n_rows, hidden_size)
    target1d = target.view(n_rows)
    if world == 1 and vocab_start in (None, 0):
        return _forward_single(hidden2d, weight, target1d, target.shape, red, ignore_index)
    stats = local_stats(hidden2d, weight, target1d, _resolve_vocab_start(vocab_start, process_group, v_local, dev),
                        _path_flags())
    loss, lse, _ = finalize(parallel.gather_stats(stats, process_group), target1d, reduction, ignore_index)
    if red == _lib.REDUCTION_NONE:
        loss = loss.view(target.shape)
    return loss, lse


# ----------------------------------------------------------------------------------------------
# backward
# ----------------------------------------------------------------------------------------------
def _backward(grad_out: torch.Tensor, hidden2d: torch.Tensor, weight: torch.Tensor, target1d: torch.Tensor,
              logsumexp: torch.Tensor, reduction: str, ignore_index: int, process_group: Any,
              vocab_start: int | None, need_dx: bool, need_dw: bool,
              reduce_dx: bool = True) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    red = _check_reduction(reduction)
    n_rows, hidden_size = hidden2d.shape
    v_local = weight.shape[0]
    dev = hidden2d.device
    rank, world = parallel.group_rank_size(process_group)
    sharded = world > 1 and reduce_dx
    L = _lib.lib()

    flags = _path_flags()
    if not need_dx:
        flags |= _lib.FLAG_NO_DX
    if not need_dw:
        flags |= _lib.FLAG_NO_DW
    if sharded and need_dx:
        flags |= _lib.FLAG_DX_F32  # partial sums leave in fp32 and are rounded once, after the reduce

    if n_rows == 0:
        # reference: empty dX and an all-zero dW (tritium/ops/cross_entropy.py:911-913)
        return (torch.empty_like(hidden2d) if need_dx else None,
                torch.zeros_like(weight) if need_dw else None)
    dw = torch.empty_like(weight) if need_dw else None

    if grad_out.dtype != torch.float32:
        grad_out = grad_out.float()
    grad_out = grad_out.contiguous()
    dtype = _DTYPE_CODE[hidden2d.dtype]
    block = _block_bytes()
    vstart = _resolve_vocab_start(vocab_start, process_group, v_local, dev)
    ws = _workspace(L.lce_backward_workspace_bytes(n_rows, hidden_size, v_local, dtype, flags, block), dev)

    # Sharded: two ways to sum the partial dX over the group.
    #  "p2p" (default): the dX GEMM's epilogue stores finished rows straight into the owning rank's staging
    #        buffer over NVLink (reduce-scatter inside the GEMM); a small kernel then sums and all-gathers.
    #        Falls back to "nccl" for the whole group if peer-mapped memory cannot be set up.
    #  "nccl": fp32 partial dX per row chunk, all-reduced on a side stream as soon as the library signals
    #        the chunk final, while the remaining dW GEMMs run on the main stream.
    events, event_array, chunk_rows, scatter, peers, staging_index = None, None, n_rows, None, None, 0
    if sharded and need_dx:
        plan = (ctypes.c_int64 * 4)()
        _lib.check(L.lce_backward_plan(n_rows, hidden_size, v_local, dtype, flags, block, hidden2d.data_ptr(),
                                       weight.data_ptr(), plan), "lce_backward_plan")
        chunk_rows, n_chunks = int(plan[0]), int(plan[2])
        events = parallel.ready_events(dev, n_chunks)
        event_array = (ctypes.c_void_p * n_chunks)(*[e.cuda_event for e in events])
        if _dx_reduce_mode() == "p2p" and hidden_size % 4 == 0 and world <= 8:
            peers = parallel.peer_buffers(process_group, n_rows, hidden_size, dev)
        if peers is not None:
            staging_index = peers.next_buffer()
            scatter = _lib.PeerScatter()
            for k, ptr in enumerate(peers.staging_ptrs[staging_index]):
                scatter.staging[k] = ptr
            scatter.rank, scatter.world = rank, world
        elif not parallel.ranks_agree(process_group, ("dx-chunks", n_rows, hidden_size, dtype, flags, block),
                                      (chunk_rows, n_chunks), dev):
            # each rank plans its row chunks from its own shard height; if the plans differ (uneven shards
            # at a plan boundary) chunk-wise collectives would not match up: reduce dX in one piece instead
            events, chunk_rows = events[-1:], n_rows
    dx = None
    if need_dx and peers is None:  # with peer buffers nothing is written locally: rows leave through the epilogue
        dx = torch.empty((n_rows, hidden_size), dtype=torch.float32 if sharded else hidden2d.dtype, device=dev)

    # the head's share of the gradient norm, summed up by the dW epilogue while it stores (no second read of dW)
    dw_sumsq = torch.empty((), dtype=torch.float32, device=dev) if (dw is not None and grad_norm.enabled()) else None
    with _on_device(dev):
        _lib.check(
            L.lce_backward(hidden2d.data_ptr(), weight.data_ptr(), target1d.data_ptr(),
                           int(target1d.dtype == torch.int64), logsumexp.data_ptr(), grad_out.data_ptr(), n_rows,
                           hidden_size, v_local, vstart, dtype, ignore_index, red, _ptr(dx), _ptr(dw), ws.data_ptr(),
                           ws.numel(), flags, block, event_array, ctypes.byref(scatter) if scatter is not None else None,
                           _ptr(dw_sumsq), _stream(dev)),
            "lce_backward",
        )
    if dw_sumsq is not None:
        grad_norm.remember(dw, dw_sumsq)
    if peers is not None:
        dx = _finish_peer_reduce(peers, staging_index, events, n_rows, hidden_size, hidden2d.dtype, dev)
    elif sharded and dx is not None:
        dx = parallel.reduce_dx_chunks(dx, chunk_rows, events, hidden2d.dtype, process_group)
    return dx, dw


def _dx_reduce_mode() -> str:
    return os.environ.get("HELION_B200_DX_REDUCE", "p2p")


def _finish_peer_reduce(peers, staging_index: int, events, n_rows: int, hidden_size: int, dtype: torch.dtype,
                        dev: torch.device) -> torch.Tensor:
    """Second half of the fused dX reduction, on the side stream so that it overlaps the remaining dW GEMMs:
    once this rank's last dX rows have left (event), one 4-byte all-reduce orders the ranks (every rank's
    partial rows have landed in their owners' staging buffers), this rank sums the slots of its own row
    slice, and an all-gather of the rounded slices gives every rank the whole dX."""
    import torch.distributed as dist

    L = _lib.lib()
    main = torch.cuda.current_stream(dev)
    side = parallel.comm_stream(dev)
    side.wait_event(events[-1])
    rpr = -(-n_rows // peers.world)
    with torch.cuda.stream(side):
        peers.order_ranks()
        piece = torch.empty((rpr, hidden_size), dtype=dtype, device=dev)
        gathered = torch.empty((peers.world * rpr, hidden_size), dtype=dtype, device=dev)
        _lib.check(L.lce_dx_reduce_slice(peers.staging[staging_index].data_ptr(), peers.world, peers.rank, n_rows,
                                         hidden_size, _DTYPE_CODE[dtype], piece.data_ptr(), side.cuda_stream),
                   "lce_dx_reduce_slice")
        dist.all_gather_into_tensor(gathered, piece, group=peers.group)
    main.wait_stream(side)
    piece.record_stream(main)
    gathered.record_stream(main)
    return gathered[:n_rows]


def linear_cross_entropy_backward(
    grad_out: torch.Tensor,
    hidden: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    logsumexp: torch.Tensor,
    *,
    reduction: str = "mean",
    ignore_index: int = -100,
    process_group: Any = None,
    vocab_start: int | None = None,
    reduce_dx: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Gradients of ``linear_cross_entropy`` from a saved logsumexp: ``(dhidden[N,H], dweight[V,H])``.

    Same positional contract as the reference (tritium/ops/cross_entropy.py:863-869): ``grad_out`` is a
    0-dim device tensor (shape of ``target`` for ``reduction="none"``) and is read on the device.
    With a ``process_group``, ``weight`` is this rank's vocabulary shard, ``logsumexp`` is global,
    ``dweight`` is local and ``dhidden`` is summed over the group unless ``reduce_dx=False``.
    """
    n_rows, hidden_size, _ = check_inputs(hidden, weight, target)
    red = _check_reduction(reduction)
    grad_shape = tuple(target.shape) if red == _lib.REDUCTION_NONE else ()
    check_backward_inputs(grad_out, hidden, logsumexp, n_rows, grad_shape)
    dx, dw = _backward(grad_out.reshape(-1) if grad_shape else grad_out, hidden.view(n_rows, hidden_size), weight,
                       target.view(n_rows), logsumexp, reduction, ignore_index, process_group, vocab_start,
                       True, True, reduce_dx)
    return dx, dw


class _LinearCrossEntropy(torch.autograd.Function):
    """Autograd node; saves views of the inputs plus logsumexp[N], never the logits (reference :663-705)."""

    @staticmethod
    def forward(ctx: Any, hidden, weight, target, reduction, ignore_index, process_group, vocab_start):
        loss, lse = _forward(hidden, weight, target, reduction, ignore_index, process_group, vocab_start)
        n_rows = target.numel()
        ctx.hidden_shape = tuple(hidden.shape)
        ctx.opts = (reduction, ignore_index, process_group, vocab_start)
        ctx.save_for_backward(hidden.view(n_rows, hidden.shape[-1]), weight, target.view(n_rows), lse)
        return loss

    @staticmethod
    def backward(ctx: Any, *grad_outputs):
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not need_dx and not need_dw:
            return (None,) * 7
        hidden2d, weight, target1d, lse = ctx.saved_tensors
        reduction, ignore_index, process_group, vocab_start = ctx.opts
        grad = grad_outputs[0]
        if reduction == "none":
            grad = grad.reshape(-1)
        dx, dw = _backward(grad, hidden2d, weight, target1d, lse, reduction, ignore_index, process_group,
                           vocab_start, need_dx, need_dw)
        if dx is not None:
            dx = dx.view(ctx.hidden_shape)
        return dx, dw, None, None, None, None, None


def linear_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    *,
    reduction: str = "mean",
    ignore_index: int = -100,
    process_group: Any = None,
    vocab_start: int | None = None,
) -> torch.Tensor:
    """Cross-entropy of ``hidden @ weight.T`` against ``target`` without materialising the logits.

    ``hidden[..., H]`` and ``weight[V, H]`` are contiguous CUDA tensors of one float dtype, ``target`` has
    shape ``hidden.shape[:-1]`` (int32 / int64). Returns a 0-dim float32 loss (``target``-shaped for
    ``reduction="none"``). Called with three positional arguments it behaves as the reference op
    (tritium/ops/cross_entropy.py:716-725): the mean over all rows. With a ``process_group`` the weight is
    this rank's contiguous vocabulary shard (rows ``vocab_start ..``, default ``rank * V_local``) and every
    rank returns the same loss.
    """
    if not (torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad)):
        loss, _ = _forward(hidden, weight, target, reduction, ignore_index, process_group, vocab_start)
        return loss
    return _LinearCrossEntropy.apply(hidden, weight, target, reduction, ignore_index, process_group, vocab_start)


def debug_gemm(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool, b_mn_major: bool,
               one_cta: bool = False) -> torch.Tensor:
    """``A @ B.T`` in float32 on the tcgen05 GEMM core (test hook for the operand layouts)."""
    m, k = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    n = b.shape[1] if b_mn_major else b.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    with _on_device(a.device):
        _lib.check(
            _lib.lib().lce_debug_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, int(a_mn_major),
                                      int(b_mn_major), _DTYPE_CODE[a.dtype],
                                      _lib.FLAG_ONE_CTA if one_cta else 0, _stream(a.device)),
            "lce_debug_gemm",
        )
    return out
