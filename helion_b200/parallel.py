"""Vocabulary-parallel plumbing: one process per GPU, weight rows sharded contiguously by vocabulary.

The reference is single-GPU (it has no torch.distributed code at all), so this layer has no reference
counterpart; its contract is "the same numbers as one GPU". Forward: every rank computes softmax
statistics (max, sum-exp, target logit) of its shard, ONE collective exchanges those 3 floats per row,
and every rank merges them in rank order, so all ranks hold bit-identical losses. Backward: dW is local;
the partial dX = G_r @ W_r of each rank is summed over the group in fp32 and rounded once.

The functions below touch no kernels and work on any backend (NCCL on GPUs, gloo on CPU tensors in
tests); ops.py calls them between the kernel launches.
"""

from __future__ import annotations

from typing import Any

import torch


def group_rank_size(process_group: Any) -> tuple[int, int]:
    if process_group is None:
        return 0, 1
    import torch.distributed as dist

    return dist.get_rank(process_group), dist.get_world_size(process_group)


def shard_bounds(vocab_size: int, world_size: int, rank: int) -> tuple[int, int]:
    """Rows ``[start, end)`` of the full weight that ``rank`` owns: equal contiguous shards, the last
    ranks one row shorter when the vocabulary does not divide evenly."""
    base, extra = divmod(vocab_size, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_weight(weight: torch.Tensor, process_group: Any) -> tuple[torch.Tensor, int]:
    """This rank's contiguous slice of a full ``[V, H]`` weight and its first global row."""
    rank, world = group_rank_size(process_group)
    start, end = shard_bounds(weight.shape[0], world, rank)
    return weight[start:end].contiguous(), start


def gather_stats(stats: torch.Tensor, process_group: Any) -> torch.Tensor:
    """``[3, N]`` local statistics -> ``[R, 3, N]`` ordered by rank (one all-gather of 12 bytes per row)."""
    rank, world = group_rank_size(process_group)
    if world == 1:
        return stats.unsqueeze(0)
    import torch.distributed as dist

    out = torch.empty((world,) + tuple(stats.shape), dtype=stats.dtype, device=stats.device)
    # the output is the concatenation of the inputs along dim 0: [R*3, N] viewed as [R, 3, N]
    dist.all_gather_into_tensor(out.view((world * stats.shape[0],) + tuple(stats.shape[1:])), stats.contiguous(),
                                group=process_group)
    return out


def pack_greedy(token: torch.Tensor, logprob: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
    """One shard's greedy result as ``[4, N]`` float32: (largest logit, logsumexp, the int64 token's two
    32-bit halves) - a single buffer, so that one all-gather carries everything."""
    n = token.numel()
    buf = torch.empty((4, n), dtype=torch.float32, device=token.device)
    buf[0] = logprob.reshape(-1) + lse.reshape(-1)
    buf[1] = lse.reshape(-1)
    buf[2:4].reshape(-1).view(torch.int64).copy_(token.reshape(-1))
    return buf


def merge_greedy(gathered: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[R, 4, N]`` packed shard results (rank order) -> (token, logprob, logsumexp) of the whole vocabulary.
    The row's logsumexp is the logsumexp of the shards'; the token comes from the shard with the largest
    logit, the lowest rank - i.e. the lowest index for contiguous ascending shards - on ties."""
    world, _, n = gathered.shape
    tops, lses = gathered[:, 0], gathered[:, 1]
    tokens = gathered[:, 2:4].reshape(world, 2 * n).contiguous().view(torch.int64)
    lse = torch.logsumexp(lses, dim=0)
    best = tops.argmax(dim=0, keepdim=True)
    return tokens.gather(0, best)[0], tops.gather(0, best)[0] - lse, lse


def reduce_dx(dx_partial: torch.Tensor, out_dtype: torch.dtype, process_group: Any) -> torch.Tensor:
    """Sum the fp32 partial ``dX`` of all ranks and round to ``out_dtype`` once."""
    rank, world = group_rank_size(process_group)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(dx_partial, op=dist.ReduceOp.SUM, group=process_group)
    return dx_partial if dx_partial.dtype == out_dtype else dx_partial.to(out_dtype)


# ---- overlap of the dX reduction with the rest of the backward pass ---------------------------------
_comm_streams: dict[int, "torch.cuda.Stream"] = {}
_event_pool: dict[int, list["torch.cuda.Event"]] = {}


def comm_stream(device: torch.device) -> "torch.cuda.Stream":
    """The side stream (one per device) on which partial dX is reduced."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _comm_streams:
        _comm_streams[idx] = torch.cuda.Stream(device=device)
    return _comm_streams[idx]


def ready_events(device: torch.device, count: int) -> list["torch.cuda.Event"]:
    """``count`` reusable CUDA events whose raw handles the C ABI may record.

    torch creates an event lazily on its first ``record``; each event is recorded once here so that
    ``cuda_event`` is a real handle before it crosses the C ABI."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    pool = _event_pool.setdefault(idx, [])
    while len(pool) < count:
        ev = torch.cuda.Event(enable_timing=False)
        ev.record(torch.cuda.current_stream(device))
        pool.append(ev)
    return pool[:count]


def reduce_dx_chunks(dx_partial: torch.Tensor, chunk_rows: int, events, out_dtype: torch.dtype,
                     process_group: Any) -> torch.Tensor:
    """All-reduce ``dx_partial`` row chunk by row chunk on the side stream, each chunk as soon as its
    event fires; the calling stream then waits for the side stream and rounds once to ``out_dtype``."""
    import torch.distributed as dist

    dev = dx_partial.device
    main = torch.cuda.current_stream(dev)
    side = comm_stream(dev)
    for i, ev in enumerate(events):
        side.wait_event(ev)
        with torch.cuda.stream(side):
            dist.all_reduce(dx_partial[i * chunk_rows:(i + 1) * chunk_rows], op=dist.ReduceOp.SUM,
                            group=process_group)
    main.wait_stream(side)
    return dx_partial if dx_partial.dtype == out_dtype else dx_partial.to(out_dtype)


# ---- dX reduce-scatter fused into the GEMM epilogue (peer stores over NVLink) ----------------------
class PeerBuffers:
    """Symmetric (peer-mapped) buffers of one (group, N, H, dtype) problem, allocated once and reused:

    * ``staging``  [world, rows_per_rank, H] fp32 on every rank: rank r's dX epilogue stores the partial
      rows owned by rank o into slot r of rank o's staging buffer;
    * ``final``    [N, H] in the op dtype on every rank: the owner of a row slice sums its ``world`` slots
      and stores the rounded result into every rank's ``final``.

    Two tiny all-reduces order the ranks (everyone has scattered before anyone sums; everyone has
    gathered before the buffers are reused). No kernel of this package waits on another GPU.
    """

    def __init__(self, process_group: Any, n_rows: int, hidden: int, dtype: torch.dtype, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world = group_rank_size(process_group)
        self.group = process_group
        self.rows_per_rank = -(-n_rows // self.world)
        self.staging = symm_mem.empty((self.world, self.rows_per_rank, hidden), dtype=torch.float32, device=device)
        self.final = symm_mem.empty((n_rows, hidden), dtype=dtype, device=device)
        self._staging_handle = symm_mem.rendezvous(self.staging, process_group)
        self._final_handle = symm_mem.rendezvous(self.final, process_group)
        self.staging_ptrs = [int(p) for p in self._staging_handle.buffer_ptrs]
        self.final_ptrs = [int(p) for p in self._final_handle.buffer_ptrs]
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)

    def order_ranks(self) -> None:
        """Stream-ordered barrier: a 4-byte all-reduce on the current stream."""
        import torch.distributed as dist

        dist.all_reduce(self.flag, group=self.group)


_peer_buffers: dict[tuple, PeerBuffers | None] = {}


def peer_buffers(process_group: Any, n_rows: int, hidden: int, dtype: torch.dtype,
                 device: torch.device) -> PeerBuffers | None:
    """The cached peer buffers of this problem, or None if peer-mapped memory cannot be set up on this
    machine. The decision is collective (a MIN all-reduce over the group), so either every rank takes the
    fused path or every rank takes the NCCL path."""
    key = (id(process_group), n_rows, hidden, dtype, device.index)
    if key not in _peer_buffers:
        import torch.distributed as dist

        try:
            bufs = PeerBuffers(process_group, n_rows, hidden, dtype, device)
        except Exception:  # noqa: BLE001 - e.g. no peer access between these GPUs
            bufs = None
        agreed = torch.tensor([1.0 if bufs is not None else 0.0], device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=process_group)
        _peer_buffers[key] = bufs if float(agreed.item()) == 1.0 else None
    return _peer_buffers[key]
