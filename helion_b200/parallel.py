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


def group_key(process_group: Any):
    """A key for per-group caches: the group's unique name where torch gives it one (an ``id()`` can be handed
    to a new group after the old one is gone), else the object's id."""
    return getattr(process_group, "group_name", None) or id(process_group)


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
    """Symmetric (peer-mapped) staging buffers of one (group, H, device), allocated once for a capacity
    in rows and reused by every problem that fits:

    * two ``staging`` buffers ``[world, rows_per_rank, H]`` fp32 on every rank: rank r's dX epilogue stores
      the partial rows owned by rank o into slot r of rank o's staging buffer. Calls alternate between
      the two buffers.

    One 4-byte all-reduce per call orders the ranks (everyone has scattered before anyone sums). The
    owner then sums the ``world`` slots of its row slice in rank order, rounds once, and an NCCL
    all-gather hands every rank the whole dX. Why two buffers make a second barrier unnecessary: a rank
    scatters into buffer b again two calls later, after it has passed the barrier of the call in
    between, which every rank enters only after it has finished summing buffer b (same stream).
    No kernel of this package waits on another GPU, and nothing here uses an NVLink multicast object:
    the buffers are only ever written with plain peer stores, so multicast binding is switched off
    for the allocation (a rank that exits while its memory is bound to a multicast object can raise
    NVLink faults on its peers).
    """

    def __init__(self, process_group: Any, capacity_rows: int, hidden: int, device: torch.device):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world = group_rank_size(process_group)
        self.group = process_group
        self.hidden = hidden
        self.capacity_rows = capacity_rows
        slot_rows = -(-capacity_rows // self.world)
        self.staging, self.staging_ptrs = [], []
        self._handles = []
        for _ in range(2):
            buf = symm_mem.empty((self.world * slot_rows * hidden,), dtype=torch.float32, device=device)
            handle = symm_mem.rendezvous(buf, process_group)
            self.staging.append(buf)
            self._handles.append(handle)
            self.staging_ptrs.append([int(p) for p in handle.buffer_ptrs])
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.calls = 0

    def next_buffer(self) -> int:
        """Index (0 / 1) of the staging buffer this call scatters into; alternates call by call, in the
        same order on every rank because every rank makes the same sequence of calls."""
        b = self.calls & 1
        self.calls += 1
        return b

    def order_ranks(self) -> None:
        """Stream-ordered barrier: a 4-byte all-reduce on the current stream."""
        import torch.distributed as dist

        dist.all_reduce(self.flag, group=self.group)


_peer_buffers: dict[tuple, PeerBuffers | None] = {}


def peer_buffers(process_group: Any, n_rows: int, hidden: int, device: torch.device) -> PeerBuffers | None:
    """The cached peer buffers that hold ``n_rows`` rows of ``hidden`` floats, or None if peer-mapped
    memory cannot be set up on this machine. One pair of buffers per (group, hidden, device): a batch of
    fewer rows reuses it, a larger one replaces it (collectively - every rank sees the same ``n_rows``),
    so variable-length batches neither leak symmetric memory nor rendezvous again. The decision to use the
    fused path is collective too (a MIN all-reduce over the group), so either every rank takes it or
    every rank takes the NCCL path."""
    key = (group_key(process_group), hidden, device.index)
    have = _peer_buffers.get(key, False)
    if have is None:
        return None
    if have is False or have.capacity_rows < n_rows:
        import torch.distributed as dist

        if have is not False:
            # a smaller pair is being replaced: nothing on this GPU or its peers may still be writing into it
            torch.cuda.synchronize(device)
            dist.barrier(group=process_group)
        _peer_buffers.pop(key, None)  # drop the smaller pair before its replacement is allocated
        del have
        try:
            bufs = PeerBuffers(process_group, n_rows, hidden, device)
        except Exception:  # noqa: BLE001 - e.g. no peer access between these GPUs
            bufs = None
        agreed = torch.tensor([1.0 if bufs is not None else 0.0], device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=process_group)
        _peer_buffers[key] = bufs if float(agreed.item()) == 1.0 else None
    return _peer_buffers[key]


# ---- where a shard begins, and whether the ranks agree on a plan ---------------------------------------
_shard_starts: dict[tuple, int] = {}
_agreements: dict[tuple, bool] = {}


def shard_start(process_group: Any, v_local: int, device: torch.device) -> int:
    """First global vocabulary row of this rank's shard when the caller did not say: the sum of the shard
    heights of the lower ranks (one small all-gather the first time a (group, height) pair is seen).
    With equal shards this is ``rank * v_local``; with the uneven shards of ``shard_weight`` it is not."""
    rank, world = group_rank_size(process_group)
    if world == 1:
        return 0
    key = (group_key(process_group), v_local)
    if key not in _shard_starts:
        import torch.distributed as dist

        mine = torch.tensor([v_local], dtype=torch.int64, device=device)
        heights = torch.empty((world,), dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(heights, mine, group=process_group)
        _shard_starts[key] = int(heights[:rank].sum().item())
    return _shard_starts[key]


def ranks_agree(process_group: Any, key: tuple, values: tuple[int, ...], device: torch.device) -> bool:
    """True if every rank of the group passes the same ``values`` (checked once per ``key`` with one small
    all-gather). Used before a sequence of collectives whose count and sizes each rank derives locally."""
    rank, world = group_rank_size(process_group)
    if world == 1:
        return True
    full_key = (group_key(process_group),) + key
    if full_key not in _agreements:
        import torch.distributed as dist

        mine = torch.tensor(values, dtype=torch.int64, device=device)
        everyone = torch.empty((world * len(values),), dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(everyone, mine, group=process_group)
        _agreements[full_key] = bool((everyone.view(world, len(values)) == mine).all().item())
    return _agreements[full_key]


def gather_rows(local_rows: torch.Tensor, n_rows: int, process_group: Any) -> torch.Tensor:
    """All-gather of row slices: rank r holds rows ``[r * rpr, (r+1) * rpr)`` of an ``[n_rows, ...]`` tensor
    (rpr = ceil(n_rows / world); the last ranks' slices may be short or empty but arrive padded to rpr rows).
    Returns the full tensor on every rank. Used to rebuild activations that were copied to the GPUs one
    slice per rank, so that a batch crosses the host link once instead of once per GPU."""
    rank, world = group_rank_size(process_group)
    if world == 1:
        return local_rows[:n_rows]
    import torch.distributed as dist

    rpr = local_rows.shape[0]
    out = torch.empty((world * rpr,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    dist.all_gather_into_tensor(out, local_rows.contiguous(), group=process_group)
    return out[:n_rows]
