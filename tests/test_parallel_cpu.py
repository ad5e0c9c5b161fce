"""World-size-2 tests of the vocabulary-parallel plumbing on CPU ranks (gloo). The kernels are replaced by
the oracle's per-shard statistics; what is under test is helion_b200.parallel: shard bounds, the
statistics exchange, the dX reduction, and that a rank which never joins surfaces as an error."""

from __future__ import annotations

import datetime
import os
import socket
import sys
import traceback
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    g = torch.Generator().manual_seed(11)
    x = torch.randn(96, 40, generator=g).bfloat16()
    w = (torch.randn(1003, 40, generator=g) * 0.2).bfloat16()
    t = torch.randint(0, 1003, (96,), generator=g)
    t[::7] = -100
    return x, w, t


def _worker(rank: int, world: int, port: int, scenario: str, results) -> None:
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from helion_b200 import parallel
    from oracle import oracle

    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
        x, w, t = _problem()
        if scenario == "rank1_never_joins" and rank == 1:
            results[rank] = "left"
            return  # leaves between steps, with nothing in flight
        w_loc, start = parallel.shard_weight(w, dist.group.WORLD)
        assert (start, start + w_loc.shape[0]) == parallel.shard_bounds(w.shape[0], world, rank)
        # 1003 rows over two ranks are 502 + 501: the default start of rank 1 is 502, not rank * 501
        cpu = torch.device("cpu")
        assert parallel.shard_start(dist.group.WORLD, w_loc.shape[0], cpu) == start
        assert parallel.shard_start(dist.group.WORLD, w_loc.shape[0], cpu) == start  # cached: no second collective
        # plans derived from the local shard height: equal values agree, rank-dependent ones do not
        assert parallel.ranks_agree(dist.group.WORLD, ("same",), (96, 3), cpu)
        assert not parallel.ranks_agree(dist.group.WORLD, ("differ",), (96, 3 + rank), cpu)
        # a batch copied to the ranks one row slice each is rebuilt by one all-gather (96 rows -> 48 + 48;
        # 95 rows -> 48 + 47 padded to 48)
        for n in (96, 95):
            rpr = -(-n // world)
            piece = torch.zeros(rpr, 40, dtype=x.dtype)
            mine = x[:n][rank * rpr:(rank + 1) * rpr]
            piece[:mine.shape[0]] = mine
            assert torch.equal(parallel.gather_rows(piece, n, dist.group.WORLD), x[:n])
        stats = parallel.gather_stats(oracle.shard_stats(x, w_loc, t, start), dist.group.WORLD)
        assert stats.shape == (world, 3, 96)
        merged = oracle.merge_stats(stats, t)
        full = oracle.expression(x, w, t)
        torch.testing.assert_close(merged["loss"], full["loss"], rtol=1e-5, atol=1e-5)
        # partial dX of this shard: G restricted to the local columns, with the GLOBAL logsumexp
        z = x.float() @ w_loc.float().T
        g = torch.exp(z - merged["lse"][:, None])
        rel = t - start
        inside = (rel >= 0) & (rel < w_loc.shape[0])
        g[torch.arange(96)[inside], rel[inside]] -= 1.0
        valid = t != -100
        g *= (valid.float() / valid.sum())[:, None]
        dx = parallel.reduce_dx(g @ w_loc.float(), torch.bfloat16, dist.group.WORLD)
        assert dx.dtype == torch.bfloat16
        err = (dx.float() - full["dx"]).abs().max() / full["dx"].abs().max()
        assert err < 1e-2, float(err)
        # greedy head: each rank reduces its shard, one all-gather, every rank merges to the unsharded answer
        local = oracle.greedy_expression(x, w_loc)
        packed = parallel.pack_greedy(local["token"] + start, local["logprob"], local["lse"])
        token, logprob, lse = parallel.merge_greedy(parallel.gather_stats(packed, dist.group.WORLD))
        whole = oracle.greedy_expression(x, w)
        assert torch.equal(token, whole["token"])
        torch.testing.assert_close(logprob, whole["logprob"], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(lse, whole["lse"], rtol=1e-5, atol=1e-5)
        # every rank ends with identical bits
        gathered = [torch.empty_like(merged["lse"]) for _ in range(world)]
        dist.all_gather(gathered, merged["lse"])
        assert all(torch.equal(gathered[0], other) for other in gathered)
        results[rank] = "ok"
    except Exception:  # noqa: BLE001 - reported to the parent
        results[rank] = "error: " + traceback.format_exc(limit=3)
    finally:
        if dist.is_initialized() and scenario == "normal":
            dist.destroy_process_group()


def _run(scenario: str) -> dict:
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, scenario, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish: the collective must time out, not hang")
    return dict(results)


def test_two_rank_exchange_matches_single_rank():
    assert _run("normal") == {0: "ok", 1: "ok"}


def test_missing_rank_becomes_an_error_not_a_hang():
    res = _run("rank1_never_joins")
    assert res[1] == "left"
    assert res[0].startswith("error"), res


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_greedy_merge_over_shards_is_the_unsharded_argmax(world):
    """The merge alone (no process group): tokens beyond 2^31 survive the float32 packing, and a maximum
    that appears in two shards resolves to the lower index."""
    from helion_b200 import parallel
    from oracle import oracle

    g = torch.Generator().manual_seed(world)
    x = torch.randn(33, 24, generator=g).bfloat16()
    w = (torch.randn(8 * 125, 24, generator=g) * 0.3).bfloat16()
    w[900] = w[17] = x[0] * 3  # the same winning row in the first and in the last shard
    packed = []
    for r in range(world):
        s, e = parallel.shard_bounds(w.shape[0], world, r)
        loc = oracle.greedy_expression(x, w[s:e])
        packed.append(parallel.pack_greedy(loc["token"] + s, loc["logprob"], loc["lse"]))
    token, logprob, lse = parallel.merge_greedy(torch.stack(packed))
    whole = oracle.greedy_expression(x, w)
    assert torch.equal(token, whole["token"]) and int(token[0]) == 17
    torch.testing.assert_close(logprob, whole["logprob"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lse, whole["lse"], rtol=1e-5, atol=1e-5)
    big = torch.tensor([5_000_000_123, 7], dtype=torch.int64)
    buf = parallel.pack_greedy(big, torch.zeros(2), torch.zeros(2))
    assert torch.equal(parallel.merge_greedy(buf[None])[0], big)
