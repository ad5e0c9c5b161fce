"""Vocabulary-parallel runs on 2+ real GPUs (NCCL): same loss and gradients as the unsharded op.
Skipped on a single-GPU box. Ranks are child processes; no kernel here waits on another rank."""

from __future__ import annotations

import os
import socket
import sys
import traceback
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results, dx_reduce: str = "p2p") -> None:
    sys.path.insert(0, str(ROOT))
    os.environ["HELION_B200_DX_REDUCE"] = dx_reduce
    try:
        import torch.distributed as dist

        from helion_b200 import _lib, inputs, ops, parallel

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        for name, shape, red in [("llama3-8b", dict(rows=640, hidden=512, vocab=4 * 1002), "mean"),
                                 ("14b-class", dict(rows=1536, hidden=256, vocab=4 * 594), "sum")]:
            cfg = inputs.scaled(inputs.CONFIGS[name], **shape)
            d = inputs.make_inputs(cfg)
            go = torch.tensor(0.8, device=dev)
            x = d["hidden"].to(dev).requires_grad_(True)
            w_full = d["weight"].to(dev).requires_grad_(True)
            t = d["target"].to(dev)
            ref = ops.linear_cross_entropy(x, w_full, t, reduction=red)
            ref.backward(go)
            xs = d["hidden"].to(dev).requires_grad_(True)
            w_loc, start = parallel.shard_weight(d["weight"].to(dev), dist.group.WORLD)
            w_loc.requires_grad_(True)
            for _ in range(2):  # twice: the peer buffers of the first step are reused by the second
                xs.grad = w_loc.grad = None
                loss = ops.linear_cross_entropy(xs, w_loc, t, reduction=red, process_group=dist.group.WORLD,
                                                vocab_start=start)
                loss.backward(go)
            torch.cuda.synchronize()
            assert abs(float(loss) - float(ref)) <= 1e-6 * abs(float(ref)), (float(loss), float(ref))
            edx = float((xs.grad.float() - x.grad.float()).abs().max() / x.grad.float().abs().max())
            sl = w_full.grad[start:start + w_loc.shape[0]].float()
            edw = float((w_loc.grad.float() - sl).abs().max() / sl.abs().max())
            # the merged logsumexp may differ from the unsharded one in the last bit, which can flip a rounding of G
            assert edx <= 8e-3 and edw <= 8e-3, (name, edx, edw)
            # every rank holds the same bits
            both = [torch.empty_like(loss) for _ in range(world)]
            dist.all_gather(both, loss)
            assert all(torch.equal(both[0], b) for b in both)
        # greedy head over the sharded vocabulary = greedy head over the whole one
        from helion_b200 import decode_ops

        tok_full, lp_full = decode_ops.greedy_head(x.detach(), w_full.detach())
        tok, lp = decode_ops.greedy_head(xs.detach(), w_loc.detach(), process_group=dist.group.WORLD)
        assert torch.equal(tok, tok_full)
        torch.testing.assert_close(lp, lp_full, rtol=1e-5, atol=1e-5)
        assert _lib.device_status() == 0
        dist.barrier()
        dist.destroy_process_group()
        results[rank] = "ok"
    except Exception:  # noqa: BLE001
        results[rank] = "error: " + traceback.format_exc(limit=4)


@pytest.mark.parametrize("dx_reduce", ["p2p", "nccl"])
@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_matches_single_gpu(world, dx_reduce):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results, dx_reduce)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
    assert dict(results) == {r: "ok" for r in range(world)}
