"""Full-size parity of the benchmark configurations that the CPU oracle cannot reach: the large-vocabulary
head (16384 x 2304 x 256000, the only one above the 131072-column limit of the reference's own backward
kernel), one rank's shard of the 14B-class head (65536 x 5120 x 19008 of 152064, row-chunk plan, sum
reduction, upstream gradient 1/65536) and the 65536-token point of the Llama-3 sweep, forward-only and
forward+backward. The oracle is the same fp32 expression as everywhere else, evaluated row chunk by row
chunk on the GPU with TF32 off. Tolerances: tests/_helpers.py. GPU only; each case holds a few GB."""

from __future__ import annotations

import ctypes
import gc

import pytest
import torch

from _helpers import GRAD_RTOL_16BIT, LOSS_RTOL, rel_loss_err, scaled_max_err
from helion_b200 import _lib, inputs, ops
from oracle import oracle
from test_gpu_guards import Guarded, stream

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _exact_fp32_and_clean_memory():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a kernel reported a bounded wait that ran out"
    gc.collect()
    torch.cuda.empty_cache()


def scaled_err_gpu(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max|got - ref| / max|ref| without moving GB-sized gradients to the host."""
    return float((got.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-30))


def test_large_vocab_head_full_size():
    cfg = inputs.CONFIGS["large-vocab"]
    d = inputs.make_inputs(cfg)
    n, h, v = cfg.rows, cfg.hidden, cfg.vocab
    x = d["hidden"].to(DEV).requires_grad_(True)
    w = d["weight"].to(DEV).requires_grad_(True)
    t = d["target"].to(DEV)
    assert int((t == -100).sum()) == round(0.01 * n)
    loss = ops.linear_cross_entropy(x, w, t)
    loss.backward()
    torch.cuda.synchronize()
    ref = oracle.expression_chunked(x.detach(), w.detach(), t, chunk_rows=512)
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert scaled_err_gpu(x.grad.view(n, h), ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_err_gpu(w.grad, ref["dw"]) <= GRAD_RTOL_16BIT
    # rows of G sum to zero, so dW summed over the vocabulary vanishes; ignored rows get no gradient
    col_sum = w.grad.float().sum(dim=0)
    assert float(col_sum.abs().max()) <= 2e-2 * float(w.grad.float().abs().sum(dim=0).max())
    assert float(x.grad.view(n, h)[t.view(-1) == -100].abs().max()) == 0.0


@pytest.mark.parametrize("rows", [65536])
def test_llama3_sweep_longest_point(rows):
    cfg = inputs.sweep_config(rows)
    d = inputs.make_inputs(cfg)
    n, h, v = cfg.rows, cfg.hidden, cfg.vocab
    x = d["hidden"].to(DEV).requires_grad_(True)
    w = d["weight"].to(DEV).requires_grad_(True)
    t = d["target"].to(DEV)
    ref = oracle.expression_chunked(x.detach(), w.detach(), t, chunk_rows=1024)
    # forward only: per-token loss (= -log-probability of the target), nothing reduced
    with torch.no_grad():
        per_token = ops.linear_cross_entropy(x.detach(), w.detach(), t, reduction="none")
    ref_none = oracle.expression_chunked(x.detach(), w.detach(), t, reduction="none", want_grads=False, chunk_rows=1024)
    assert per_token.shape == t.shape and per_token.dtype == torch.float32
    torch.testing.assert_close(per_token, ref_none["loss"], rtol=LOSS_RTOL, atol=1e-4)
    # forward + backward, mean
    loss = ops.linear_cross_entropy(x, w, t)
    loss.backward()
    torch.cuda.synchronize()
    assert rel_loss_err(loss, ref["loss"]) <= LOSS_RTOL
    assert scaled_err_gpu(x.grad.view(n, h), ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_err_gpu(w.grad, ref["dw"]) <= GRAD_RTOL_16BIT


def test_14b_class_shard_of_one_rank_full_size():
    """Rank 3 of 8 of the 14B-class head: weight rows [57024, 76032), all 65536 tokens. The global logsumexp
    comes from the fp32 oracle over the whole vocabulary, as the other seven ranks would have supplied it."""
    cfg = inputs.CONFIGS["14b-class"]
    d = inputs.make_inputs(cfg)
    n, h, v = cfg.rows, cfg.hidden, cfg.vocab
    v_loc, rank = v // 8, 3
    start = rank * v_loc
    L = _lib.lib()
    code = _lib.DTYPE_BF16
    x = d["hidden"].to(DEV).view(n, h)
    t = d["target"].to(DEV).view(n)
    w_full = d["weight"].to(DEV)
    full = oracle.expression_chunked(x, w_full, t, reduction="sum", want_grads=False, chunk_rows=1024)
    w_loc = w_full[start:start + v_loc].contiguous()
    del w_full
    go = d["grad_out"].to(DEV)
    assert abs(float(go) - 1.0 / 65536) < 1e-12
    scale = torch.where(t != -100, go.expand(n), torch.zeros(n, device=DEV))
    ref = oracle.shard_backward_chunked(x, w_loc, t, start, full["lse"], scale, chunk_rows=2048)

    # forward statistics of the shard
    stats = ops.local_stats(x, w_loc, t, start)
    torch.cuda.synchronize()
    torch.testing.assert_close(stats[0], ref["stats"][0], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(stats[1], ref["stats"][1], rtol=2e-4, atol=1e-4)
    assert torch.equal(torch.isinf(stats[2]), torch.isinf(ref["stats"][2]))
    inside = ~torch.isinf(stats[2])
    assert int(inside.sum()) > 0
    torch.testing.assert_close(stats[2][inside], ref["stats"][2][inside], rtol=1e-4, atol=1e-4)

    # the plan: 65536 x 19008 x 2 bytes of G is ten times the 256 MiB block cap, and with many rows and a short
    # shard the cheapest grid has several row chunks (dW summed over them in fp32) - here 4 chunks x 3 bands
    plan = (ctypes.c_int64 * 4)()
    _lib.check(L.lce_backward_plan(n, h, v_loc, code, 0, 0, x.data_ptr(), w_loc.data_ptr(), plan), "lce_backward_plan")
    nr, nc, n_rblk, n_cblk = (int(p) for p in plan)
    assert n_rblk > 1 and nr * n_rblk >= n and nc * n_cblk >= v_loc and nr * nc * 2 <= 256 << 20
    assert (nr, nc) == (16384, 8192)

    # backward through the C ABI, outputs and workspace between guard zones, twice: same bits both times
    runs = []
    for _ in range(2):
        dx, dw = Guarded(n * h * 2), Guarded(v_loc * h * 2)
        ws = Guarded(L.lce_backward_workspace_bytes(n, h, v_loc, code, 0, 0))
        _lib.check(L.lce_backward(x.data_ptr(), w_loc.data_ptr(), t.data_ptr(), 1, full["lse"].data_ptr(), go.data_ptr(),
                                  n, h, v_loc, start, code, -100, _lib.REDUCTION_SUM, dx.ptr, dw.ptr, ws.ptr, ws.nbytes,
                                  0, 0, None, None, None, stream()), "lce_backward")
        torch.cuda.synchronize()
        assert dx.intact() and dw.intact() and ws.intact()
        runs.append((dx.view(torch.bfloat16, (n, h)).clone(), dw.view(torch.bfloat16, (v_loc, h)).clone()))
        del dx, dw, ws
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][1], runs[1][1])
    assert scaled_err_gpu(runs[0][0], ref["dx"]) <= GRAD_RTOL_16BIT
    assert scaled_err_gpu(runs[0][1], ref["dw"]) <= GRAD_RTOL_16BIT
    assert float(runs[0][0][t == -100].abs().max()) == 0.0
