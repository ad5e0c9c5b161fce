"""Parity of the plain cross-entropy kernels (materialised logits) with the oracle. GPU only."""

from __future__ import annotations

import importlib.util
import math
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

import helion_b200
from _helpers import reference_tolerances, rel_loss_err, scaled_max_err
from helion_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DEV = "cuda"


# ---- the reference's own tests, restated (tests/tritium/test_cross_entropy.py:11-56, 117-122) ---------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab_size", [16, 128, 1024])
@pytest.mark.parametrize("n_rows", [1, 16, 128])
def test_cross_entropy_forward(dtype, vocab_size, n_rows):
    logits = torch.randn(n_rows, vocab_size, device=DEV, dtype=dtype)
    target = torch.randint(vocab_size, (n_rows,), device=DEV)
    loss = helion_b200.cross_entropy(logits, target)
    torch.testing.assert_close(loss, F.cross_entropy(logits.float(), target), rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cross_entropy_backward(dtype):
    logits = torch.randn(64, 256, device=DEV, dtype=dtype)
    target = torch.randint(256, (64,), device=DEV)
    grad_out = torch.randn((), device=DEV, dtype=torch.float32)
    lse = torch.logsumexp(logits.float(), dim=-1)
    dlogits = helion_b200.cross_entropy_backward(grad_out, logits, target, lse)
    ref = logits.detach().float().clone().requires_grad_(True)
    F.cross_entropy(ref, target).backward(grad_out)
    rtol, atol = reference_tolerances(dtype)
    torch.testing.assert_close(dlogits, ref.grad.to(dtype), rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cross_entropy_autograd(dtype):
    logits = torch.randn(32, 128, device=DEV, dtype=dtype, requires_grad=True)
    target = torch.randint(128, (32,), device=DEV)
    helion_b200.cross_entropy(logits, target).backward()
    ref = logits.detach().float().clone().requires_grad_(True)
    F.cross_entropy(ref, target).backward()
    rtol, atol = reference_tolerances(dtype)
    torch.testing.assert_close(logits.grad, ref.grad.to(dtype), rtol=rtol, atol=atol)


def test_cross_entropy_rejects_non_contiguous():
    logits = torch.randn(4, 16, device=DEV).T
    with pytest.raises(ValueError, match="contiguous"):
        helion_b200.cross_entropy(logits, torch.randint(4, (16,), device=DEV))


# ---- committed fixtures (oracle expression + what the reference's kernels returned on a B200) --------
CASES = [(i, c) for i, c in enumerate(make_golden.case_list()) if c.get("op") == "plain"]
ORACLE_FIXTURE = torch.load(GOLDEN / "oracle_cases.pt", weights_only=False)
REFERENCE_FIXTURE = torch.load(GOLDEN / "reference_b200.pt", weights_only=False)


@pytest.mark.parametrize("index,case", CASES, ids=[c["name"] for _, c in CASES])
def test_against_committed_fixtures(index, case):
    inp = make_golden.make_case_inputs(case, index)
    exp = ORACLE_FIXTURE[case["name"]]["expected"]
    ref = REFERENCE_FIXTURE[case["name"]]
    dtype = inp["logits"].dtype
    z = inp["logits"].to(DEV).requires_grad_(case["grads"])
    loss = helion_b200.cross_entropy(z, inp["target"].to(DEV))
    assert rel_loss_err(loss, exp["loss"]) <= 1e-5
    torch.testing.assert_close(loss.cpu(), ref["loss"], rtol=1e-5, atol=1e-5)
    if case["grads"]:
        loss.backward(inp["grad_out"].to(DEV))
        tol = 1e-5 if dtype == torch.float32 else 8e-3
        assert scaled_max_err(z.grad, exp["dlogits"]) <= tol
        assert scaled_max_err(z.grad, ref["dlogits"].float()) <= tol


# ---- beyond the reference's sizes: chunked rows, ragged widths, reductions, ignored labels -----------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 1), (5, 7), (33, 8191), (17, 8192), (9, 8193), (4, 40000), (2, 200001)])
def test_shapes_including_rows_longer_than_one_chunk(shape, dtype):
    n, v = shape
    g = torch.Generator().manual_seed(n * 31 + v)
    z = (torch.randn(n, v, generator=g) * 3).to(dtype)
    t = torch.randint(0, v, (n,), generator=g)
    ref = oracle.plain_expression(z, t, grad_out=torch.tensor(0.7))
    zd = z.to(DEV).requires_grad_(True)
    loss = helion_b200.cross_entropy(zd, t.to(DEV))
    loss.backward(torch.tensor(0.7, device=DEV))
    if v > 1:
        assert rel_loss_err(loss, ref["loss"]) <= 1e-5
        tol = 1e-5 if dtype == torch.float32 else 8e-3
        assert scaled_max_err(zd.grad, ref["dlogits"]) <= tol
    else:
        assert abs(float(loss)) <= 1e-6  # a single class: the loss is zero up to the exp2/log round trip
    assert zd.grad.dtype == dtype and _lib.device_status() == 0


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_reductions_and_ignore_index(reduction):
    g = torch.Generator().manual_seed(5)
    z = torch.randn(300, 1000, generator=g).bfloat16()
    t = torch.randint(0, 1000, (300,), generator=g)
    t[::5] = -100
    go = torch.randn(300, generator=g) if reduction == "none" else torch.tensor(3.0)
    ref = oracle.plain_expression(z, t, reduction=reduction, grad_out=go)
    zd = z.to(DEV).requires_grad_(True)
    loss = helion_b200.cross_entropy(zd, t.to(DEV), reduction=reduction)
    loss.backward(go.to(DEV))
    assert rel_loss_err(loss, ref["loss"]) <= 1e-5
    assert scaled_max_err(zd.grad, ref["dlogits"]) <= 8e-3
    assert float(zd.grad[0].abs().max()) == 0.0  # ignored rows get exactly zero


def test_empty_batch_int32_targets_and_determinism():
    empty = helion_b200.cross_entropy(torch.empty(0, 50, device=DEV), torch.empty(0, dtype=torch.int64, device=DEV))
    assert float(empty) == 0.0
    z = torch.randn(64, 30000, device=DEV, dtype=torch.bfloat16)
    t = torch.randint(0, 30000, (64,), device=DEV)
    a = helion_b200.cross_entropy(z, t)
    b = helion_b200.cross_entropy(z, t.int())
    assert torch.equal(a, b) and torch.equal(a, helion_b200.cross_entropy(z, t))
    assert math.isinf(float(helion_b200.cross_entropy(z, torch.full_like(t, 30000))))  # matches no column
