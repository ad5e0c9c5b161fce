"""CPU tests of the oracle: its layers agree with each other, with the committed fixtures and - through
reference_b200.pt - with what the reference's own kernels returned on a B200."""

from __future__ import annotations

import importlib.util
import math
from pathlib import Path

import pytest
import torch

from oracle import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)

CASES = make_golden.case_list()
ORACLE_FIXTURE = torch.load(GOLDEN / "oracle_cases.pt", weights_only=False)
REF_PATH = GOLDEN / "reference_b200.pt"
REFERENCE_FIXTURE = torch.load(REF_PATH, weights_only=False) if REF_PATH.exists() else None


def _inputs(name: str) -> tuple[dict, dict]:
    idx = next(i for i, c in enumerate(CASES) if c["name"] == name)
    return CASES[idx], make_golden.make_case_inputs(CASES[idx], idx)


LINEAR = [c for c in CASES if c.get("op") != "plain"]
PLAIN = [c for c in CASES if c.get("op") == "plain"]


@pytest.mark.parametrize("name", [c["name"] for c in CASES])
def test_expression_matches_committed_fixture(name):
    case, inp = _inputs(name)
    rec = ORACLE_FIXTURE[name]
    # the seeded inputs are the ones the fixture was made from
    assert make_golden.input_checksums(inp) == pytest.approx(rec["input_checksums"], rel=0, abs=0)
    if case.get("op") == "plain":
        got = oracle.plain_expression(inp["logits"], inp["target"], grad_out=inp["grad_out"], want_grads=case["grads"])
    else:
        got = oracle.expression(inp["hidden"], inp["weight"], inp["target"], grad_out=inp["grad_out"],
                                want_grads=case["grads"])
    for key, exp in rec["expected"].items():
        torch.testing.assert_close(got[key], exp, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_chunked_expression_equals_expression(reduction):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 50, 48, generator=g).bfloat16()
    w = torch.randn(333, 48, generator=g).bfloat16()
    t = torch.randint(0, 333, (3, 50), generator=g)
    t[0, :7] = -100
    go = torch.randn(3, 50, generator=g) if reduction == "none" else torch.tensor(0.3)
    a = oracle.expression(x, w, t, reduction=reduction, grad_out=go)
    b = oracle.expression_chunked(x, w, t, reduction=reduction, grad_out=go, chunk_rows=32)
    for key in ("loss", "lse", "dx", "dw"):
        torch.testing.assert_close(a[key], b[key], rtol=2e-4, atol=1e-5)


@pytest.mark.parametrize("vocab", [65, 256, 257, 1000])
def test_restated_forward_is_the_mean_cross_entropy(vocab):
    g = torch.Generator().manual_seed(vocab)
    x = torch.randn(40, 64, generator=g)
    w = torch.randn(vocab, 64, generator=g)
    t = torch.randint(0, vocab, (40,), generator=g)
    r = oracle.restated_forward(x, w, t)
    e = oracle.expression(x, w, t, want_grads=False)
    torch.testing.assert_close(r["loss"], e["loss"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(r["lse"], e["lse"], rtol=1e-5, atol=1e-5)


def test_restated_forward_unmatched_target_gives_infinite_loss():
    # the reference has no ignored label: -100 matches no column (tritium/ops/cross_entropy.py:240-244)
    x, w = torch.randn(4, 8), torch.randn(300, 8)
    t = torch.tensor([1, -100, 2, 3])
    assert math.isinf(float(oracle.restated_forward(x, w, t)["loss"]))


@pytest.mark.parametrize("shape", [(32, 64, 256), (80, 64, 832), (48, 72, 300)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_restated_backward_tracks_expression(shape, dtype):
    n, h, v = shape
    g = torch.Generator().manual_seed(n + v)
    x = torch.randn(n, h, generator=g).to(dtype)
    w = torch.randn(v, h, generator=g).to(dtype)
    t = torch.randint(0, v, (n,), generator=g)
    go = torch.tensor(1.7)
    e = oracle.expression(x, w, t, grad_out=go)
    r = oracle.restated_backward(go, x, w, t, e["lse"])
    # The reference's chunk loop rounds the LOGITS to the input dtype before the softmax
    # (tritium/ops/cross_entropy.py:937); with std-1 weights that alone moves 16-bit gradients by
    # several percent of their maximum. The fused small-shape kernel keeps fp32 logits.
    fused = h <= 64 and v >= 256 and n * v <= 65_536
    tol = 1e-5 if dtype == torch.float32 else (3e-2 if fused else 1.5e-1)
    for key in ("dx", "dw"):
        err = (r[key].float() - e[key]).abs().max() / e[key].abs().max()
        assert err <= tol, (key, float(err))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("vocab", [1000, 1003])
def test_sharded_statistics_merge_to_the_unsharded_result(world, vocab):
    from helion_b200 import parallel

    g = torch.Generator().manual_seed(world * vocab)
    x = torch.randn(64, 32, generator=g).bfloat16()
    w = (torch.randn(vocab, 32, generator=g) * 0.3).bfloat16()
    t = torch.randint(0, vocab, (64,), generator=g)
    t[::9] = -100
    stats = []
    for r in range(world):
        s, e = parallel.shard_bounds(vocab, world, r)
        stats.append(oracle.shard_stats(x, w[s:e], t, s))
    for red in ("mean", "sum", "none"):
        merged = oracle.merge_stats(torch.stack(stats), t, reduction=red)
        full = oracle.expression(x, w, t, reduction=red, want_grads=False)
        torch.testing.assert_close(merged["loss"], full["loss"], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(merged["lse"], full["lse"], rtol=1e-5, atol=1e-5)


# ---- pinning against the reference's own kernels (fixture produced on a B200) ------------------------
needs_reference_fixture = pytest.mark.skipif(REFERENCE_FIXTURE is None, reason="reference_b200.pt not committed")


def test_restated_plain_op_is_the_mean_cross_entropy():
    g = torch.Generator().manual_seed(77)
    z = torch.randn(50, 333, generator=g).bfloat16()
    t = torch.randint(0, 333, (50,), generator=g)
    e = oracle.plain_expression(z, t, grad_out=torch.tensor(1.3))
    r = oracle.restated_plain_forward(z, t)
    torch.testing.assert_close(r["loss"], e["loss"], rtol=1e-5, atol=1e-5)
    dz = oracle.restated_plain_backward(torch.tensor(1.3), z, t, r["lse"])
    assert (dz.float() - e["dlogits"]).abs().max() / e["dlogits"].abs().max() < 8e-3


@needs_reference_fixture
@pytest.mark.parametrize("name", [c["name"] for c in PLAIN])
def test_restated_plain_op_matches_reference_kernels(name):
    case, inp = _inputs(name)
    ref = REFERENCE_FIXTURE[name]
    got = oracle.restated_plain_forward(inp["logits"], inp["target"])
    torch.testing.assert_close(got["loss"], ref["loss"], rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(got["lse"], ref["lse"], rtol=2e-5, atol=2e-5)
    if case["grads"]:
        dz = oracle.restated_plain_backward(inp["grad_out"], inp["logits"], inp["target"], ref["lse"])
        dtype = inp["logits"].dtype
        tol = 2e-5 if dtype == torch.float32 else 8e-3  # one rounding of the output
        for variant in ("dlogits", "dlogits_direct"):
            r = ref[variant].float()
            assert (dz.float() - r).abs().max() / r.abs().max() <= tol, variant
        # and the ground-truth expression is within the reference's own tolerance of its kernels
        exp = ORACLE_FIXTURE[name]["expected"]
        rtol, atol = (1e-5, 1e-5) if dtype == torch.float32 else (2e-2, 2e-2)
        torch.testing.assert_close(ref["dlogits"].float(), exp["dlogits"].to(dtype).float(), rtol=rtol, atol=atol)


@needs_reference_fixture
@pytest.mark.parametrize("name", [c["name"] for c in LINEAR])
def test_restated_forward_matches_reference_kernels(name):
    case, inp = _inputs(name)
    ref = REFERENCE_FIXTURE[name]
    got = oracle.restated_forward(inp["hidden"], inp["weight"], inp["target"])
    # the reference's own test tolerance for the loss (tests/tritium/test_cross_entropy.py:73) is
    # rtol 2e-2 / atol 2e-3; the restatement accumulates in fp32 exactly like the kernels, so it is
    # held to a far tighter bound
    torch.testing.assert_close(got["loss"], ref["loss"], rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(got["lse"], ref["lse"].reshape(-1), rtol=2e-5, atol=2e-5)


@needs_reference_fixture
@pytest.mark.parametrize("name", [c["name"] for c in LINEAR if c["grads"]])
def test_restated_backward_matches_reference_kernels(name):
    case, inp = _inputs(name)
    ref = REFERENCE_FIXTURE[name]
    lse = ref["lse"].reshape(-1)
    got = oracle.restated_backward(inp["grad_out"], inp["hidden"], inp["weight"], inp["target"], lse)
    dtype = inp["hidden"].dtype
    # 16-bit results may differ by one rounding of the output (different summation order inside the GEMMs)
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    for key in ("dx", "dw"):
        for variant in (key, key + "_direct"):
            r = ref[variant].float()
            err = (got[key].float() - r).abs().max() / r.abs().max()
            assert err <= tol, (variant, float(err))


@needs_reference_fixture
@pytest.mark.parametrize("name", [c["name"] for c in LINEAR if c["grads"]])
def test_expression_is_within_the_reference_tolerance_of_its_kernels(name):
    """The ground-truth expression and the reference's kernels agree at the reference's own tolerances
    (its tests/_utils.py:14-29), so parity against the expression is parity against the reference."""
    case, inp = _inputs(name)
    ref = REFERENCE_FIXTURE[name]
    exp = ORACLE_FIXTURE[name]["expected"]
    dtype = inp["hidden"].dtype
    rtol, atol = (1e-5, 1e-5) if dtype == torch.float32 else (3e-2, 3e-2)
    torch.testing.assert_close(ref["loss"], exp["loss"], rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(ref["dx"].float(), exp["dx"].to(dtype).float().reshape(ref["dx"].shape), rtol=rtol, atol=atol)
    torch.testing.assert_close(ref["dw"].float(), exp["dw"].to(dtype).float(), rtol=rtol, atol=atol)


def test_sharded_backward_of_all_ranks_adds_up_to_the_unsharded_gradients():
    """The per-rank oracle used for the full-size shard test: partial dX summed over the shards, the local dW
    blocks side by side and the merged statistics reproduce the unsharded expression."""
    g = torch.Generator().manual_seed(21)
    x = torch.randn(70, 48, generator=g).bfloat16()
    w = (torch.randn(403, 48, generator=g) * 0.2).bfloat16()
    t = torch.randint(0, 403, (70,), generator=g)
    t[::9] = -100
    full = oracle.expression(x, w, t, reduction="sum", grad_out=torch.tensor(0.25))
    scale = torch.where(t != -100, torch.tensor(0.25), torch.tensor(0.0))
    dx = torch.zeros(70, 48)
    stats, dws = [], []
    for start, end in [(0, 101), (101, 202), (202, 303), (303, 403)]:
        part = oracle.shard_backward_chunked(x, w[start:end], t, start, full["lse"], scale, chunk_rows=32)
        dx += part["dx"]
        dws.append(part["dw"])
        stats.append(part["stats"])
        torch.testing.assert_close(part["stats"], oracle.shard_stats(x, w[start:end], t, start))
    torch.testing.assert_close(dx, full["dx"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.cat(dws), full["dw"], rtol=1e-5, atol=1e-6)
    merged = oracle.merge_stats(torch.stack(stats), t, reduction="sum")
    torch.testing.assert_close(merged["loss"], full["loss"], rtol=1e-5, atol=1e-5)
