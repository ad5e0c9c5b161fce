"""Sampling head (top-k candidates + logsumexp without logits) against the fp32 oracle, and the sampling rule
built on it against a restatement of the reference's ``sample_next_token``. GPU only.

Tolerance: a logit is an H-long dot product accumulated in fp32 in a different order than the oracle's, so two
logits closer than ``tol = 1e-4 * max|z| + 1e-6`` may swap places. Values must agree to ``tol`` position by
position; indices must be bit-exact wherever a value is further than ``4 * tol`` from both neighbours in the
oracle's sorted list and from the first value left out."""

from __future__ import annotations

import pytest
import torch

import helion_b200
from helion_b200 import decode_ops
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def check_topk(hidden, weight, k, temperature=1.0):
    values, indices, lse = helion_b200.topk_head(hidden, weight, k, temperature=temperature)
    torch.cuda.synchronize()
    v = weight.shape[0]
    kk = min(k, v)
    ref = oracle.topk_expression(hidden.cpu(), weight.cpu(), kk + 1 if kk < v else kk, temperature)
    assert values.shape == hidden.shape[:-1] + (k,) and values.dtype == torch.float32
    assert indices.shape == values.shape and indices.dtype == torch.int64
    got_v = values.cpu().reshape(-1, k)
    got_i = indices.cpu().reshape(-1, k)
    ref_v = ref["values"].reshape(got_v.shape[0], -1)
    ref_i = ref["indices"].reshape(got_v.shape[0], -1)
    y = ref["logits"]
    tol = 1e-4 * float(y.abs().max()) + 1e-6
    if k > v:  # the tail beyond the vocabulary is -inf / -1
        assert torch.all(torch.isinf(got_v[:, v:])) and torch.all(got_i[:, v:] == -1)
    torch.testing.assert_close(got_v[:, :kk], ref_v[:, :kk], rtol=0, atol=tol)
    # every returned index points at a logit equal (to tol) to the value returned with it
    assert int(got_i[:, :kk].min()) >= 0 and int(got_i[:, :kk].max()) < v
    torch.testing.assert_close(y.gather(1, got_i[:, :kk]), got_v[:, :kk], rtol=0, atol=tol)
    # no index twice in a row
    assert all(len(set(r.tolist())) == kk for r in got_i[:, :kk])
    # bit-exact indices where the oracle's ordering is clear of rounding
    pad = torch.full((ref_v.shape[0], 1), float("inf"))
    ext = torch.cat([pad, ref_v, -pad], dim=1) if ref_v.shape[1] == kk else torch.cat([pad, ref_v], dim=1)
    gap_up = ext[:, :kk] - ext[:, 1:kk + 1]
    gap_down = ext[:, 1:kk + 1] - ext[:, 2:kk + 2]
    clear = (gap_up > 4 * tol) & (gap_down > 4 * tol)
    assert torch.equal(got_i[:, :kk][clear], ref_i[:, :kk][clear])
    assert float(clear.float().mean()) > 0.5, "the test data should leave most positions unambiguous"
    torch.testing.assert_close(lse.cpu().reshape(-1), ref["lse"].reshape(-1), rtol=1e-4, atol=1e-4)
    return values, indices, lse


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,k", [(((1,), 64, 1000), 5), (((7,), 256, 5003), 40), (((64,), 512, 32000), 64),
                                     (((2, 5), 128, 777), 8), (((3,), 72, 300), 50), (((130,), 768, 50304), 50),
                                     (((4,), 64, 20), 32)])
def test_topk_head_matches_the_oracle(shape, k, dtype):
    lead, h, v = shape
    g = torch.Generator().manual_seed(h + v + k)
    hidden = torch.randn(*lead, h, generator=g).to(dtype).to(DEV)
    weight = (torch.randn(v, h, generator=g) / h ** 0.5).to(dtype).to(DEV)
    check_topk(hidden, weight, k)
    check_topk(hidden, weight, min(k, 16), temperature=0.7)


@pytest.mark.parametrize("force", ["tc", "tc1", "simt"])
def test_a_tile_that_holds_most_of_the_best_is_repaired(force, monkeypatch):
    """All of the k best logits sit in ONE 256-column tile (and in one 128-column tile of the CUDA-core path):
    the epilogue delivers 8 per tile, the merge must notice and recompute the tile."""
    monkeypatch.setenv("HELION_B200_FORCE", force)
    g = torch.Generator().manual_seed(5)
    h, v, k = 256, 6000, 48
    hidden = torch.randn(9, h, generator=g).bfloat16()
    weight = (torch.randn(v, h, generator=g) * 0.02).bfloat16()
    # rows 2560 .. 2623 of the weight point along the hidden states' mean direction with distinct lengths
    direction = hidden.float().mean(dim=0)
    direction = direction / direction.norm()
    hidden = (hidden.float() + 4.0 * direction).bfloat16()
    for j in range(64):
        weight[2560 + j] = (direction * (0.5 + 0.03 * j)).bfloat16()
    values, indices, _ = check_topk(hidden.to(DEV), weight.to(DEV), k)
    assert bool(((indices >= 2560) & (indices < 2624)).all())


def test_equal_logits_resolve_to_the_lower_index():
    h, v = 64, 3000
    hidden = torch.ones(3, h, dtype=torch.bfloat16, device=DEV)
    weight = torch.zeros(v, h, dtype=torch.bfloat16, device=DEV)
    weight[[5, 700, 701, 2999]] = 1.0  # four logits of 64, everything else 0
    values, indices, lse = helion_b200.topk_head(hidden, weight, 8)
    assert indices[0].tolist() == [5, 700, 701, 2999, 0, 1, 2, 3]
    assert values[0].tolist() == [64.0] * 4 + [0.0] * 4


def test_sampling_distribution_is_the_reference_rule():
    g = torch.Generator().manual_seed(11)
    h, v = 256, 8000
    hidden = (torch.randn(1, h, generator=g) * 2).bfloat16()
    weight = (torch.randn(v, h, generator=g) * 0.08).bfloat16()
    logits = (hidden.float() @ weight.float().T).reshape(-1)
    top = torch.topk(logits, 6).indices.tolist()
    seen = [top[0], top[2], 17, 4000]
    for kw in [dict(temperature=0.8, top_k=40, top_p=1.0, repetition_penalty=1.0),
               dict(temperature=1.3, top_k=20, top_p=0.9, repetition_penalty=1.0),
               dict(temperature=0.7, top_k=30, top_p=0.95, repetition_penalty=1.3),
               dict(temperature=0.25, top_k=0, top_p=0.6, repetition_penalty=1.0)]:
        idx, probs = decode_ops.sampling_distribution(hidden.to(DEV), weight.to(DEV), seen_token_ids=seen, **kw)
        ref = oracle.reference_sampling_distribution(logits, seen_token_ids=seen, **kw)
        dense = torch.zeros(v)
        ok = idx[0] >= 0
        dense[idx[0][ok].cpu()] = probs[0][ok].cpu()
        assert abs(float(dense.sum()) - 1.0) < 1e-5
        torch.testing.assert_close(dense, ref, rtol=2e-2, atol=2e-4)
    tok = helion_b200.sample_head(hidden.to(DEV), weight.to(DEV), temperature=0.8, top_k=40,
                                  generator=torch.Generator(device=DEV).manual_seed(0))
    assert tok.shape == (1,) and int(tok) in torch.topk(logits, 40).indices.tolist()
    with pytest.raises(ValueError, match="whole vocabulary"):
        helion_b200.sample_head(hidden.to(DEV), weight.to(DEV), top_k=0, top_p=1.0)
    with pytest.raises(ValueError, match="candidates"):
        helion_b200.sample_head(hidden.to(DEV), weight.to(DEV), top_k=60, repetition_penalty=1.2,
                                seen_token_ids=list(range(10)))
