"""Greedy decoding head against the CPU oracle (fp32 logits of the rounded inputs). GPU only."""

from __future__ import annotations

import pytest
import torch

import helion_b200
from oracle import oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DEV = "cuda"


def check(hidden, weight, **kw):
    token, logprob, lse = helion_b200.greedy_head(hidden, weight, return_logsumexp=True, **kw)
    ref = oracle.greedy_expression(hidden.cpu(), weight.cpu())
    assert token.shape == hidden.shape[:-1] and token.dtype == torch.int64
    assert logprob.shape == hidden.shape[:-1] and logprob.dtype == torch.float32
    z = ref["logits"]
    tok = token.cpu().reshape(-1) - kw.get("vocab_start", 0)
    assert int(tok.min()) >= 0 and int(tok.max()) < weight.shape[0]
    picked = z.gather(1, tok[:, None])[:, 0]
    top2 = z.topk(min(2, z.shape[1]), dim=-1).values
    # the chosen logit is the maximum up to the accumulation-order noise of an H-long fp32 dot product ...
    tol = 1e-4 * float(z.abs().max()) + 1e-6
    assert torch.all(picked >= top2[:, 0] - tol)
    # ... and wherever the runner-up is further away than that, the token is THE argmax
    clear = (top2[:, 0] - top2[:, -1] > 4 * tol) if z.shape[1] > 1 else torch.ones_like(tok, dtype=torch.bool)
    assert torch.equal(tok[clear], ref["token"].reshape(-1)[clear])
    torch.testing.assert_close(lse.cpu().reshape(-1), ref["lse"].reshape(-1), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(logprob.cpu().reshape(-1), (picked - ref["lse"].reshape(-1)), rtol=1e-3, atol=2e-4)
    return token, logprob


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [((1,), 64, 1000), ((7,), 256, 5003), ((128,), 512, 32000), ((300,), 768, 50304),
                                   ((2, 5), 128, 777), ((3,), 72, 300), ((16,), 4096, 8192)])
def test_greedy_head_matches_the_oracle(dtype, shape):
    lead, h, v = shape
    hidden = torch.randn(*lead, h, device=DEV, dtype=dtype)
    weight = (torch.randn(v, h, device=DEV) * 0.05).to(dtype)
    check(hidden, weight)


@pytest.mark.parametrize("force", ["tc", "tc1", "simt"])
def test_every_gemm_path(force, monkeypatch):
    monkeypatch.setenv("HELION_B200_FORCE", force)
    hidden = torch.randn(200, 512, device=DEV, dtype=torch.bfloat16)
    weight = (torch.randn(9000, 512, device=DEV) * 0.05).bfloat16()
    check(hidden, weight)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_first_index_wins_on_exact_ties(dtype):
    """Identical weight rows give bit-identical logits (same contraction order in every tile), so the
    maximum is attained several times; torch.argmax and this op both return the first index."""
    h, v = 256, 3000
    weight = (torch.randn(v, h, device=DEV) * 0.02).to(dtype)
    hidden = torch.randn(40, h, device=DEV, dtype=dtype)
    best = (hidden.float() @ weight.float().T).argmax(dim=-1)  # make row i's winner reappear elsewhere
    big = weight[best[0]].clone() * 4  # one row vector that dominates for hidden[0]
    hidden[0] = big.float().sign().to(dtype)
    for idx in (37, 5, 700, 2999, 1290):  # same tile, other tiles, last column
        weight[idx] = big
    token, _ = helion_b200.greedy_head(hidden, weight)
    assert int(token[0]) == 5
    ref = oracle.greedy_expression(hidden.cpu(), weight.cpu())
    assert int(ref["token"][0]) == 5


def test_vocab_start_offsets_the_token_and_matches_the_fused_loss():
    hidden = torch.randn(64, 384, device=DEV, dtype=torch.bfloat16)
    weight = (torch.randn(4100, 384, device=DEV) * 0.05).bfloat16()
    token, logprob = check(hidden, weight)
    shifted, _ = helion_b200.greedy_head(hidden, weight, vocab_start=1000)
    assert torch.equal(shifted, token + 1000)
    # log-probability of the greedy token = minus the per-token loss of the fused op at that token
    nll = helion_b200.linear_cross_entropy(hidden, weight, token, reduction="none")
    torch.testing.assert_close(logprob, -nll, rtol=1e-5, atol=1e-5)


def test_empty_and_rejections():
    w = torch.randn(100, 32, device=DEV)
    token, logprob = helion_b200.greedy_head(torch.empty(0, 32, device=DEV), w)
    assert token.shape == (0,) and logprob.shape == (0,)
    with pytest.raises(ValueError, match="CUDA tensor"):
        helion_b200.greedy_head(torch.randn(2, 32), w)
    with pytest.raises(ValueError, match="Shape mismatch"):
        helion_b200.greedy_head(torch.randn(2, 31, device=DEV), w)
    with pytest.raises(ValueError, match="Dtype mismatch"):
        helion_b200.greedy_head(torch.randn(2, 32, device=DEV, dtype=torch.float16), w)


def test_llama3_head_decode_batch_is_deterministic():
    """Decode-sized batch on the full Llama-3 head (16 x 4096 x 128256 bf16): two runs give the same bits,
    and the tokens are the argmax of fp32 logits computed on the GPU."""
    hidden = torch.randn(16, 4096, device=DEV, dtype=torch.bfloat16)
    weight = (torch.randn(128256, 4096, device=DEV) * 0.02).bfloat16()
    a = helion_b200.greedy_head(hidden, weight)
    b = helion_b200.greedy_head(hidden, weight)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    torch.backends.cuda.matmul.allow_tf32 = False
    z = hidden.float() @ weight.float().T
    top2 = z.topk(2, dim=-1).values
    clear = top2[:, 0] - top2[:, 1] > 1e-3
    assert torch.equal(a[0][clear], z.argmax(dim=-1)[clear])
    torch.testing.assert_close(a[1], torch.log_softmax(z, dim=-1).gather(1, a[0][:, None])[:, 0], rtol=1e-3, atol=1e-3)
