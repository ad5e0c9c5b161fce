"""A Helion training loop with the op swapped in: the UNMODIFIED reference packages (helion modules,
helion.optim.AdamW, tritium ops) train a small language model whose loss is
``tritium.linear_cross_entropy(hidden, lm_head, targets)`` - the call of the reference's
TinyLanguageModel (examples/common.py:123-125) - once with the reference's Triton op and once after
``helion_b200.install()``. Same seed, same data: the two loss curves must agree step by step.
Needs the reference installed under baseline/_ref and a GPU; skipped otherwise."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _train(steps: int, dtype: torch.dtype, use_ours: bool) -> tuple[list[float], int]:
    import helion
    import tritium

    import helion_b200
    from helion_b200 import _lib

    torch.manual_seed(0)
    vocab, hidden, batch, seq = 1000, 128, 8, 64

    class TinyLM(nn.Module):  # embedding -> two helion Linear layers with SwiGLU-free GELU-free mixing -> LM head
        def __init__(self):
            super().__init__()
            self.embed = helion.Embedding(vocab, hidden)
            self.up = helion.Linear(hidden, 2 * hidden, bias=False)
            self.down = helion.Linear(2 * hidden, hidden, bias=False)
            self.norm = helion.RMSNorm(hidden)
            self.lm_head = nn.Parameter(torch.empty(vocab, hidden))
            nn.init.normal_(self.lm_head, std=0.02)

        def forward(self, tokens, targets):
            x = self.embed(tokens)
            x = x + self.down(torch.tanh(self.up(x)))
            hidden_states = self.norm(x)
            return tritium.linear_cross_entropy(hidden_states.contiguous(), self.lm_head, targets)

    model = TinyLM().to("cuda").to(dtype)
    opt = helion.AdamW(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, vocab, (steps, batch, seq), generator=g).cuda()
    targets = (tokens * 7 + 3) % vocab  # a function of the current token: learnable within a few steps
    if use_ours:
        helion_b200.install()
    launches = _lib.lib().lce_launch_count()
    losses = []
    try:
        for i in range(steps):
            opt.zero_grad()
            loss = model(tokens[i], targets[i])
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
    finally:
        if use_ours:
            helion_b200.uninstall()
    return losses, _lib.lib().lce_launch_count() - launches


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_training_curve_matches_the_reference_op(dtype):
    if not (REF / "tritium").exists() or not (REF / "helion").exists():
        pytest.skip("reference not installed under baseline/_ref")
    sys.path.insert(0, str(REF))
    try:
        ref_losses, ref_launches = _train(30, dtype, use_ours=False)
        our_losses, our_launches = _train(30, dtype, use_ours=True)
    finally:
        sys.path.remove(str(REF))
    assert ref_launches == 0 and our_launches > 0  # the second run really went through libhelion_lce.so
    assert our_losses[-1] < our_losses[0]  # it trains
    # two trainings diverge slowly as rounding differences feed back through the optimizer: tight at the
    # start, looser at the end
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-4
    for i, (a, b) in enumerate(zip(our_losses, ref_losses)):
        assert abs(a - b) <= tol * (1 + i) * abs(b), (i, our_losses, ref_losses)
