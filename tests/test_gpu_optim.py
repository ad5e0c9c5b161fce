"""AdamW step and gradient-norm kernels: the reference's test restated (tests/tritium/test_adamw.py:11-52:
one step against torch.optim.AdamW), the oracle's restatement over several steps, and the fused clipping
coefficient. GPU only."""

from __future__ import annotations

import pytest
import torch

import helion_b200
from oracle import oracle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DEV = "cuda"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 128, 4096, 100003])
def test_adamw_step_matches_torch_reference(dtype, n):
    lr, betas, eps, wd = 3e-4, (0.9, 0.999), 1e-8, 0.01
    param = torch.randn(n, device=DEV, dtype=dtype)
    grad = torch.randn(n, device=DEV, dtype=dtype)
    exp_avg = torch.zeros(n, device=DEV, dtype=torch.float32)
    exp_avg_sq = torch.zeros(n, device=DEV, dtype=torch.float32)
    ref = torch.optim.AdamW([param.detach().float().clone().requires_grad_(True)], lr=lr, betas=betas, eps=eps,
                            weight_decay=wd)
    ref.param_groups[0]["params"][0].grad = grad.float()
    ref.step()
    helion_b200.adamw_step(param, grad, exp_avg, exp_avg_sq, lr=lr, beta1=betas[0], beta2=betas[1], eps=eps,
                           weight_decay=wd, step=1)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(param.float(), ref.param_groups[0]["params"][0].detach().to(dtype).float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_adamw_steps_follow_the_restated_kernel(dtype):
    g = torch.Generator().manual_seed(3)
    shape = (257, 130)
    p = torch.randn(shape, generator=g).to(dtype)
    m = torch.zeros(shape)
    v = torch.zeros(shape)
    pd, md, vd = p.to(DEV), m.to(DEV), v.to(DEV)
    for step in range(1, 5):
        grad = torch.randn(shape, generator=g).to(dtype)
        ref = oracle.restated_adamw_step(p, grad, m, v, lr=1e-2, weight_decay=0.1, step=step, grad_scale=0.5)
        p, m, v = ref["param"], ref["exp_avg"], ref["exp_avg_sq"]
        helion_b200.adamw_step(pd, grad.to(DEV), md, vd, lr=1e-2, weight_decay=0.1, step=step,
                               grad_scale=torch.tensor(0.5, device=DEV))
        # fp32 moments: equal up to the rounding of a fused multiply-add
        torch.testing.assert_close(md.cpu(), m, rtol=2e-6, atol=1e-7)
        torch.testing.assert_close(vd.cpu(), v, rtol=2e-6, atol=1e-9)
        tol = 1e-6 if dtype == torch.float32 else 8e-3
        torch.testing.assert_close(pd.float().cpu(), p.float(), rtol=tol, atol=tol)


def test_adamw_validation_messages():
    p = torch.randn(8, device=DEV)
    with pytest.raises(ValueError, match="CUDA tensor"):
        helion_b200.adamw_step(p.cpu(), p.cpu(), p.cpu(), p.cpu(), lr=1e-3)
    with pytest.raises(ValueError, match="Shape mismatch: param"):
        helion_b200.adamw_step(p, p[:4], p.clone(), p.clone(), lr=1e-3)
    with pytest.raises(ValueError, match="exp_avg must have dtype float32"):
        helion_b200.adamw_step(p.half(), p.half(), p.half(), p.clone(), lr=1e-3)
    with pytest.raises(ValueError, match="contiguous for tritium.adamw_step"):
        helion_b200.adamw_step(torch.randn(4, 4, device=DEV).t(), torch.randn(4, 4, device=DEV), torch.zeros(4, 4, device=DEV),
                               torch.zeros(4, 4, device=DEV), lr=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gradient_norm_is_deterministic_and_clipping_fuses_into_the_step(dtype):
    g = torch.Generator().manual_seed(4)
    params = [torch.nn.Parameter(torch.randn(s, generator=g).to(dtype).to(DEV)) for s in [(1000, 300), (7,), (128256 // 8, 64)]]
    for prm in params:
        prm.grad = (torch.randn(prm.shape, generator=g) * 3).to(dtype).to(DEV)
    ref_norm = torch.norm(torch.stack([q.grad.norm(dtype=torch.float32) for q in params]))
    norm, coef = helion_b200.clip_grad_norm(params, max_norm=1.0)
    norm2, _ = helion_b200.clip_grad_norm(params, max_norm=1.0)
    assert torch.equal(norm, norm2)  # fixed summation order
    torch.testing.assert_close(norm, ref_norm, rtol=1e-5, atol=0)
    torch.testing.assert_close(coef, (1.0 / (ref_norm + 1e-6)).clamp(max=1.0), rtol=1e-5, atol=0)
    # clipped step through the fused coefficient == reference order: rescale the gradient, then step
    prm = params[0]
    m1, v1 = torch.zeros_like(prm, dtype=torch.float32), torch.zeros_like(prm, dtype=torch.float32)
    m2, v2 = m1.clone(), v1.clone()
    a, b = prm.detach().clone(), prm.detach().clone()
    helion_b200.adamw_step(a, prm.grad, m1, v1, lr=1e-2, grad_scale=coef)
    helion_b200.adamw_step(b, (prm.grad.float() * coef).to(dtype), m2, v2, lr=1e-2)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    torch.testing.assert_close(a.float(), b.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("force", ["tc", "tc1", "simt"])
@pytest.mark.parametrize("shape,block", [((300, 128, 1500), 0),        # one block, dW stored directly
                                         ((1200, 256, 2100), 1_300_000),  # vocabulary bands
                                         ((2100, 256, 1200), 1_100_000),  # row chunks: dW summed over chunks in fp32
                                         ((4096, 256, 65), 0)])           # short vocabulary: dW contraction split
def test_gradient_norm_from_the_dw_epilogue(shape, block, force, monkeypatch):
    """The sum of squares the dW GEMM adds up while storing equals a separate pass over the stored gradient
    (``lce_sumsq``; fp32 sums in two different fixed orders) and the float64 sum, is bit-identical from run to
    run, and is what ``clip_grad_norm`` uses for the head - as helion.clip_grad_norm (helion/training.py:36-49
    of the reference) would compute from the gradient."""
    from helion_b200 import _lib, grad_norm, ops, optim_ops

    monkeypatch.setenv("HELION_B200_FORCE", force)
    monkeypatch.setenv("HELION_B200_BLOCK_BYTES", str(block))
    n, h, v = shape
    g = torch.Generator().manual_seed(n + v)
    x = torch.randn(n, h, generator=g).bfloat16().to(DEV).requires_grad_(True)
    w = (torch.randn(v, h, generator=g) * 0.1).bfloat16().to(DEV).requires_grad_(True)
    t = torch.randint(0, v, (n,), generator=g).to(DEV)
    grad_norm.enable(True)
    try:
        sums = []
        for _ in range(2):
            x.grad = w.grad = None
            ops.linear_cross_entropy(x, w, t).backward(torch.tensor(37.0, device=DEV))
            fused = grad_norm.lookup(w.grad)
            assert fused is not None, "autograd handed the gradient over without a copy; its sum must be found"
            sums.append(fused.clone())
        assert torch.equal(sums[0], sums[1])
        launches = _lib.lib().lce_launch_count()
        via_registry = optim_ops.grad_sumsq([w.grad])
        assert _lib.lib().lce_launch_count() == launches, "the head's gradient must not be read again"
        assert torch.equal(via_registry, sums[0])
        exact = float(w.grad.double().pow(2).sum())
        assert abs(float(sums[0]) - exact) <= 1e-5 * exact
        grad_norm.enable(False)
        separate = optim_ops.grad_sumsq([w.grad])
        assert _lib.lib().lce_launch_count() > launches
        assert abs(float(separate) - float(sums[0])) <= 2e-6 * exact
        # a gradient that was written after the backward no longer matches its remembered sum
        grad_norm.enable(True)
        x.grad = w.grad = None
        ops.linear_cross_entropy(x, w, t).backward()
        w.grad.mul_(2.0)
        assert grad_norm.lookup(w.grad) is None
        norm, coef = helion_b200.clip_grad_norm([x, w], 1.0)
        ref = torch.sqrt(x.grad.double().pow(2).sum() + w.grad.double().pow(2).sum())
        assert abs(float(norm) - float(ref)) <= 1e-5 * float(ref)
    finally:
        grad_norm.enable(False)
