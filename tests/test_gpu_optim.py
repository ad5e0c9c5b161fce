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
