"""CPU oracle for the fused linear-cross-entropy path. TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this module: only tests/, __graft_entry__.smoke() and the CPU-baseline
legs of bench.py may call it, and only as the checker or the timed CPU baseline. The product path
(helion_b200) has no CPU route and fails loudly without its CUDA library.

Two layers:

1. ``expression`` / ``expression_chunked`` - the ground truth the reference itself tests and benchmarks
   against: ``F.cross_entropy(F.linear(hidden, weight).float(), target)`` evaluated in fp32 on inputs that
   were first rounded to the working dtype (reference ``tests/tritium/test_cross_entropy.py:72, 91-93,
   106-108``; ``benchmarks/bench_linear_cross_entropy.py:34-39``). The reference has no CPU
   implementation of the op (CPU tensors are rejected, ``tritium/ops/_utils.py:25-27``), so this
   expression is also the reference's CPU path for timing purposes.
2. ``restated_forward`` / ``restated_backward`` - a plain restatement of the algorithm the reference's
   kernels run (block-partial softmax statistics merged per row; chunked recompute backward), following
   ``tritium/ops/cross_entropy.py`` line by line, including where it rounds to the input dtype.

Pinning: the reference ships no golden vectors for this path. The restatement is pinned against outputs
of the reference's own Triton kernels, produced on a B200 by tests/golden/make_golden.py and committed
under tests/golden/ (forward and the small-shape fused backward). The reference's large-shape backward
(cuBLAS chunk loop, ``cross_entropy.py:927-957``) has no test in the reference; fixtures from a run of
it are committed as well, and where none exists for a shape that branch is "parity unpinned" and
``expression`` stands in.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

REFERENCE_BLOCK_V = 128              # LINEAR_CE_BLOCK_V, tritium/ops/cross_entropy.py:24
REFERENCE_DIRECT_MAX_VOCAB = 256     # LINEAR_CE_DIRECT_MAX_VOCAB, :25
REFERENCE_MAX_LOGIT_ELEMENTS = 67_108_864  # LINEAR_CE_BACKWARD_MAX_LOGIT_ELEMENTS, :22


# ----------------------------------------------------------------------------------------------
# 1. the ground-truth expression
# ----------------------------------------------------------------------------------------------
def expression(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, *, reduction: str = "mean",
               ignore_index: int = -100, grad_out: torch.Tensor | None = None, want_grads: bool = True) -> dict:
    """fp32 ``F.cross_entropy(F.linear(h, w), t)`` and its autograd gradients (tests :88-95)."""
    h32 = hidden.detach().float().reshape(-1, hidden.shape[-1]).clone().requires_grad_(want_grads)
    w32 = weight.detach().float().clone().requires_grad_(want_grads)
    t = target.reshape(-1).long()
    logits = F.linear(h32, w32)
    loss = F.cross_entropy(logits, t, ignore_index=ignore_index, reduction=reduction)
    out = {"loss": loss.detach().reshape(target.shape if reduction == "none" else ()),
           "lse": torch.logsumexp(logits.detach(), dim=-1)}
    if want_grads:
        if grad_out is None:
            grad_out = torch.ones_like(loss)
        loss.backward(grad_out.detach().float().reshape(loss.shape))
        out["dx"] = h32.grad
        out["dw"] = w32.grad
    return out


def expression_chunked(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, *,
                       reduction: str = "mean", ignore_index: int = -100, grad_out: torch.Tensor | None = None,
                       want_grads: bool = True, chunk_rows: int = 1024) -> dict:
    """Same numbers as ``expression`` with O(chunk_rows x V) memory (for shapes whose logits do not fit)."""
    h32 = hidden.detach().float().reshape(-1, hidden.shape[-1])
    w32 = weight.detach().float()
    t = target.reshape(-1).long()
    n = h32.shape[0]
    valid = t != ignore_index
    count = valid.sum().to(torch.float32)
    lse = torch.empty(n, dtype=torch.float32, device=h32.device)
    nll = torch.zeros(n, dtype=torch.float32, device=h32.device)
    if grad_out is None:
        grad_out = torch.ones(n if reduction == "none" else (), dtype=torch.float32, device=h32.device)
    go = grad_out.detach().float().to(h32.device)
    if reduction == "none":
        scale = go.reshape(-1)
    elif reduction == "sum":
        scale = go.expand(n)
    else:
        scale = (go / count).expand(n)
    scale = torch.where(valid, scale, torch.zeros_like(scale))
    dx = torch.empty_like(h32) if want_grads else None
    dw = torch.zeros_like(w32) if want_grads else None
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        z = h32[r0:r1] @ w32.T
        l = torch.logsumexp(z, dim=-1)
        lse[r0:r1] = l
        tc = t[r0:r1]
        vc = valid[r0:r1]
        safe = torch.where(vc, tc, torch.zeros_like(tc))
        nll[r0:r1] = torch.where(vc, l - z.gather(1, safe[:, None])[:, 0], torch.zeros_like(l))
        if want_grads:
            g = torch.exp(z - l[:, None])
            g[torch.arange(r1 - r0, device=g.device)[vc], safe[vc]] -= 1.0
            g *= scale[r0:r1, None]
            dx[r0:r1] = g @ w32
            dw += g.T @ h32[r0:r1]
    if reduction == "none":
        loss = nll.reshape(target.shape)
    elif reduction == "sum":
        loss = nll.sum()
    else:
        loss = nll.sum() / count
    out = {"loss": loss, "lse": lse}
    if want_grads:
        out["dx"], out["dw"] = dx, dw
    return out


# ----------------------------------------------------------------------------------------------
# 2. restatement of the reference's algorithm
# ----------------------------------------------------------------------------------------------
def restated_forward(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor) -> dict:
    """What the reference's forward kernels compute (tritium/ops/cross_entropy.py:563-640).

    Logits are accumulated in fp32 from the working-dtype inputs (:220-233). For V <= 256 one block
    holds the whole row (:134-189); otherwise each 128-wide vocab block yields (max, sum exp(z - max),
    target logit or -inf) (:235-248) and a second pass merges the blocks per row (:251-293). The loss is
    the mean over ALL rows (divisor n_rows, :189, :293); there is no ignored label, so a target no
    column matches leaves target_logit = -inf and an infinite loss.
    """
    h32 = hidden.detach().float().reshape(-1, hidden.shape[-1])
    w32 = weight.detach().float()
    t = target.reshape(-1).long()
    n, v = h32.shape[0], w32.shape[0]
    z = h32 @ w32.T
    cols = torch.arange(v)
    if v <= REFERENCE_DIRECT_MAX_VOCAB:
        row_max = z.max(dim=1).values
        lse = torch.log(torch.exp(z - row_max[:, None]).sum(dim=1)) + row_max
        tlogit = torch.where(cols[None, :] == t[:, None], z, torch.full_like(z, -math.inf)).max(dim=1).values
    else:
        pm, ps, pt = [], [], []
        for b0 in range(0, v, REFERENCE_BLOCK_V):
            zb = z[:, b0:b0 + REFERENCE_BLOCK_V]
            bm = zb.max(dim=1).values
            pm.append(bm)
            ps.append(torch.exp(zb - bm[:, None]).sum(dim=1))
            hit = cols[None, b0:b0 + REFERENCE_BLOCK_V] == t[:, None]
            pt.append(torch.where(hit, zb, torch.full_like(zb, -math.inf)).max(dim=1).values)
        pm, ps, pt = torch.stack(pm), torch.stack(ps), torch.stack(pt)
        row_max = pm.max(dim=0).values
        lse = torch.log((ps * torch.exp(pm - row_max[None, :])).sum(dim=0)) + row_max
        tlogit = pt.max(dim=0).values
    nll = lse - tlogit
    return {"loss": nll.sum() / n if n != 1 else nll.sum(), "lse": lse}


def restated_backward(grad_out: torch.Tensor, hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor,
                      lse: torch.Tensor) -> dict:
    """What linear_cross_entropy_backward computes (tritium/ops/cross_entropy.py:863-959).

    Small shapes (H <= 64, V >= 256, N*V <= 65536; :522-531) run the fused kernel: fp32 logits,
    G = (exp(z - lse) - onehot) * grad_out / n_rows rounded to the input dtype, dX and dW summed in fp32
    and rounded once (:335-381, :860). Larger shapes run a row-chunk loop (:927-957): logits rounded to
    the input dtype by F.linear (:937), G formed from those rounded logits and stored in the input dtype
    (:103-131), dX = G @ W per chunk (:945), dW accumulated across chunks in the weight dtype (:947-957).
    """
    dt = hidden.dtype
    h = hidden.detach().reshape(-1, hidden.shape[-1])
    w = weight.detach()
    t = target.reshape(-1).long()
    n, hsz = h.shape
    v = w.shape[0]
    go = grad_out.detach().float().reshape(())
    rows = torch.arange(n)
    if hsz <= 64 and v >= 256 and n * v <= 65_536:
        z = h.float() @ w.float().T
        g = torch.exp(z - lse[:, None])
        g[rows, t] -= 1.0
        g = (g * (go / n)).to(dt).float()
        return {"dx": (g @ w.float()).to(dt), "dw": (g.T @ h.float()).to(dt)}
    chunk = min(n, max(1, REFERENCE_MAX_LOGIT_ELEMENTS // v))
    dx = torch.empty_like(h)
    dw = torch.zeros_like(w)
    first = True
    for r0 in range(0, n, chunk):
        r1 = min(n, r0 + chunk)
        z = (h[r0:r1].float() @ w.float().T).to(dt).float()
        g = torch.exp(z - lse[r0:r1, None])
        g[torch.arange(r1 - r0), t[r0:r1]] -= 1.0
        g = (g * (go / n)).to(dt).float()
        dx[r0:r1] = (g @ w.float()).to(dt)
        part = g.T @ h[r0:r1].float()
        dw = part.to(dt) if first else (dw.float() + part).to(dt)
        first = False
    return {"dx": dx, "dw": dw}


# ----------------------------------------------------------------------------------------------
# the plain op on materialised logits (same reference file)
# ----------------------------------------------------------------------------------------------
def plain_expression(logits: torch.Tensor, target: torch.Tensor, *, reduction: str = "mean",
                     ignore_index: int = -100, grad_out: torch.Tensor | None = None, want_grads: bool = True) -> dict:
    """``F.cross_entropy(logits.float(), target)`` and its gradient: what the reference's tests compare
    ``tritium.cross_entropy`` against (tests/tritium/test_cross_entropy.py:24-25, 40-42, 54-56)."""
    z = logits.detach().float().clone().requires_grad_(want_grads)
    loss = F.cross_entropy(z, target.long(), ignore_index=ignore_index, reduction=reduction)
    out = {"loss": loss.detach(), "lse": torch.logsumexp(z.detach(), dim=-1)}
    if want_grads:
        loss.backward(torch.ones_like(loss) if grad_out is None else grad_out.detach().float().reshape(loss.shape))
        out["dlogits"] = z.grad
    return out


def restated_plain_forward(logits: torch.Tensor, target: torch.Tensor) -> dict:
    """The reference's row kernel (tritium/ops/cross_entropy.py:36-68): fp32 row max, sum of
    exp(z - max), lse = log(sum) + max, nll = lse - z[target]; mean over ALL rows (:66-68)."""
    z = logits.detach().float()
    n = z.shape[0]
    row_max = z.max(dim=1).values
    lse = torch.log(torch.exp(z - row_max[:, None]).sum(dim=1)) + row_max
    nll = lse - z.gather(1, target.long()[:, None])[:, 0]
    return {"loss": nll.sum() if n == 1 else (nll / n).sum(), "lse": lse}


def restated_plain_backward(grad_out: torch.Tensor, logits: torch.Tensor, target: torch.Tensor,
                            lse: torch.Tensor) -> torch.Tensor:
    """The reference's backward row kernel (:71-100): (exp(z - lse) - onehot) * grad_out / n_rows, computed
    in fp32 and stored in the logits dtype."""
    z = logits.detach().float()
    n = z.shape[0]
    g = torch.exp(z - lse[:, None])
    g[torch.arange(n), target.long()] -= 1.0
    return (g * (grad_out.detach().float().reshape(()) / n)).to(logits.dtype)


# ----------------------------------------------------------------------------------------------
# consumers of dW
# ----------------------------------------------------------------------------------------------
def restated_adamw_step(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, *,
                        lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                        weight_decay: float = 0.01, step: int = 1, grad_scale: float = 1.0) -> dict:
    """The reference's AdamW kernel (tritium/ops/adamw.py:36-54) in fp32 torch: returns the new
    (param in its dtype, exp_avg, exp_avg_sq)."""
    p = param.detach().float()
    g = grad.detach().float() * grad_scale
    # the kernel receives beta1 / beta2 as fp32 arguments and forms (1 - beta) in fp32 (:46-47)
    b1 = torch.tensor(beta1, dtype=torch.float32)
    b2 = torch.tensor(beta2, dtype=torch.float32)
    m = b1 * exp_avg.detach().float() + (1.0 - b1) * g
    v = b2 * exp_avg_sq.detach().float() + (1.0 - b2) * g * g
    p = p - lr * weight_decay * p
    denom = torch.sqrt(v / (1.0 - beta2 ** step)) + eps
    p = p - (lr / (1.0 - beta1 ** step)) * m / denom
    return {"param": p.to(param.dtype), "exp_avg": m, "exp_avg_sq": v}


# ----------------------------------------------------------------------------------------------
# greedy decoding head
# ----------------------------------------------------------------------------------------------
def greedy_expression(hidden: torch.Tensor, weight: torch.Tensor) -> dict:
    """What the reference's decode step computes before sampling (examples/common.py:127-131: logits =
    hidden @ lm_head.T), reduced the greedy way: fp32 logits of the dtype-rounded inputs, their argmax
    (first index on ties, as torch.argmax), log_softmax at it, and the logsumexp."""
    z = hidden.detach().float().reshape(-1, hidden.shape[-1]) @ weight.detach().float().T
    lse = torch.logsumexp(z, dim=-1)
    token = z.argmax(dim=-1)
    top = z.gather(1, token[:, None])[:, 0]
    shape = hidden.shape[:-1]
    return {"token": token.reshape(shape), "logprob": (top - lse).reshape(shape), "lse": lse.reshape(shape),
            "logits": z}


# ----------------------------------------------------------------------------------------------
# producer of the hidden states: RMSNorm / residual RMSNorm
# ----------------------------------------------------------------------------------------------
def restated_rmsnorm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                             residual: torch.Tensor | None = None) -> dict:
    """The reference's forward kernels (tritium/ops/rmsnorm.py:29-84) in fp32 torch: the sum is
    formed in fp32 (float64 here, rounded once, so the restatement does not depend on a summation
    order), the outputs are rounded to the input dtype. With ``residual`` the normalised value is
    the UNROUNDED fp32 sum z = x + residual (:76-81); ``residual_out`` is z rounded."""
    z = x.detach().float()
    if residual is not None:
        z = z + residual.detach().float()
    mean_sq = (z.double() * z.double()).mean(dim=-1, keepdim=True).float()
    rstd = 1.0 / torch.sqrt(mean_sq + torch.tensor(eps, dtype=torch.float32))
    out = (z * rstd * weight.detach().float()).to(x.dtype)
    res = {"out": out, "rstd": rstd.reshape(-1)}
    if residual is not None:
        res["residual_out"] = z.to(x.dtype)
    return res


def restated_rmsnorm_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                              rstd: torch.Tensor | None = None, dresidual: torch.Tensor | None = None) -> dict:
    """The reference's backward (tritium/ops/rmsnorm.py:105-130, :225-280): dx per row from the saved
    (or recomputed, :163-191) rstd, dweight = sum over rows of dy * x * rstd in fp32, both rounded to
    the input dtype. ``dresidual`` is added the way the residual autograd function adds it (:728):
    onto the already rounded dx, in the input dtype."""
    h = x.shape[-1]
    xf = x.detach().float().reshape(-1, h)
    dyf = dy.detach().float().reshape(-1, h)
    wf = weight.detach().float()
    if rstd is None:
        mean_sq = (xf.double() * xf.double()).mean(dim=-1, keepdim=True).float()
        r = 1.0 / torch.sqrt(mean_sq + torch.tensor(eps, dtype=torch.float32))
    else:
        r = rstd.detach().float().reshape(-1, 1)
    weighted = dyf * wf
    c = (weighted.double() * xf.double()).sum(dim=-1, keepdim=True).float()
    dx = (r * weighted - (r * r * r / h) * xf * c).to(x.dtype)
    if dresidual is not None:
        dx = dx + dresidual.detach().reshape(-1, h).to(x.dtype)
    dweight = (dyf.double() * xf.double() * r.double()).sum(dim=0).float().to(weight.dtype)
    return {"dx": dx.reshape(x.shape), "dweight": dweight}


def rmsnorm_expression(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                       residual: torch.Tensor | None = None, *, dy: torch.Tensor | None = None,
                       dresidual_out: torch.Tensor | None = None) -> dict:
    """What the op MEANS, through torch autograd in float64: out = z * rsqrt(mean(z^2) + eps) * w with
    z = x (+ residual), and the gradients of sum(out * dy) (+ sum(z * dresidual_out))."""
    xd = x.detach().double().requires_grad_(dy is not None)
    wd = weight.detach().double().requires_grad_(dy is not None)
    z = xd if residual is None else xd + residual.detach().double()
    out = z * torch.rsqrt((z * z).mean(dim=-1, keepdim=True) + eps) * wd
    res = {"out": out.detach(), "z": z.detach()}
    if dy is not None:
        obj = (out * dy.detach().double()).sum()
        if dresidual_out is not None:
            obj = obj + (z * dresidual_out.detach().double()).sum()
        obj.backward()
        res["dx"], res["dweight"] = xd.grad, wd.grad
    return res


# ----------------------------------------------------------------------------------------------
# vocabulary sharding algebra (what each rank contributes and how the merge must come out)
# ----------------------------------------------------------------------------------------------
def shard_stats(hidden: torch.Tensor, weight_shard: torch.Tensor, target: torch.Tensor, vocab_start: int) -> torch.Tensor:
    """``[3, N]`` fp32: (max, sum exp(z - max), target logit or -inf) over one contiguous vocab shard."""
    h32 = hidden.detach().float().reshape(-1, hidden.shape[-1])
    z = h32 @ weight_shard.detach().float().T
    t = target.reshape(-1).long() - vocab_start
    m = z.max(dim=1).values
    s = torch.exp(z - m[:, None]).sum(dim=1)
    inside = (t >= 0) & (t < z.shape[1])
    safe = torch.where(inside, t, torch.zeros_like(t))
    tl = torch.where(inside, z.gather(1, safe[:, None])[:, 0], torch.full_like(m, -math.inf))
    return torch.stack([m, s, tl])


def merge_stats(stats: torch.Tensor, target: torch.Tensor, *, reduction: str = "mean", ignore_index: int = -100) -> dict:
    """Merge ``[R, 3, N]`` shard statistics into the global loss and logsumexp."""
    m = stats[:, 0].max(dim=0).values
    s = (stats[:, 1] * torch.exp(stats[:, 0] - m[None, :])).sum(dim=0)
    lse = m + torch.log(s)
    tl = stats[:, 2].max(dim=0).values
    t = target.reshape(-1)
    valid = t != ignore_index
    nll = torch.where(valid, lse - tl, torch.zeros_like(lse))
    if reduction == "none":
        loss = nll.reshape(target.shape)
    elif reduction == "sum":
        loss = nll.sum()
    else:
        loss = nll.sum() / valid.sum()
    return {"loss": loss, "lse": lse}


def shard_backward_chunked(hidden: torch.Tensor, weight_shard: torch.Tensor, target: torch.Tensor, vocab_start: int,
                           lse: torch.Tensor, scale: torch.Tensor, chunk_rows: int = 1024) -> dict:
    """What ONE rank of a vocabulary-parallel backward contributes, in fp32 with O(chunk_rows x V_local) memory:
    ``G = (exp(z_local - lse_global) - onehot) * scale`` over the shard's columns, the partial ``dx = G @ W_r``
    (to be summed over ranks) and the local ``dw = G^T @ X``. ``scale`` is the per-row factor (0 for ignored
    rows). Also returns the shard's ``[3, N]`` statistics as ``shard_stats`` defines them."""
    h32 = hidden.detach().float().reshape(-1, hidden.shape[-1])
    w32 = weight_shard.detach().float()
    t = target.reshape(-1).long() - vocab_start
    n = h32.shape[0]
    dx = torch.empty_like(h32)
    dw = torch.zeros_like(w32)
    stats = torch.empty((3, n), dtype=torch.float32, device=h32.device)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        z = h32[r0:r1] @ w32.T
        tc = t[r0:r1]
        inside = (tc >= 0) & (tc < z.shape[1])
        safe = torch.where(inside, tc, torch.zeros_like(tc))
        m = z.max(dim=1).values
        stats[0, r0:r1] = m
        stats[1, r0:r1] = torch.exp(z - m[:, None]).sum(dim=1)
        stats[2, r0:r1] = torch.where(inside, z.gather(1, safe[:, None])[:, 0], torch.full_like(m, -math.inf))
        g = torch.exp(z - lse[r0:r1, None].float())
        g[torch.arange(r1 - r0, device=g.device)[inside], safe[inside]] -= 1.0
        g *= scale[r0:r1, None].float()
        dx[r0:r1] = g @ w32
        dw += g.T @ h32[r0:r1]
    return {"dx": dx, "dw": dw, "stats": stats}


def topk_expression(hidden: torch.Tensor, weight: torch.Tensor, k: int, temperature: float = 1.0) -> dict:
    """Ground truth of the sampling head: the ``k`` largest of ``hidden @ weight.T / temperature`` in fp32 (largest
    first, lower index first among equal values), their indices, and the logsumexp of the scaled logits - what the
    reference's decode step obtains from materialised logits with ``torch.topk`` (examples/common.py:288-289)."""
    y = (hidden.detach().float().reshape(-1, hidden.shape[-1]) @ weight.detach().float().T) / temperature
    order = torch.sort(y, dim=1, descending=True, stable=True).indices[:, :k]
    shape = tuple(hidden.shape[:-1])
    return {"values": y.gather(1, order).reshape(shape + (order.shape[1],)),
            "indices": order.reshape(shape + (order.shape[1],)),
            "lse": torch.logsumexp(y, dim=1).reshape(shape), "logits": y}


def reference_sampling_distribution(logits: torch.Tensor, *, temperature: float, top_k: int, top_p: float,
                                    repetition_penalty: float, seen_token_ids) -> torch.Tensor:
    """The probability vector the reference's ``sample_next_token`` draws from (examples/common.py:263-306),
    restated for one row of unscaled fp32 logits: repetition penalty, temperature, top-k mask, nucleus mask,
    softmax. Everything up to (not including) its ``torch.multinomial`` call."""
    z = logits.float().reshape(-1).clone()
    if repetition_penalty != 1.0 and seen_token_ids:
        ids = torch.tensor(sorted(set(int(i) for i in seen_token_ids)), device=z.device)
        sel = z[ids]
        z[ids] = torch.where(sel < 0, sel * repetition_penalty, sel / repetition_penalty)
    z = z / temperature
    if 0 < top_k < z.numel():
        threshold = torch.topk(z, top_k).values[-1]
        z = z.masked_fill(z < threshold, -math.inf)
    if top_p < 1.0:
        sorted_z, sorted_i = torch.sort(z, descending=True)
        cumulative = torch.softmax(sorted_z, dim=-1).cumsum(dim=-1)
        remove = cumulative > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        z = z.scatter(0, sorted_i[remove], torch.full_like(sorted_z[remove], -math.inf))
    return torch.softmax(z, dim=-1)
