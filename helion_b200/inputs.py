"""Seeded synthetic LM-head workloads: the shapes and value distributions of the five benchmark
configurations (GPT-2-small head, Llama-3-8B head, large-vocab head, 14B-class head, N sweep).

No dataset is involved: activations are Gaussian (optionally rescaled to unit RMS per row), weights
are N(0, 0.02), targets are uniform or Zipf(s=1.1) over a seeded permutation of the vocabulary, and a
fixed fraction of positions carries ``ignore_index``. Everything is drawn on the CPU from one
``torch.Generator`` in the order X, W, targets, ignore mask, then X and W are rounded to ``dtype``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class HeadConfig:
    name: str
    batch: int
    seq: int
    hidden: int
    vocab: int
    target_max: int | None = None  # uniform targets drawn from [0, target_max); default vocab
    zipf: bool = False
    unit_rms: bool = True
    ignore_frac: float = 0.0
    reduction: str = "mean"
    grad_out: float = 1.0
    seed: int = 0

    @property
    def rows(self) -> int:
        return self.batch * self.seq


CONFIGS = {
    # seconds-sized workload for harness self-tests
    "smoke": HeadConfig("smoke", 1, 256, 128, 1000, zipf=True, ignore_frac=0.02),
    # GPT-2-small head; the one case small enough to run in full on the CPU
    "gpt2-small": HeadConfig("gpt2-small", 4, 1024, 768, 50304, target_max=50257, unit_rms=False,
                             ignore_frac=0.01),
    # Llama-3-8B head: the configuration the headline metric is quoted on
    "llama3-8b": HeadConfig("llama3-8b", 1, 8192, 4096, 128256, zipf=True, ignore_frac=0.02),
    # large vocabulary, small hidden size; sharded by vocabulary over 1/2/4/8 GPUs
    "large-vocab": HeadConfig("large-vocab", 2, 8192, 2304, 256000, zipf=True, ignore_frac=0.01),
    # 14B-class head over 8 GPUs (19008 weight rows per rank), sum reduction, upstream grad 1/N
    "14b-class": HeadConfig("14b-class", 8, 8192, 5120, 152064, ignore_frac=0.05, reduction="sum",
                            grad_out=1.0 / 65536),
}


def sweep_config(rows: int) -> HeadConfig:
    """Llama-3-8B head with ``rows`` tokens, uniform targets, nothing ignored (the N sweep)."""
    return HeadConfig(f"sweep-{rows}", 1, rows, 4096, 128256)


def scaled(cfg: HeadConfig, *, rows: int | None = None, hidden: int | None = None,
           vocab: int | None = None) -> HeadConfig:
    """Same distributions on a smaller shape (for parity tests an fp32 CPU run finishes quickly)."""
    rows = cfg.rows if rows is None else rows
    vocab = cfg.vocab if vocab is None else vocab
    tmax = None if cfg.target_max is None else min(cfg.target_max, vocab)
    return HeadConfig(cfg.name + "-scaled", 1, rows, cfg.hidden if hidden is None else hidden, vocab, tmax,
                      cfg.zipf, cfg.unit_rms, cfg.ignore_frac, cfg.reduction, cfg.grad_out, cfg.seed)


def make_inputs(cfg: HeadConfig, dtype: torch.dtype = torch.bfloat16, ignore_index: int = -100,
                chunk_rows: int = 8192) -> dict:
    """Returns ``{"hidden": [B,S,H], "weight": [V,H], "target": [B,S] int64, "grad_out": 0-dim fp32}`` on CPU."""
    g = torch.Generator(device="cpu").manual_seed(cfg.seed)
    n, h, v = cfg.rows, cfg.hidden, cfg.vocab
    x = torch.empty((n, h), dtype=dtype)
    for r0 in range(0, n, chunk_rows):
        blk = torch.randn((min(chunk_rows, n - r0), h), generator=g, dtype=torch.float32)
        if cfg.unit_rms:
            blk = blk / blk.pow(2).mean(dim=1, keepdim=True).sqrt()
        x[r0:r0 + blk.shape[0]] = blk.to(dtype)
    w = torch.empty((v, h), dtype=dtype)
    for r0 in range(0, v, chunk_rows):
        blk = torch.randn((min(chunk_rows, v - r0), h), generator=g, dtype=torch.float32) * 0.02
        w[r0:r0 + blk.shape[0]] = blk.to(dtype)
    if cfg.zipf:
        ranks = torch.arange(1, v + 1, dtype=torch.float64)
        prob = ranks.pow(-1.1)
        drawn = torch.multinomial(prob / prob.sum(), n, replacement=True, generator=g)
        target = torch.randperm(v, generator=g)[drawn]
    else:
        target = torch.randint(0, cfg.target_max or v, (n,), generator=g, dtype=torch.int64)
    n_ignored = int(round(cfg.ignore_frac * n))
    if n_ignored:
        target[torch.randperm(n, generator=g)[:n_ignored]] = ignore_index
    return {
        "hidden": x.view(cfg.batch, cfg.seq, h),
        "weight": w,
        "target": target.view(cfg.batch, cfg.seq),
        "grad_out": torch.tensor(cfg.grad_out, dtype=torch.float32),
        "reduction": cfg.reduction,
        "ignore_index": ignore_index,
    }
