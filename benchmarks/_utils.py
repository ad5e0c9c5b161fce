"""Timing helpers for the benchmark harness: the reference's conventions (``benchmarks/_utils.py:14-23`` of
the reference: median of ``TRITIUM_BENCH_REPEATS`` runs of ``triton.testing.do_bench``) restated with CUDA
events so that nothing here depends on Triton."""

from __future__ import annotations

import os
import statistics

import torch


def bench_repeats() -> int:
    return int(os.environ.get("TRITIUM_BENCH_REPEATS", "5"))


def do_bench(fn, warmup_ms: float = 25.0, rep_ms: float = 100.0) -> float:
    """Mean device time of ``fn`` in ms. Like ``triton.testing.do_bench``: the run count comes from a
    time budget, and a 256 MB buffer is overwritten before every timed run so each run starts with a
    cold L2 (``HELION_BENCH_FLUSH=0`` shrinks that write to 4 bytes: same launches, L2 left as the previous
    run left it)."""
    fn()
    torch.cuda.synchronize()
    flush = os.environ.get("HELION_BENCH_FLUSH", "1") != "0"
    cache = torch.empty((256 << 20) if flush else 4, dtype=torch.int8, device="cuda")
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(5):
        cache.zero_()
        fn()
    end.record()
    torch.cuda.synchronize()
    estimate = start.elapsed_time(end) / 5
    n_warmup = max(1, int(warmup_ms / estimate))
    n_repeat = max(1, int(rep_ms / estimate))
    for _ in range(n_warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return statistics.fmean(s.elapsed_time(e) for s, e in zip(starts, ends))


def bench_ms(fn, repeats: int | None = None) -> float:
    repeats = bench_repeats() if repeats is None else repeats
    torch.cuda.synchronize()
    return statistics.median(do_bench(fn) for _ in range(repeats))


def loop_ms(fn, calls: int = 300) -> float:
    """Wall time per call of ``calls`` back-to-back calls (one synchronise at the end), in ms: what a training
    loop pays per call, host time included. For launch-bound shapes this, not the device time between two
    events, is the throughput-relevant figure."""
    import time

    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(calls):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / calls * 1e3


def tflops(flops: float, ms: float) -> float:
    return flops / (ms * 1e-3) / 1e12


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required to run benchmarks.")
