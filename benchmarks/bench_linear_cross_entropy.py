"""Forward and backward timings of the fused linear-cross-entropy, Triton-free.

Restates the reference's harness (``benchmarks/bench_linear_cross_entropy.py`` of the reference): the same
seven (n_rows, hidden, vocab) shapes with fp16 ``randn`` inputs (std-1 weights), forward timed as the op on
non-grad tensors, backward timed as a direct call of ``linear_cross_entropy_backward`` with a precomputed
logsumexp, median of ``TRITIUM_BENCH_REPEATS`` x a do_bench-style mean. Added: the benchmark head
configurations in bf16, forward+backward through autograd, tokens/s, TFLOP/s and the fraction of the
measured bf16 tensor peak (2 N H V FLOPs forward, 6 N H V backward).

Providers: ``helion_b200`` (this repository), ``torch_eager`` (F.linear + F.cross_entropy on the GPU, where
the logits fit), ``tritium`` (the reference's own Triton/cuBLAS op, only if a copy is installed under
baseline/_ref). One JSON object per line on stdout.

    python -m benchmarks.bench_linear_cross_entropy [--configs] [--shapes] [--sweep] [--fp32] [--providers a,b]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import helion_b200  # noqa: E402
from benchmarks._utils import bench_ms, loop_ms, require_cuda, tflops  # noqa: E402
from helion_b200 import inputs  # noqa: E402

# (n_rows, hidden_size, vocab_size), as in the reference harness (its lines 23-31)
SHAPES = [
    (16, 512, 1024),
    (128, 512, 1024),
    (128, 1024, 8192),
    (128, 2048, 32768),
    (512, 4096, 32000),
    (512, 4096, 128256),
    (1024, 4096, 32000),
]
FP32_SHAPES = [(512, 1024, 8192), (2048, 1024, 32768), (4096, 2048, 32000)]  # CUDA-core path (no TF32)
CONFIG_NAMES = ["gpt2-small", "llama3-8b", "large-vocab"]
SWEEP_ROWS = [1024, 4096, 16384, 65536]


def _peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    return json.loads(path.read_text())["bf16_tflops"] if path.exists() else 1590.0


def _torch_linear_cross_entropy(hidden, weight, target):
    return F.cross_entropy(F.linear(hidden, weight).float().view(-1, weight.shape[0]), target.view(-1))


def _reference_module():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "tritium").exists():
        return None
    sys.path.insert(0, str(ref))
    try:
        import tritium

        return tritium
    except Exception:  # noqa: BLE001 - optional provider
        return None


def time_case(label: str, hidden, weight, target, providers, peak: float, eager_limit: int = 1 << 33) -> None:
    n = target.numel()
    h, v = weight.shape[1], weight.shape[0]
    grad_out = torch.tensor(1.0, device="cuda")
    nhv = float(n) * h * v
    tritium = _reference_module() if "tritium" in providers else None
    for provider in providers:
        rec = {"case": label, "n_rows": n, "hidden": h, "vocab": v, "dtype": str(hidden.dtype).replace("torch.", ""),
               "provider": provider}
        try:
            if provider == "helion_b200":
                fwd = bench_ms(lambda: helion_b200.linear_cross_entropy(hidden, weight, target))
                lse = torch.empty(n, dtype=torch.float32, device="cuda")
                stats = helion_b200.ops.local_stats(hidden.view(n, h), weight, target.view(n), 0)
                _, lse, _ = helion_b200.ops.finalize(stats.view(1, 3, n), target.view(n), "mean", -100)
                bwd = bench_ms(lambda: helion_b200.linear_cross_entropy_backward(grad_out, hidden, weight, target, lse))
                if nhv < 1e11:  # launch-bound shapes: also the per-call time of back-to-back calls
                    rec["fwd_loop_ms"] = loop_ms(lambda: helion_b200.linear_cross_entropy(hidden, weight, target))
                    rec["bwd_loop_ms"] = loop_ms(lambda: helion_b200.linear_cross_entropy_backward(grad_out, hidden, weight, target, lse))
                hg, wg = hidden.clone().requires_grad_(True), weight.clone().requires_grad_(True)

                def both():
                    hg.grad = wg.grad = None
                    helion_b200.linear_cross_entropy(hg, wg, target).backward(grad_out)

                rec["autograd_fwd_bwd_ms"] = bench_ms(both)
            elif provider == "torch_eager":
                if n * v > eager_limit:
                    continue
                fwd = bench_ms(lambda: _torch_linear_cross_entropy(hidden, weight, target))
                hg, wg = hidden.clone().requires_grad_(True), weight.clone().requires_grad_(True)
                loss = _torch_linear_cross_entropy(hg, wg, target)
                bwd = bench_ms(lambda: loss.backward(grad_out, retain_graph=True))
            elif provider == "tritium":
                if tritium is None:
                    continue
                fwd = bench_ms(lambda: tritium.linear_cross_entropy(hidden, weight, target))
                lse = torch.logsumexp(F.linear(hidden, weight).float().view(n, v), dim=-1) if n * v <= eager_limit else None
                if lse is None:
                    continue
                bwd = bench_ms(lambda: tritium.linear_cross_entropy_backward(grad_out, hidden.view(n, h), weight,
                                                                             target.view(n), lse))
                if nhv < 1e11:
                    rec["fwd_loop_ms"] = loop_ms(lambda: tritium.linear_cross_entropy(hidden, weight, target))
                    rec["bwd_loop_ms"] = loop_ms(lambda: tritium.linear_cross_entropy_backward(
                        grad_out, hidden.view(n, h), weight, target.view(n), lse))
            else:
                raise ValueError(f"Unknown provider: {provider}")
        except Exception as exc:  # noqa: BLE001 - one provider failing must not hide the others
            rec["error"] = f"{type(exc).__name__}: {exc}"[:200]
            print(json.dumps(rec), flush=True)
            continue
        total = fwd + bwd  # like the reference's tables: forward and backward timed separately
        rec.update({
            "fwd_ms": fwd, "bwd_ms": bwd, "fwd_bwd_ms": total,
            "fwd_tflops": tflops(2 * nhv, fwd), "bwd_tflops": tflops(6 * nhv, bwd),
            "fwd_bwd_tflops": tflops(8 * nhv, total), "tokens_per_s": n / (total * 1e-3),
            "frac_of_measured_bf16_peak": tflops(8 * nhv, total) / peak,
        })
        print(json.dumps(rec), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", action="store_true", help="the reference harness's seven fp16 shapes")
    ap.add_argument("--configs", action="store_true", help="the benchmark head configurations (bf16)")
    ap.add_argument("--sweep", action="store_true", help="Llama-3 head, N in {1024, 4096, 16384, 65536}")
    ap.add_argument("--fp32", action="store_true", help="fp32 inputs: the CUDA-core GEMM path, three shapes")
    ap.add_argument("--providers", default="helion_b200,torch_eager,tritium")
    args = ap.parse_args()
    require_cuda()
    providers = args.providers.split(",")
    peak = _peak()
    if not (args.shapes or args.configs or args.sweep or args.fp32):
        args.shapes = args.configs = True
    if args.fp32:
        torch.backends.cuda.matmul.allow_tf32 = False
        for n, h, v in FP32_SHAPES:
            hidden = torch.randn(n, h, device="cuda")
            weight = torch.randn(v, h, device="cuda") * 0.05
            target = torch.randint(v, (n,), device="cuda")
            time_case(f"fp32-{n}x{h}x{v}", hidden, weight, target, providers, peak)
    if args.shapes:
        for n, h, v in SHAPES:
            hidden = torch.randn(n, h, device="cuda", dtype=torch.float16)
            weight = torch.randn(v, h, device="cuda", dtype=torch.float16)
            target = torch.randint(v, (n,), device="cuda")
            time_case(f"shape-{n}x{h}x{v}", hidden, weight, target, providers, peak)
    cfgs = [inputs.CONFIGS[c] for c in CONFIG_NAMES] if args.configs else []
    cfgs += [inputs.sweep_config(r) for r in SWEEP_ROWS] if args.sweep else []
    for cfg in cfgs:
        d = inputs.make_inputs(cfg)
        time_case(cfg.name, d["hidden"].cuda(), d["weight"].cuda(), d["target"].cuda(), providers, peak)
        del d
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
