"""Forward / backward timings of the plain cross-entropy on materialised logits, in effective GB/s.

Restates the reference's harness (``benchmarks/bench_cross_entropy.py`` of the reference: fp16 logits,
shapes (1, 1024) ... (16, 32768), effective bandwidth = logits bytes / time) with CUDA-event timing, and adds
LM-sized rows (8192 x 128256, 16384 x 256000 in bf16) with the fraction of the measured HBM copy bandwidth.
Forward moves N*V*elem bytes (one read), backward 2*N*V*elem (read + write).

    python -m benchmarks.bench_cross_entropy [--providers helion_b200,torch_eager,tritium]
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
from benchmarks._utils import bench_ms, require_cuda  # noqa: E402

SHAPES = [(1, 1024), (16, 1024), (128, 1024), (16, 8192), (16, 32768)]  # the reference's
LARGE = [(4096, 50304), (8192, 128256), (16384, 256000)]


def _hbm_peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    return json.loads(path.read_text())["hbm_gbs"] if path.exists() else 6650.0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--providers", default="helion_b200,torch_eager,tritium")
    args = ap.parse_args()
    require_cuda()
    peak = _hbm_peak()
    tritium = None
    if "tritium" in args.providers and (ROOT / "baseline" / "_ref" / "tritium").exists():
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import tritium  # noqa: F811
    grad_out = torch.tensor(1.0, device="cuda")
    for n, v in SHAPES + LARGE:
        dtype = torch.float16 if (n, v) in SHAPES else torch.bfloat16
        logits = torch.randn(n, v, device="cuda", dtype=dtype)
        target = torch.randint(v, (n,), device="cuda")
        lse = torch.logsumexp(logits.float(), dim=-1)
        nbytes = logits.numel() * logits.element_size()
        for provider in args.providers.split(","):
            rec = {"n_rows": n, "vocab": v, "dtype": str(dtype).replace("torch.", ""), "provider": provider}
            try:
                if provider == "helion_b200":
                    fwd = bench_ms(lambda: helion_b200.cross_entropy(logits, target))
                    bwd = bench_ms(lambda: helion_b200.cross_entropy_backward(grad_out, logits, target, lse))
                elif provider == "torch_eager":
                    fwd = bench_ms(lambda: F.cross_entropy(logits.float(), target))
                    zg = logits.clone().requires_grad_(True)
                    loss = F.cross_entropy(zg.float(), target)
                    bwd = bench_ms(lambda: loss.backward(grad_out, retain_graph=True))
                elif provider == "tritium":
                    if tritium is None:
                        continue
                    fwd = bench_ms(lambda: tritium.cross_entropy(logits, target))
                    bwd = bench_ms(lambda: tritium.cross_entropy_backward(grad_out, logits, target, lse))
                else:
                    raise ValueError(f"Unknown provider: {provider}")
            except Exception as exc:  # noqa: BLE001
                rec["error"] = f"{type(exc).__name__}: {exc}"[:160]
                print(json.dumps(rec), flush=True)
                continue
            rec.update({"fwd_ms": fwd, "bwd_ms": bwd, "fwd_gbs": nbytes / (fwd * 1e-3) / 1e9,
                        "bwd_gbs": 2 * nbytes / (bwd * 1e-3) / 1e9,
                        "fwd_frac_of_hbm": nbytes / (fwd * 1e-3) / 1e9 / peak,
                        "bwd_frac_of_hbm": 2 * nbytes / (bwd * 1e-3) / 1e9 / peak})
            print(json.dumps(rec), flush=True)
        del logits, lse


if __name__ == "__main__":
    main()
