"""Forward / backward timings of RMSNorm and residual RMSNorm, in GB/s of algorithmic traffic.

Restates the reference's harness (``benchmarks/bench_rmsnorm.py`` of the reference: fp16, shapes (1, 1024)
... (128, 8192)) with CUDA-event timing, and adds LM-sized activations (16384 x 4096 and 8192 x 8192 in
bf16) with the fraction of the measured HBM copy bandwidth. Bytes counted per element of the activation:
forward 2 (read x, write out), residual forward 4 (x, residual in; out, residual_out out), backward 3
(dy, x in; dx out), residual backward 4 (dy, dresidual, residual_out in; dz out). The reference's backward
reads dy and x a second time for dweight; that extra traffic is not counted for either provider.

    python -m benchmarks.bench_rmsnorm [--providers helion_b200,torch_eager,tritium] [--shapes 16384x4096,...]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import helion_b200  # noqa: E402
from benchmarks._utils import bench_ms, require_cuda  # noqa: E402

SHAPES = [(1, 1024), (16, 1024), (128, 1024), (1024, 1024), (4096, 1024), (128, 2048), (128, 4096), (128, 8192)]
LARGE = [(16384, 4096), (8192, 8192), (32768, 2048)]
EPS = 1e-6


def _hbm_peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    return json.loads(path.read_text())["hbm_gbs"] if path.exists() else 6650.0


def _torch_rmsnorm(x, w):
    rstd = torch.rsqrt(x.float().pow(2).mean(dim=-1, keepdim=True) + EPS)
    return (x.float() * rstd * w.float()).to(x.dtype)


def _torch_backward(dy, x, w):
    xf, dyf, wf = x.float(), dy.float(), w.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + EPS)
    dot = (dyf * wf * xf).sum(dim=-1, keepdim=True)
    dx = dyf * wf * rstd - xf * dot * rstd.pow(3) / x.shape[-1]
    return dx.to(x.dtype), (dyf * xf * rstd).sum(dim=0).to(w.dtype)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--providers", default="helion_b200,torch_eager,tritium")
    ap.add_argument("--shapes", default="", help="comma-separated NxH (bf16) instead of the built-in list")
    args = ap.parse_args()
    require_cuda()
    peak = _hbm_peak()
    tritium = None
    if "tritium" in args.providers and (ROOT / "baseline" / "_ref" / "tritium").exists():
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import tritium  # noqa: F811
    shapes = [tuple(int(v) for v in item.split("x")) for item in args.shapes.split(",") if item] or SHAPES + LARGE
    for n, h in shapes:
        dtype = torch.float16 if (n, h) in SHAPES else torch.bfloat16
        x = torch.randn(n, h, device="cuda", dtype=dtype)
        r, dy, dz = torch.randn_like(x), torch.randn_like(x), torch.randn_like(x)
        w = torch.randn(h, device="cuda", dtype=dtype)
        nbytes = x.numel() * x.element_size()
        for provider in args.providers.split(","):
            rec = {"n_rows": n, "hidden": h, "dtype": str(dtype).replace("torch.", ""), "provider": provider}
            try:
                if provider in ("helion_b200", "tritium"):
                    mod = helion_b200 if provider == "helion_b200" else tritium
                    if mod is None:
                        continue
                    fwd = bench_ms(lambda: mod.rmsnorm(x, w, EPS))
                    res = bench_ms(lambda: mod.residual_rmsnorm(x, r, w, EPS))
                    bwd = bench_ms(lambda: mod.rmsnorm_backward(dy, x, w, EPS))
                    xg, rg, wg = (t.clone().requires_grad_(True) for t in (x, r, w))
                    o, z = mod.residual_rmsnorm(xg, rg, wg, EPS)
                    res_bwd = bench_ms(lambda: torch.autograd.grad([o, z], [xg, rg, wg], [dy, dz], retain_graph=True))
                elif provider == "torch_eager":
                    fwd = bench_ms(lambda: _torch_rmsnorm(x, w))
                    res = bench_ms(lambda: _torch_rmsnorm((x.float() + r.float()).to(dtype), w))
                    bwd = bench_ms(lambda: _torch_backward(dy, x, w))
                    res_bwd = bench_ms(lambda: _torch_backward(dy, x, w)[0] + dz)
                else:
                    raise ValueError(f"Unknown provider: {provider}")
            except Exception as exc:  # noqa: BLE001
                rec["error"] = f"{type(exc).__name__}: {exc}"[:160]
                print(json.dumps(rec), flush=True)
                continue
            for key, ms, mult in (("fwd", fwd, 2), ("residual_fwd", res, 4), ("bwd", bwd, 3), ("residual_bwd", res_bwd, 4)):
                rec[f"{key}_ms"] = ms
                rec[f"{key}_gbs"] = mult * nbytes / (ms * 1e-3) / 1e9
                rec[f"{key}_frac_of_hbm"] = rec[f"{key}_gbs"] / peak
            print(json.dumps(rec), flush=True)
        del x, r, dy, dz


if __name__ == "__main__":
    main()
