"""Square fp16 matrix products, the reference's matmul benchmark restated without Triton.

The reference's harness (``benchmarks/bench_matmul.py`` of the reference) times ``C = A @ B`` for square fp16
matrices of 14 sizes from 256 to 4096 and reports TFLOP/s (2 n^3 / t) per provider. Providers here:
``helion_b200`` (``helion_b200.matmul``: the tcgen05 GEMM core of the fused loss with a plain store epilogue,
B read MN-major as stored, K split for sizes with few output tiles), ``torch_eager`` (``torch.matmul``, i.e.
cuBLAS) and ``tritium`` (the reference's autotuned Triton kernel, only if a copy is installed under
baseline/_ref). Added: three LM-shaped products in bf16 (tokens x hidden x vocabulary). One JSON object per
line.

    python -m benchmarks.bench_matmul [--providers a,b] [--sizes 256,1024,...]
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
from benchmarks._utils import bench_ms, require_cuda, tflops  # noqa: E402

SIZES = [256, 512, 768, 1024, 1280, 1536, 1792, 2048, 2304, 2560, 3072, 3328, 3584, 4096]  # the reference's list
LM_SHAPES = [(8192, 4096, 4096), (8192, 4096, 14336), (4096, 4096, 128256)]  # (M, K, N) bf16


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--providers", default="helion_b200,torch_eager,tritium")
    ap.add_argument("--sizes", default="")
    args = ap.parse_args()
    require_cuda()
    peaks = ROOT / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text())["bf16_tflops"] if peaks.exists() else 1590.0
    providers = args.providers.split(",")
    tritium = _reference_module() if "tritium" in providers else None
    sizes = [int(v) for v in args.sizes.split(",") if v] or SIZES
    cases = [(n, n, n, torch.float16) for n in sizes] + [(m, k, n, torch.bfloat16) for m, k, n in LM_SHAPES]
    for m, k, n, dtype in cases:
        a = torch.randn(m, k, device="cuda", dtype=dtype)
        b = torch.randn(k, n, device="cuda", dtype=dtype)
        for provider in providers:
            fn = {"helion_b200": lambda: helion_b200.matmul(a, b), "torch_eager": lambda: torch.matmul(a, b),
                  "tritium": (lambda: tritium.matmul(a, b)) if tritium is not None else None}[provider]
            if fn is None:
                continue
            rec = {"m": m, "k": k, "n": n, "dtype": str(dtype).replace("torch.", ""), "provider": provider}
            try:
                ms = bench_ms(fn)
                rec.update({"ms": ms, "tflops": tflops(2.0 * m * k * n, ms), "frac_of_measured_bf16_peak": tflops(2.0 * m * k * n, ms) / peak})
            except Exception as exc:  # noqa: BLE001 - one provider failing must not hide the others
                rec["error"] = f"{type(exc).__name__}: {exc}"[:200]
            print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
