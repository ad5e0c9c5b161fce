"""Decode-step timings of the greedy head and the top-k sampling head on the Llama-3-8B LM head
(4096 x 128256, bf16).

A decode step reads the whole weight once (V*H*elem bytes; the batch is tiny), so the yardstick is HBM
bandwidth. Providers: ``helion_b200`` (``greedy_head``: argmax and log-probability, logits never written),
``helion_b200_topk50`` (``topk_head`` with k = 50: the candidates and the logsumexp that temperature / top-k /
nucleus sampling needs), ``torch_eager`` (``hidden @ weight.T`` in bf16, then argmax / logsumexp of the
materialised logits), ``torch_eager_topk50`` (the same product, then ``torch.topk(logits.float(), 50)`` and
``logsumexp``, as the reference's ``sample_next_token`` does, examples/common.py:284-289),
``reference_decode`` (what the reference's model does per step, examples/common.py:127-131:
``matmul(hidden, lm_head.T.contiguous())`` - the transpose copy included - then argmax; torch.matmul stands in
for tritium.matmul so that only the extra copy and the logits write are being compared).

    python -m benchmarks.bench_greedy_head [--rows 1,16,128,1024] [--providers helion_b200,...]
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="1,16,128,1024")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--providers", default="helion_b200,helion_b200_topk50,torch_eager,torch_eager_topk50,reference_decode")
    args = ap.parse_args()
    require_cuda()
    peaks = ROOT / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks.read_text())["hbm_gbs"] if peaks.exists() else 6650.0
    h, v = args.hidden, args.vocab
    weight = (torch.randn(v, h, device="cuda") * 0.02).bfloat16()
    wbytes = weight.numel() * weight.element_size()
    for n in (int(r) for r in args.rows.split(",")):
        hidden = torch.randn(n, h, device="cuda", dtype=torch.bfloat16)

        def eager():
            z = hidden @ weight.T
            return z.argmax(dim=-1), torch.logsumexp(z.float(), dim=-1)

        def eager_topk():
            z = (hidden @ weight.T).float()
            return torch.topk(z, 50, dim=-1), torch.logsumexp(z, dim=-1)

        for provider, fn in (("helion_b200", lambda: helion_b200.greedy_head(hidden, weight)),
                             ("helion_b200_topk50", lambda: helion_b200.topk_head(hidden, weight, 50)),
                             ("torch_eager", eager), ("torch_eager_topk50", eager_topk), ("reference_decode", lambda: (hidden @ weight.T.contiguous()).argmax(dim=-1))):  # the transpose copy per step
            if provider not in args.providers.split(","):
                continue
            ms = bench_ms(fn)
            print(json.dumps({"rows": n, "hidden": h, "vocab": v, "provider": provider, "ms": ms,
                              "weight_gbs": wbytes / (ms * 1e-3) / 1e9, "frac_of_hbm": wbytes / (ms * 1e-3) / 1e9 / hbm}),
                  flush=True)


if __name__ == "__main__":
    main()
