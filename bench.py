#!/usr/bin/env python
"""Headline benchmark: fused linear-cross-entropy forward+backward on the Llama-3-8B LM head.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one forward + backward of the loss over one batch of synthetic tokens. At N GPUs the weight
is sharded by vocabulary (one process per GPU, launched by torch.distributed.run) and the same batch is
processed by all ranks together, so total work is fixed ("strong" scaling). Rank 0 prints ONE JSON line.

``--impl reference`` times the reference's ground-truth expression (fp32 F.linear + F.cross_entropy +
autograd, the expression the reference's tests and benchmark compare against) on the host CPU, on a
bounded row sample of the same workload. The reference has no CPU implementation of its own and its GPU
kernels are not the CPU baseline.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "linear_ce_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"


def load_traffic(workload: str, world: int):
    """DRAM bytes per launch of the forward GEMM from the committed ncu capture of this workload
    (profiles/dram_traffic.json: dram__bytes_read.sum + dram__bytes_write.sum), or None."""
    path = ROOT / "profiles" / "dram_traffic.json"
    if not path.exists() or world != 1:
        return None
    return json.loads(path.read_text()).get(workload, {}).get("forward_gemm_bytes_per_launch")


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"burst": d["bf16_tflops"], "sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML every few milliseconds while the timed
    region runs (read-only queries; nothing on the GPU is changed)."""

    def __init__(self, gpu_index: int, period_s: float = 0.005):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples: list[tuple[int, float, int]] = []
        self.sm_max = None
        self.error = None
        self._stop = threading.Event()
        self._thread = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu_index]) if visible else self.gpu_index
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception as exc:  # noqa: BLE001 - reported in the JSON line
            self.error = f"nvml unavailable: {exc}"
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                clock = nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
                power = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                self.samples.append((clock, power, reasons))
            except Exception as exc:  # noqa: BLE001
                self.error = str(exc)
                return
            time.sleep(self.period_s)

    def mark(self) -> None:
        """Forget what was sampled so far: the region of interest starts now. Starting the sampler well before
        that region keeps NVML's start-up and its first, slow queries out of it."""
        self.samples = []

    def stop(self) -> dict:
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": [self.error or "not started"]}
        self._stop.set()
        self._thread.join(timeout=2)
        nv = self._nvml
        names = {
            "hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
            "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
            "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
            "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap,
        }
        seen = set()
        for _, _, mask in self.samples:
            for name, bit in names.items():
                if mask & bit:
                    seen.add(name)
        clocks = [c for c, _, _ in self.samples]
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": self.sm_max,
            "power_w_max": max((p for _, p, _ in self.samples), default=None),
            "samples": len(clocks),
            "reasons": sorted(seen),
        }


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        if world != n_gpus:
            raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}")
        return rank, world, local, dist
    if n_gpus != 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    torch.cuda.set_device(0)
    return 0, 1, 0, None


def build_workload(name: str):
    from helion_b200 import inputs

    if name.startswith("sweep-"):
        return inputs.sweep_config(int(name.split("-", 1)[1]))
    if name.startswith("shape-"):  # shape-<tokens>x<hidden>x<vocab>: uniform targets, nothing ignored
        n, h, v = (int(p) for p in name.split("-", 1)[1].split("x"))
        return inputs.HeadConfig(name, 1, n, h, v)
    return inputs.CONFIGS[name]


def workload_config(cfg, world: int, reduction: str) -> dict:
    """The `config` object of the JSON line; both arms (ours and --impl reference) print the same keys."""
    v_loc = cfg.vocab // world
    return {"workload": cfg.name, "tokens": cfg.rows, "hidden": cfg.hidden, "vocab": cfg.vocab,
            "vocab_per_gpu": v_loc, "reduction": reduction, "parallelism": f"vocab-parallel x{world}",
            "l2": "weight shard (%.0f MB) exceeds L2, no explicit flush" % (v_loc * cfg.hidden * 2 / 1e6)}


def host_threads() -> int:
    """Host cores this process may use (its CPU affinity), whatever OMP_NUM_THREADS a launcher exported."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(data: dict, sample_rows: int, repeats: int, warmup: int) -> dict:
    """fp32 ground-truth expression on the host cores over the first `sample_rows` rows x full vocab."""
    from oracle import oracle

    # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm uses every core it may at every GPU count
    torch.set_num_threads(host_threads())
    h = data["hidden"].reshape(-1, data["hidden"].shape[-1])[:sample_rows]
    t = data["target"].reshape(-1)[:sample_rows]
    red = data["reduction"]
    go = data["grad_out"]
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        oracle.expression(h, data["weight"], t, reduction=red, ignore_index=data["ignore_index"], grad_out=go)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = statistics.median(times)
    return {
        "value": sample_rows / sec,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "sample": f"first {sample_rows} rows x full vocab, fp32 F.linear+F.cross_entropy+autograd, "
                  f"median of {repeats} after {warmup} warm-up, {sec:.3f} s each",
        "seconds_per_sample": sec,
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from helion_b200 import inputs

    cfg = build_workload(args.workload)
    data = inputs.make_inputs(cfg)
    flops_per_row = 8.0 * cfg.hidden * cfg.vocab
    # at most 2e12 FLOP of CPU work per step and 1e14 FLOP per run: a couple of minutes on 16 cores
    per_step = min(2.0e12, 1.0e14 / max(1, args.steps + min(args.warmup, 2)))
    sample_rows = max(16, min(cfg.rows, int(per_step / flops_per_row)))
    base = cpu_baseline(data, sample_rows, repeats=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    sec = base["seconds_per_sample"]
    line = {
        "impl": "reference",
        "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, max(1, args.gpus), cfg.reduction),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "host_cpus", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    from helion_b200 import _lib, inputs, ops, parallel

    rank, world, local, dist = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    cfg = build_workload(args.workload)
    data = inputs.make_inputs(cfg)
    n, h, v = cfg.rows, cfg.hidden, cfg.vocab
    if v % world:
        raise SystemExit(f"vocab {v} is not divisible by {world} ranks")
    v_loc = v // world
    group = dist.group.WORLD if world > 1 else None

    x_host = data["hidden"].pin_memory()
    t_host = data["target"].pin_memory()
    w = data["weight"][rank * v_loc:(rank + 1) * v_loc].to(dev).requires_grad_(True)
    x = x_host.to(dev).requires_grad_(True)
    t = t_host.to(dev)
    go = data["grad_out"].to(dev)
    red, ign = cfg.reduction, data["ignore_index"]
    L = _lib.lib()

    fwd_only = args.forward_only
    if fwd_only:
        red = "none"  # per-token loss (= -logprob of the target), the inference-side use of the head

    def step(xx, tt):
        if fwd_only:
            with torch.no_grad():
                return ops.linear_cross_entropy(xx, w, tt, reduction=red, ignore_index=ign, process_group=group)
        xx.grad = None
        w.grad = None
        loss = ops.linear_cross_entropy(xx, w, tt, reduction=red, ignore_index=ign, process_group=group)
        loss.backward(go)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        tt = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    # ---- device-resident timing ------------------------------------------------------------
    # Warm-up by step count, then by time: a GPU that has idled starts at its boost clock and settles to the
    # clock its power cap sustains only after a second or two of load. Short timed regions (8 GPUs: tens of
    # milliseconds) would otherwise be measured at a clock a training run never sees.
    for _ in range(max(args.warmup, 3)):
        loss = step(x, t)
    barrier()
    sampler = ClockSampler(local, args.clock_period_ms / 1e3)
    sampler.start()  # every rank samples its own GPU; started here so that NVML's start-up is over by the timed region
    preheat_steps = 0
    t_heat = time.perf_counter()
    while args.preheat_s > 0:
        for _ in range(5):
            loss = step(x, t)
        preheat_steps += 5
        torch.cuda.synchronize()
        go_on = torch.tensor([1.0 if time.perf_counter() - t_heat < args.preheat_s else 0.0], device=dev)
        if world > 1:  # every rank leaves the loop after the same number of steps
            dist.all_reduce(go_on, op=dist.ReduceOp.MIN)
        if float(go_on.item()) == 0.0:
            break
    preheat_s = time.perf_counter() - t_heat
    launches0 = L.lce_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark()
    e0.record()
    for _ in range(args.steps):
        loss = step(x, t)
    e1.record()
    barrier()
    launches = L.lce_launch_count() - launches0
    ms_local = e0.elapsed_time(e1)
    ms_total = max_over_ranks(ms_local)
    clocks = sampler.stop()
    ms_step = ms_total / args.steps
    loss_value = float(loss.float().mean().item())
    # time x clock per rank: what the step costs in SM cycles, comparable across runs at different clocks
    my_mhz = float(clocks["sm_mhz"] or 0.0)
    per_rank = [(ms_local / args.steps, my_mhz)]
    if world > 1:
        mine = torch.tensor([ms_local / args.steps, my_mhz], dtype=torch.float64, device=dev)
        everyone = torch.empty((world, 2), dtype=torch.float64, device=dev)
        dist.all_gather_into_tensor(everyone.view(-1), mine)
        per_rank = [(float(a), float(b)) for a, b in everyone.tolist()]
    reasons = clocks["reasons"]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, reasons)
        reasons = sorted({r for rr in gathered for r in rr})

    # ---- end to end: every step's activations and labels come from pinned host memory and its loss goes
    # back to the host, all inside the timed region. As in a training loop with a prefetching loader, the
    # copy of step i+1 runs on a copy stream while step i computes (two device buffers). With several GPUs
    # the batch crosses the host link ONCE: rank r copies rows [r * N/R, (r+1) * N/R) and one all-gather over
    # NVLink rebuilds the batch on every rank (replicating it by R host copies made the copy the bottleneck).
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    rpr = -(-n // world)
    r0, r1 = min(n, rank * rpr), min(n, (rank + 1) * rpr)
    x2d_host, t1d_host = x_host.view(n, h), t_host.view(n)
    xb = [torch.empty_like(x).requires_grad_(True) for _ in range(2)]
    tb = [torch.empty_like(t) for _ in range(2)]
    x_piece = torch.zeros((rpr, h), dtype=x.dtype, device=dev)
    t_piece = torch.zeros((rpr,), dtype=t.dtype, device=dev)
    ready = [torch.cuda.Event() for _ in range(2)]     # copy into buffer b has landed
    consumed = [torch.cuda.Event() for _ in range(2)]  # step using buffer b has finished
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    h2d_bytes = (r1 - r0) * (h * x.element_size() + t.element_size())

    def prefetch(b):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])
            with torch.no_grad():
                if world == 1:
                    xb[b].copy_(x_host, non_blocking=True)
                    tb[b].copy_(t_host, non_blocking=True)
                else:
                    x_piece[:r1 - r0].copy_(x2d_host[r0:r1], non_blocking=True)
                    t_piece[:r1 - r0].copy_(t1d_host[r0:r1], non_blocking=True)
                    xb[b].view(n, h).copy_(parallel.gather_rows(x_piece, n, group))
                    tb[b].view(n).copy_(parallel.gather_rows(t_piece, n, group))
            ready[b].record(copy_stream)

    def run_e2e(steps):
        for b in range(2):
            consumed[b].record(main_stream)
        prefetch(0)
        for i in range(steps):
            b = i & 1
            if i + 1 < steps:
                prefetch(b ^ 1)
            main_stream.wait_event(ready[b])
            l2 = step(xb[b], tb[b])
            loss_host.copy_(l2.detach() if l2.dim() == 0 else l2.detach().sum(), non_blocking=True)
            consumed[b].record(main_stream)

    run_e2e(3)
    barrier()
    # the batch every rank computed on is the batch the host holds
    assert torch.equal(xb[0].detach(), x.detach()) and torch.equal(tb[0], t), "gathered batch differs from the host batch"
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    run_e2e(args.steps)
    e3.record()
    barrier()
    ms_e2e = max_over_ranks(e2.elapsed_time(e3)) / args.steps

    # ---- dominant kernel, timed alone through the C ABI: the forward logits GEMM + statistics
    stats = torch.empty((3, n), dtype=torch.float32, device=dev)
    ws = torch.empty(L.lce_forward_workspace_bytes(n, h, v_loc, _lib.DTYPE_BF16, 0), dtype=torch.uint8, device=dev)
    x2d = x.detach().view(n, h)
    t1d = t.view(n)

    def fwd_kernel():
        _lib.check(L.lce_forward_stats(x2d.data_ptr(), w.data_ptr(), t1d.data_ptr(), 1, n, h, v_loc, rank * v_loc,
                                       _lib.DTYPE_BF16, stats.data_ptr(), ws.data_ptr(), ws.numel(), 0,
                                       torch.cuda.current_stream().cuda_stream), "lce_forward_stats")

    def time_fwd_kernel():
        for _ in range(3):
            fwd_kernel()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(args.steps):
            fwd_kernel()
        k1.record()
        torch.cuda.synchronize()
        return k0.elapsed_time(k1) / args.steps

    # twice: straight after the steps above, on a GPU that sits at its power cap (to be read against the
    # SUSTAINED peak), and again after a rest, the condition under which the BURST peak was measured
    # (best of ten 0.7 ms GEMMs on an idle GPU); K launches back to back each time, average duration.
    ms_fwd_hot = time_fwd_kernel()
    barrier()
    rest_sampler = ClockSampler(local, args.clock_period_ms / 1e3)
    rest_sampler.start()
    time.sleep(args.rest_s)
    rest_sampler.mark()
    ms_fwd = time_fwd_kernel()
    rest_clocks = rest_sampler.stop()

    status = _lib.device_status()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    flops_step = (2.0 if fwd_only else 8.0) * n * h * v / world  # algorithmic FLOPs per GPU per step
    tf_step = flops_step / (ms_step * 1e-3) / 1e12
    flops_fwd = 2.0 * n * h * v_loc
    tf_fwd = flops_fwd / (ms_fwd * 1e-3) / 1e12
    base = None
    if world == 1 and not args.no_cpu_baseline:
        sample_rows = max(16, min(n, int(1.5e12 / (8.0 * h * v))))
        base = cpu_baseline(data, sample_rows, repeats=3, warmup=1)
        base = {k: base[k] for k in ("value", "unit", "cores", "host_cpus", "kind", "sample")}
    line = {
        "metric": "linear_ce_fwd_tokens_per_s" if fwd_only else METRIC, "value": n / (ms_step * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(cfg, world, red),
        "preheat_s": round(preheat_s, 3), "preheat_steps": preheat_steps,
        "loss": loss_value,
        "device_status": status,
        "step_tflops_per_gpu": tf_step,
        "step_frac_of_peak": {"burst_%g" % peaks["burst"]: tf_step / peaks["burst"],
                              "sustained_%g" % peaks["sustained"]: tf_step / peaks["sustained"],
                              "nominal_2250": tf_step / 2250.0},
        "roofline": {"bound": "tensor",
                     "kernel": "gemm_tc_kernel<256,6,2,K,K,bf16,EpiStats> (forward logits + softmax statistics; "
                               "timed through lce_forward_stats, which also runs the sub-1% merge kernel)",
                     "achieved": tf_fwd, "peak": peaks["burst"], "peak_source": peaks["source"] + " burst",
                     "unit": "TFLOP/s", "frac": tf_fwd / peaks["burst"], "ms_per_launch": ms_fwd,
                     "condition": "%d launches back to back after %.1f s of rest (the burst peak is a best-of-ten on "
                                  "an idle GPU); median SM clock %s MHz" % (args.steps, args.rest_s, rest_clocks["sm_mhz"]),
                     "hot_loop": {"achieved": flops_fwd / (ms_fwd_hot * 1e-3) / 1e12, "ms_per_launch": ms_fwd_hot,
                                  "peak": peaks["sustained"], "peak_source": peaks["source"] + " sustained",
                                  "frac": flops_fwd / (ms_fwd_hot * 1e-3) / 1e12 / peaks["sustained"],
                                  "frac_of_burst": flops_fwd / (ms_fwd_hot * 1e-3) / 1e12 / peaks["burst"],
                                  "condition": "the same launches straight after the timed steps, GPU at its power cap"},
                     "flops_per_launch": flops_fwd, "traffic": load_traffic(cfg.name, world),
                     "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                     "algorithmic_bytes_per_launch": (n * h + v_loc * h) * 2 + (v_loc + 255) // 256 * 3 * n * 4},
        "e2e": {"value": n / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
                "note": "bytes per rank; at N > 1 each rank copies its row slice and one all-gather over NVLink "
                        "rebuilds the batch" if world > 1 else "whole batch from pinned host memory"},
        "gpu_launches": int(launches),
        "clocks": dict(clocks, reasons=reasons),
        "cycles": {"ms_x_mhz": max(a * b for a, b in per_rank), "sm_mhz_per_rank": [b for _, b in per_rank],
                   "ms_per_step_per_rank": [a for a, _ in per_rank],
                   "note": "ms_per_step x median SM MHz, max over ranks: step cost in thousands of SM cycles"},
    }
    if base is not None:
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="llama3-8b",
                    help="llama3-8b (headline), gpt2-small, large-vocab, 14b-class, sweep-<rows>")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--clock-period-ms", type=float, default=5.0,
                    help="period of the NVML clock / power samples taken during the timed regions")
    ap.add_argument("--rest-s", type=float, default=2.0,
                    help="idle seconds before the forward kernel is timed alone against the burst peak")
    ap.add_argument("--preheat-s", type=float, default=2.0,
                    help="seconds of untimed steps before the timed region, so that it runs at the sustained clock")
    ap.add_argument("--forward-only", action="store_true",
                    help="time the forward alone with reduction='none' (per-token loss), 2 N H V FLOPs per step")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
