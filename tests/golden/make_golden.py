"""Generates the golden fixtures under tests/golden/.

    python tests/golden/make_golden.py --oracle
        CPU only. Writes oracle_cases.pt: the fp32 ground-truth expression (oracle.expression) for
        every case below, with checksums of the seeded inputs (tests rebuild the inputs with
        make_case_inputs).

    python tests/golden/make_golden.py --reference OUT.pt
        Needs a GPU and an installed copy of the reference (``pip install --target baseline/_ref``).
        Runs the reference's OWN kernels - tritium.linear_cross_entropy (Triton forward),
        its autograd backward and tritium.linear_cross_entropy_backward - on the same inputs and
        stores what they return. The committed reference_b200.pt came from this mode on a B200
        (torch 2.11.0+cu128, triton 3.6.0). It pins the oracle's restatement of the reference
        algorithm and is the closest thing to a golden vector the path has: the reference ships none.

    python tests/golden/make_golden.py --reference-rmsnorm OUT.pt
        The same for the producer of the hidden states: tritium.rmsnorm, tritium.residual_rmsnorm (forward,
        autograd backward) and tritium.rmsnorm_backward on the cases of rmsnorm_case_list(). The committed
        reference_b200_rmsnorm.pt came from this mode on a B200.

Cases follow the reference's own tests (tests/tritium/test_cross_entropy.py:59-109: H=64, V in
{128, 1024}, N in {1, 16, 128}, std-1 weights; autograd at N=32, H=64, V=256; 3-D hidden) plus one
shape that takes the reference's large-shape backward branch (row-chunk loop over cuBLAS GEMMs).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def case_list() -> list[dict]:
    cases = []
    for dt in DTYPES:
        for v in (128, 1024):
            for n in (1, 16, 128):
                cases.append({"name": f"fwd-{dt}-n{n}-v{v}", "shape": (n,), "h": 64, "v": v, "dtype": dt,
                              "grads": False})
        cases.append({"name": f"autograd-{dt}", "shape": (32,), "h": 64, "v": 256, "dtype": dt, "grads": True})
    cases.append({"name": "hidden3d-float32", "shape": (4, 16), "h": 64, "v": 128, "dtype": "float32",
                  "grads": False})
    # N*V > 65536 -> the reference leaves its fused backward kernel for the chunk loop
    cases.append({"name": "chunkloop-bfloat16", "shape": (80,), "h": 64, "v": 832, "dtype": "bfloat16",
                  "grads": True, "grad_out": 0.37})
    cases.append({"name": "chunkloop-float32", "shape": (48,), "h": 72, "v": 300, "dtype": "float32",
                  "grads": True, "grad_out": 2.5})
    # plain cross-entropy on materialised logits (reference tests :11-56): appended so that the
    # seeds of the cases above never move
    for dt in DTYPES:
        for v in (16, 1024):
            for n in (1, 128):
                cases.append({"name": f"plain-fwd-{dt}-n{n}-v{v}", "op": "plain", "shape": (n,), "v": v, "dtype": dt,
                              "grads": False})
        cases.append({"name": f"plain-autograd-{dt}", "op": "plain", "shape": (64,), "v": 256, "dtype": dt,
                      "grads": True, "grad_out": -0.8})
    return cases


def make_case_inputs(case: dict, index: int) -> dict:
    g = torch.Generator(device="cpu").manual_seed(1000 + index)
    dt = DTYPES[case["dtype"]]
    if case.get("op") == "plain":
        logits = torch.randn(*case["shape"], case["v"], generator=g).to(dt)
        target = torch.randint(0, case["v"], case["shape"], generator=g)
        return {"logits": logits, "target": target,
                "grad_out": torch.tensor(case.get("grad_out", 1.0), dtype=torch.float32)}
    hidden = torch.randn(*case["shape"], case["h"], generator=g).to(dt)
    weight = torch.randn(case["v"], case["h"], generator=g).to(dt)
    target = torch.randint(0, case["v"], case["shape"], generator=g)
    return {"hidden": hidden, "weight": weight, "target": target,
            "grad_out": torch.tensor(case.get("grad_out", 1.0), dtype=torch.float32)}


def rmsnorm_case_list() -> list[dict]:
    """Shapes after the reference's tests (tests/tritium/test_rmsnorm.py:7-9, :76-235), cut down to rows
    that keep the fixture small: a power-of-two width, an odd multiple of 8, the widest tested (11008), a
    width below 512 (the reference's atomic dweight branch, not a multiple of the vector width) and one
    just above it with >= 64 rows (its staged dweight branch)."""
    cases = []
    for dt in DTYPES:
        for shape, h in (((16,), 1024), ((2, 3), 2560), ((3,), 11008), ((130,), 100), ((70,), 520)):
            cases.append({"name": f"rms-{dt}-n{'x'.join(map(str, shape))}-h{h}", "shape": shape, "h": h, "dtype": dt})
    return cases


def make_rmsnorm_inputs(case: dict, index: int) -> dict:
    g = torch.Generator(device="cpu").manual_seed(5000 + index)
    dt = DTYPES[case["dtype"]]
    shape = (*case["shape"], case["h"])
    return {"x": torch.randn(shape, generator=g).to(dt), "residual": torch.randn(shape, generator=g).to(dt),
            "weight": torch.randn(case["h"], generator=g).to(dt), "dy": torch.randn(shape, generator=g).to(dt),
            "dres": torch.randn(shape, generator=g).to(dt), "eps": 1e-6}


def dedup(rec: dict) -> dict:
    """Store tensors that came out bit-identical once: a later key holds ("same_as", earlier key)."""
    out: dict = {}
    for key, val in rec.items():
        twin = next((k for k, v in out.items() if torch.is_tensor(v) and v.shape == val.shape and v.dtype == val.dtype
                     and torch.equal(v, val)), None)
        out[key] = ("same_as", twin) if twin is not None else val
    return out


def fixture_tensor(rec: dict, key: str) -> torch.Tensor:
    val = rec[key]
    return rec[val[1]] if isinstance(val, tuple) else val


def run_reference_rmsnorm(dest: str) -> None:
    ref_dir = ROOT / "baseline" / "_ref"
    sys.path.insert(0, str(ref_dir))
    import tritium

    dev = torch.device("cuda", 0)
    out = {"_meta": {"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0),
                     "triton": __import__("triton").__version__}}
    for i, case in enumerate(rmsnorm_case_list()):
        inp = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in make_rmsnorm_inputs(case, i).items()}
        x, r, w, dy, dres, eps = (inp[k] for k in ("x", "residual", "weight", "dy", "dres", "eps"))
        rec = {"out": tritium.rmsnorm(x, w, eps).cpu()}
        dx, dw = tritium.rmsnorm_backward(dy, x, w, eps)
        rec["dx_direct"], rec["dweight_direct"] = dx.cpu(), dw.cpu()
        xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        tritium.rmsnorm(xg, wg, eps).backward(dy)
        rec["dx"], rec["dweight"] = xg.grad.cpu(), wg.grad.cpu()
        o2, z2 = tritium.residual_rmsnorm(x, r, w, eps)
        rec["res_out"], rec["res_z"] = o2.cpu(), z2.cpu()
        xg, rg, wg = (t.clone().requires_grad_(True) for t in (x, r, w))
        o3, z3 = tritium.residual_rmsnorm(xg, rg, wg, eps)
        torch.autograd.backward([o3, z3], [dy, dres])
        rec["res_dx"], rec["res_dresidual"], rec["res_dweight"] = xg.grad.cpu(), rg.grad.cpu(), wg.grad.cpu()
        torch.cuda.synchronize()
        print(case["name"], float(rec["out"].float().abs().mean()))
        out[case["name"]] = dedup(rec)
    torch.save(out, dest)
    print(f"wrote {dest}")


def input_checksums(inp: dict) -> dict:
    """float64 sums of the seeded inputs: lets a test notice if the CPU generator ever changes."""
    return {k: float(inp[k].double().sum()) for k in ("hidden", "weight", "logits", "target") if k in inp}


def run_oracle() -> None:
    from oracle import oracle

    out = {}
    for i, case in enumerate(case_list()):
        inp = make_case_inputs(case, i)
        if case.get("op") == "plain":
            ref = oracle.plain_expression(inp["logits"], inp["target"], grad_out=inp["grad_out"],
                                          want_grads=case["grads"])
        else:
            ref = oracle.expression(inp["hidden"], inp["weight"], inp["target"], grad_out=inp["grad_out"],
                                    want_grads=case["grads"])
        out[case["name"]] = {"case": case, "input_checksums": input_checksums(inp), "expected": ref}
    torch.save(out, HERE / "oracle_cases.pt")
    print(f"wrote {HERE / 'oracle_cases.pt'} ({len(out)} cases)")


def run_reference(dest: str) -> None:
    ref_dir = ROOT / "baseline" / "_ref"
    sys.path.insert(0, str(ref_dir))
    import importlib

    import tritium

    # `tritium.ops.cross_entropy` the attribute is the re-exported function; the module is in sys.modules
    ref_ce = importlib.import_module("tritium.ops.cross_entropy")

    dev = torch.device("cuda", 0)
    out = {"_meta": {"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0),
                     "triton": __import__("triton").__version__}}
    for i, case in enumerate(case_list()):
        inp = make_case_inputs(case, i)
        if case.get("op") == "plain":
            z = inp["logits"].to(dev)
            t = inp["target"].to(dev)
            loss, lse = ref_ce._cross_entropy_forward(z, t)
            rec = {"loss": loss.cpu(), "lse": lse.cpu()}
            if case["grads"]:
                zg = z.clone().requires_grad_(True)
                tritium.cross_entropy(zg, t).backward(inp["grad_out"].to(dev))
                rec["dlogits"] = zg.grad.cpu()
                rec["dlogits_direct"] = tritium.cross_entropy_backward(inp["grad_out"].to(dev), z, t, lse).cpu()
            torch.cuda.synchronize()
            out[case["name"]] = rec
            print(case["name"], float(rec["loss"]))
            continue
        h = inp["hidden"].to(dev)
        w = inp["weight"].to(dev)
        t = inp["target"].to(dev)
        loss, lse = ref_ce._linear_cross_entropy_forward(h, w, t)
        rec = {"loss": loss.cpu(), "lse": lse.cpu()}
        if case["grads"]:
            hg = h.clone().requires_grad_(True)
            wg = w.clone().requires_grad_(True)
            l2 = tritium.linear_cross_entropy(hg, wg, t)
            l2.backward(inp["grad_out"].to(dev))
            rec["dx"], rec["dw"] = hg.grad.cpu(), wg.grad.cpu()
            dx2, dw2 = tritium.linear_cross_entropy_backward(inp["grad_out"].to(dev), h, w, t, lse)
            rec["dx_direct"], rec["dw_direct"] = dx2.cpu(), dw2.cpu()
        torch.cuda.synchronize()
        out[case["name"]] = rec
        print(case["name"], float(rec["loss"]))
    torch.save(out, dest)
    print(f"wrote {dest}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--oracle", action="store_true")
    ap.add_argument("--reference", metavar="OUT")
    ap.add_argument("--reference-rmsnorm", metavar="OUT")
    a = ap.parse_args()
    if a.oracle:
        run_oracle()
    if a.reference:
        run_reference(a.reference)
    if a.reference_rmsnorm:
        run_reference_rmsnorm(a.reference_rmsnorm)
