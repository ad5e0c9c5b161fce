"""Parity of the RMSNorm / residual RMSNorm kernels with the oracle and with what the reference's own
kernels returned on a B200. GPU only; every call goes through the C ABI."""

from __future__ import annotations

import importlib.util
from pathlib import Path

import pytest
import torch

import helion_b200
from helion_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
HIDDEN_SIZES = [1024, 1536, 2048, 2560, 3072, 3584, 4096, 5120, 6144, 8192, 11008]
DEV = "cuda"


def tolerances(dtype: torch.dtype, accumulated: bool = False) -> tuple[float, float]:
    """(rtol, atol) of the reference's own tests (tests/tritium/test_rmsnorm.py:52-63)."""
    if dtype == torch.float32:
        return (2e-4, 2e-4) if accumulated else (2e-5, 2e-5)
    return (2e-2, 2e-2) if dtype == torch.float16 else (3e-2, 3e-2)


def close(actual, expected, accumulated=False):
    rtol, atol = tolerances(actual.dtype, accumulated)
    torch.testing.assert_close(actual.cpu(), expected.cpu().to(actual.dtype), rtol=rtol, atol=atol)


def ulp_close(actual, expected, ulps=1.0):
    """Agreement to `ulps` units in the last place of the 16-bit storage dtype (plus a matching atol). For
    fp32 the unit is 2^-18: the row sum of up to 65536 squares is formed in a different order."""
    eps = {torch.float32: 2.0 ** -18, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}[actual.dtype]
    torch.testing.assert_close(actual.cpu().float(), expected.cpu().float(), rtol=ulps * eps, atol=ulps * eps)


def fwd_ref(x, w, eps=1e-6):
    return oracle.restated_rmsnorm_forward(x.cpu(), w.cpu(), eps)["out"]


def bwd_ref(dy, x, w, eps=1e-6):
    r = oracle.restated_rmsnorm_backward(dy.cpu(), x.cpu(), w.cpu(), eps)
    return r["dx"], r["dweight"]


# ---- the reference's own tests, restated (tests/tritium/test_rmsnorm.py:76-321) ----------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden_size", HIDDEN_SIZES)
@pytest.mark.parametrize("n_rows", [1, 16, 128])
def test_forward_and_backward(dtype, hidden_size, n_rows):
    x = torch.randn(n_rows, hidden_size, device=DEV, dtype=dtype)
    w = torch.randn(hidden_size, device=DEV, dtype=dtype)
    dy = torch.randn_like(x)
    close(helion_b200.rmsnorm(x, w), fwd_ref(x, w))
    dx, dw = helion_b200.rmsnorm_backward(dy, x, w)
    ref_dx, ref_dw = bwd_ref(dy, x, w)
    close(dx, ref_dx)
    close(dw, ref_dw, accumulated=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden_size", [1024, 4096, 11008])
@pytest.mark.parametrize("n_rows", [1, 16, 128])
def test_autograd(dtype, hidden_size, n_rows):
    x = torch.randn(n_rows, hidden_size, device=DEV, dtype=dtype, requires_grad=True)
    w = torch.randn(hidden_size, device=DEV, dtype=dtype, requires_grad=True)
    dy = torch.randn_like(x)
    helion_b200.rmsnorm(x, w).backward(dy)
    ref_dx, ref_dw = bwd_ref(dy, x.detach(), w.detach())
    close(x.grad, ref_dx)
    close(w.grad, ref_dw, accumulated=True)


def test_autograd_accepts_non_contiguous_grad_output():
    x = torch.randn(16, 1024, device=DEV, requires_grad=True)
    w = torch.randn(1024, device=DEV, requires_grad=True)
    dy = torch.randn(1024, 16, device=DEV).T
    assert not dy.is_contiguous()
    helion_b200.rmsnorm(x, w).backward(dy)
    ref_dx, ref_dw = bwd_ref(dy, x.detach(), w.detach())
    close(x.grad, ref_dx)
    close(w.grad, ref_dw, accumulated=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden_size", [1024, 4096, 11008])
@pytest.mark.parametrize("n_rows", [1, 16, 128])
def test_residual_forward_and_autograd(dtype, hidden_size, n_rows):
    x = torch.randn(n_rows, hidden_size, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(n_rows, hidden_size, device=DEV, dtype=dtype, requires_grad=True)
    w = torch.randn(hidden_size, device=DEV, dtype=dtype, requires_grad=True)
    dy, dz = torch.randn_like(x), torch.randn_like(x)
    with torch.no_grad():
        out0, z0 = helion_b200.residual_rmsnorm(x, r, w)
    out, z = helion_b200.residual_rmsnorm(x, r, w)
    assert torch.equal(out, out0) and torch.equal(z, z0)  # the autograd path runs the same kernel
    ref = oracle.restated_rmsnorm_forward(x.detach().cpu(), w.detach().cpu(), 1e-6, residual=r.detach().cpu())
    close(out, ref["out"])
    assert torch.equal(z.cpu(), ref["residual_out"])  # one rounding of an exact fp32 sum: bit-exact
    torch.autograd.backward([out, z], [dy, dz])
    b = oracle.restated_rmsnorm_backward(dy.cpu(), z.detach().cpu(), w.detach().cpu(), rstd=ref["rstd"],
                                         dresidual=dz.cpu())
    close(x.grad, b["dx"])
    assert torch.equal(x.grad, r.grad)
    close(w.grad, b["dweight"], accumulated=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_rows", [1, 16, 128, 1024, 4096, 4097])
def test_row_counts(dtype, n_rows):
    x = torch.randn(n_rows, 1024, device=DEV, dtype=dtype)
    w = torch.randn(1024, device=DEV, dtype=dtype)
    dy = torch.randn_like(x)
    close(helion_b200.rmsnorm(x, w), fwd_ref(x, w))
    dx, dw = helion_b200.rmsnorm_backward(dy, x, w)
    ref_dx, ref_dw = bwd_ref(dy, x, w)
    close(dx, ref_dx)
    close(dw, ref_dw, accumulated=True)


@pytest.mark.parametrize("hidden_size", [1024, 4096, 11008])
def test_large_dweight(hidden_size):
    x = torch.randn(4096, hidden_size, device=DEV, dtype=torch.float16)
    w = torch.randn(hidden_size, device=DEV, dtype=torch.float16)
    dy = torch.randn_like(x)
    _, dw = helion_b200.rmsnorm_backward(dy, x, w)
    close(dw, bwd_ref(dy, x, w)[1], accumulated=True)


def test_rejections_follow_the_reference():
    w = torch.randn(1024, device=DEV)
    with pytest.raises(ValueError, match="CUDA tensor"):
        helion_b200.rmsnorm(torch.randn(2, 1024), torch.randn(1024))
    with pytest.raises(ValueError, match="x must be contiguous"):
        helion_b200.rmsnorm(torch.randn(1024, 16, device=DEV).T, w)
    with pytest.raises(ValueError, match="Unsupported hidden size"):
        helion_b200.rmsnorm(torch.randn(2, 65537, device=DEV), torch.randn(65537, device=DEV))
    with pytest.raises(ValueError, match="Shape mismatch: weight"):
        helion_b200.rmsnorm(torch.randn(2, 512, device=DEV), w)
    with pytest.raises(ValueError, match="Dtype mismatch: weight"):
        helion_b200.rmsnorm(torch.randn(2, 1024, device=DEV, dtype=torch.float16), w)
    with pytest.raises(ValueError, match="Shape mismatch: residual"):
        helion_b200.residual_rmsnorm(torch.randn(2, 1024, device=DEV), torch.randn(3, 1024, device=DEV), w)
    with pytest.raises(ValueError, match="Shape mismatch: dy"):
        helion_b200.rmsnorm_backward(torch.randn(3, 1024, device=DEV), torch.randn(2, 1024, device=DEV), w)


# ---- beyond the reference's tests -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(5, 1), (7, 17), (130, 100), (3, 4, 520), (2, 16392), (3, 20000), (2, 40000),
                                   (2, 65536)])
def test_odd_widths_and_the_wide_path(dtype, shape):
    """Widths that are not a multiple of the 16-byte vector, widths past the register-resident kernels
    (more than 16384 columns) and leading dimensions, against the restated algorithm to one unit in
    the last place of the storage type (the summation order is the only difference)."""
    x = torch.randn(*shape, device=DEV, dtype=dtype)
    r = torch.randn(*shape, device=DEV, dtype=dtype)
    w = torch.randn(shape[-1], device=DEV, dtype=dtype)
    dy, dz = torch.randn_like(x), torch.randn_like(x)
    ref = oracle.restated_rmsnorm_forward(x.cpu(), w.cpu(), 1e-6, residual=r.cpu())
    out, z = helion_b200.residual_rmsnorm(x, r, w)
    assert torch.equal(z.cpu(), ref["residual_out"])
    ulp_close(out, ref["out"], 2)
    ulp_close(helion_b200.rmsnorm(x, w), fwd_ref(x, w), 2)
    dx, dw = helion_b200.rmsnorm_backward(dy, x, w)
    ref_dx, ref_dw = bwd_ref(dy, x, w)
    close(dx, ref_dx)
    close(dw, ref_dw, accumulated=True)


@pytest.mark.parametrize("dtype,hidden_size", [(torch.float32, 2048), (torch.float32, 2560), (torch.float32, 5120),
                                               (torch.float16, 4096), (torch.float16, 5120), (torch.float16, 11008),
                                               (torch.bfloat16, 4096), (torch.bfloat16, 5120), (torch.bfloat16, 11008)])
def test_forward_ring_kernels(dtype, hidden_size):
    """The plain forward takes the shared-memory ring only for rows of 8 KiB and more and 16 MiB of input:
    one case per dtype and vectors-per-thread variant (2, 4, 8), with a row count that leaves the last
    row group partial. The residual form of the same size stays on the register kernels."""
    elem = torch.empty((), dtype=dtype).element_size()
    n_rows = (16 << 20) // (hidden_size * elem) + 3
    x = torch.randn(n_rows, hidden_size, device=DEV, dtype=dtype)
    r = torch.randn_like(x)
    w = torch.randn(hidden_size, device=DEV, dtype=dtype)
    ulp_close(helion_b200.rmsnorm(x, w), fwd_ref(x, w), 2)
    ref = oracle.restated_rmsnorm_forward(x.cpu(), w.cpu(), 1e-6, residual=r.cpu())
    out, z = helion_b200.residual_rmsnorm(x, r, w)
    assert torch.equal(z.cpu(), ref["residual_out"])
    ulp_close(out, ref["out"], 2)


def test_unaligned_base_pointers_take_the_element_path():
    buf = torch.randn(3 * 1024 + 1, device=DEV, dtype=torch.bfloat16)
    x = buf[1:].view(3, 1024)  # 2 bytes past a 16-byte boundary
    assert x.data_ptr() % 16 != 0 and x.is_contiguous()
    w = torch.randn(1024, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(3, 1024, device=DEV, dtype=torch.bfloat16)
    ulp_close(helion_b200.rmsnorm(x, w), fwd_ref(x, w), 2)
    dx, dw = helion_b200.rmsnorm_backward(dy, x, w)
    ref_dx, ref_dw = bwd_ref(dy, x, w)
    close(dx, ref_dx)
    close(dw, ref_dw, accumulated=True)


def test_empty_batch():
    x = torch.empty(0, 256, device=DEV, dtype=torch.float16)
    w = torch.randn(256, device=DEV, dtype=torch.float16)
    assert helion_b200.rmsnorm(x, w).shape == (0, 256)
    out, z = helion_b200.residual_rmsnorm(x, x.clone(), w)
    assert out.shape == z.shape == (0, 256)
    dx, dw = helion_b200.rmsnorm_backward(x.clone(), x, w)
    assert dx.shape == (0, 256) and torch.count_nonzero(dw) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_against_float64_autograd(dtype):
    """The meaning of the op (torch autograd in float64 on the rounded inputs), not a restatement."""
    x = torch.randn(48, 768, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(48, 768, device=DEV, dtype=dtype, requires_grad=True)
    w = torch.randn(768, device=DEV, dtype=dtype, requires_grad=True)
    dy, dz = torch.randn_like(x), torch.randn_like(x)
    out, z = helion_b200.residual_rmsnorm(x, r, w)
    torch.autograd.backward([out, z], [dy, dz])
    e = oracle.rmsnorm_expression(x.detach().cpu(), w.detach().cpu(), 1e-6, r.detach().cpu(), dy=dy.cpu(),
                                  dresidual_out=dz.cpu())
    close(out, e["out"])
    close(z, e["z"])
    close(x.grad, e["dx"])
    close(w.grad, e["dweight"], accumulated=True)


def test_backward_is_deterministic():
    x = torch.randn(3000, 2048, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(2048, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    first = helion_b200.rmsnorm_backward(dy, x, w)
    for _ in range(3):
        again = helion_b200.rmsnorm_backward(dy, x, w)
        assert torch.equal(first[0], again[0]) and torch.equal(first[1], again[1])


def test_llama3_8b_shape_properties():
    """Full benchmark shape (16384 x 4096 bf16): properties that need no CPU pass over 64M elements -
    rows are independent (a slice equals the slice of the whole) and out / weight has unit RMS."""
    x = torch.randn(16384, 4096, device=DEV, dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.randn(4096, device=DEV, dtype=torch.bfloat16)
    out, z = helion_b200.residual_rmsnorm(x, r, w)
    part, zp = helion_b200.residual_rmsnorm(x[5000:5064].contiguous(), r[5000:5064].contiguous(), w)
    assert torch.equal(out[5000:5064], part) and torch.equal(z[5000:5064], zp)
    ones = torch.ones_like(w)
    rms = helion_b200.rmsnorm(z, ones).float().pow(2).mean(dim=-1).sqrt()
    torch.testing.assert_close(rms, torch.ones_like(rms), rtol=5e-3, atol=5e-3)
    dy = torch.randn_like(x)
    dx, dw = helion_b200.rmsnorm_backward(dy, z, w)
    dxp, _ = helion_b200.rmsnorm_backward(dy[5000:5064].contiguous(), z[5000:5064].contiguous(), w)
    assert torch.equal(dx[5000:5064], dxp)
    # dweight is linear in dy: dweight(dy) + dweight(-dy) = 0 exactly, dweight(2 dy) = 2 dweight(dy)
    _, dw_neg = helion_b200.rmsnorm_backward(-dy, z, w)
    assert torch.equal(dw, -dw_neg)


# ---- what the reference's kernels returned on a B200 --------------------------------------------------
FIXTURE_PATH = GOLDEN / "reference_b200_rmsnorm.pt"
FIXTURE = torch.load(FIXTURE_PATH, weights_only=False) if FIXTURE_PATH.exists() else None


@pytest.mark.skipif(FIXTURE is None, reason="reference_b200_rmsnorm.pt not committed")
@pytest.mark.parametrize("index", range(len(make_golden.rmsnorm_case_list())))
def test_against_reference_fixture(index):
    case = make_golden.rmsnorm_case_list()[index]
    rec = {k: make_golden.fixture_tensor(FIXTURE[case["name"]], k) for k in FIXTURE[case["name"]]}
    inp = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in make_golden.make_rmsnorm_inputs(case, index).items()}
    x, r, w, dy, dres, eps = (inp[k] for k in ("x", "residual", "weight", "dy", "dres", "eps"))
    ulp_close(helion_b200.rmsnorm(x, w, eps), rec["out"], 2)
    dx, dw = helion_b200.rmsnorm_backward(dy, x, w, eps)
    close(dx, rec["dx_direct"])
    close(dw, rec["dweight_direct"], accumulated=True)
    out, z = helion_b200.residual_rmsnorm(x, r, w, eps)
    ulp_close(out, rec["res_out"], 2)
    assert torch.equal(z.cpu(), rec["res_z"])
    xg, rg, wg = (t.clone().requires_grad_(True) for t in (x, r, w))
    o3, z3 = helion_b200.residual_rmsnorm(xg, rg, wg, eps)
    torch.autograd.backward([o3, z3], [dy, dres])
    close(xg.grad, rec["res_dx"])
    close(rg.grad, rec["res_dresidual"])
    close(wg.grad, rec["res_dweight"], accumulated=True)


def test_launch_counter_moves():
    before = _lib.lib().lce_launch_count()
    x = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16)
    helion_b200.rmsnorm(x, torch.ones(512, device=DEV, dtype=torch.bfloat16))
    assert _lib.lib().lce_launch_count() == before + 1
