"""CPU checks of the RMSNorm restatement in the oracle (against float64 autograd and against what the
reference's kernels returned on a B200) and of the host-side validators. No GPU, no compute calls."""

from __future__ import annotations

import importlib.util
from pathlib import Path

import pytest
import torch

from helion_b200 import norm_ops
from oracle import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
STORAGE_EPS = {torch.float32: 2.0 ** -18, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 8), (16, 100), (3, 5, 64)])
def test_restatement_is_the_float64_expression(dtype, shape):
    g = torch.Generator().manual_seed(31)
    x, r, dy, dz = (torch.randn(shape, generator=g).to(dtype) for _ in range(4))
    w = torch.randn(shape[-1], generator=g).to(dtype)
    e = oracle.rmsnorm_expression(x, w, 1e-6, r, dy=dy, dresidual_out=dz)
    f = oracle.restated_rmsnorm_forward(x, w, 1e-6, residual=r)
    tol = STORAGE_EPS[dtype]
    torch.testing.assert_close(f["out"].double(), e["out"], rtol=tol, atol=tol)
    torch.testing.assert_close(f["residual_out"].double(), e["z"], rtol=tol, atol=tol)
    # the kernels differentiate through the ROUNDED residual_out; the expression through the exact sum
    b = oracle.restated_rmsnorm_backward(dy, f["residual_out"], w, rstd=f["rstd"], dresidual=dz)
    loose = 4 * tol if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(b["dx"].double(), e["dx"], rtol=loose, atol=loose)
    torch.testing.assert_close(b["dweight"].double(), e["dweight"], rtol=loose, atol=loose * 4)


def test_recomputed_rstd_equals_saved_rstd():
    g = torch.Generator().manual_seed(5)
    x, dy = torch.randn(9, 40, generator=g), torch.randn(9, 40, generator=g)
    w = torch.randn(40, generator=g)
    f = oracle.restated_rmsnorm_forward(x, w, 1e-5)
    a = oracle.restated_rmsnorm_backward(dy, x, w, 1e-5)
    b = oracle.restated_rmsnorm_backward(dy, x, w, rstd=f["rstd"])
    assert torch.equal(a["dx"], b["dx"]) and torch.equal(a["dweight"], b["dweight"])


FIXTURE_PATH = GOLDEN / "reference_b200_rmsnorm.pt"
FIXTURE = torch.load(FIXTURE_PATH, weights_only=False) if FIXTURE_PATH.exists() else None


@pytest.mark.skipif(FIXTURE is None, reason="reference_b200_rmsnorm.pt not committed")
@pytest.mark.parametrize("index", range(len(make_golden.rmsnorm_case_list())))
def test_restatement_matches_reference_kernels(index):
    """Pins the restatement: the reference's Triton kernels, run on a B200, on the same seeded inputs."""
    case = make_golden.rmsnorm_case_list()[index]
    rec = {k: make_golden.fixture_tensor(FIXTURE[case["name"]], k) for k in FIXTURE[case["name"]]}
    inp = make_golden.make_rmsnorm_inputs(case, index)
    x, r, w, dy, dres, eps = (inp[k] for k in ("x", "residual", "weight", "dy", "dres", "eps"))
    tol = 2 * STORAGE_EPS[x.dtype]

    def same(a, b, scale=1.0):
        torch.testing.assert_close(a.float(), b.float(), rtol=tol * scale, atol=tol * scale)

    same(oracle.restated_rmsnorm_forward(x, w, eps)["out"], rec["out"])
    f = oracle.restated_rmsnorm_forward(x, w, eps, residual=r)
    same(f["out"], rec["res_out"])
    assert torch.equal(f["residual_out"], rec["res_z"])
    b = oracle.restated_rmsnorm_backward(dy, x, w, eps)
    for key in ("dx_direct", "dx"):
        same(b["dx"], rec[key], 4)
    n_rows = x.numel() // x.shape[-1]
    for key in ("dweight_direct", "dweight"):
        same(b["dweight"], rec[key], 4 * max(1.0, n_rows ** 0.5))
    rb = oracle.restated_rmsnorm_backward(dy, f["residual_out"], w, rstd=f["rstd"], dresidual=dres)
    same(rb["dx"], rec["res_dx"], 4)
    assert torch.equal(rec["res_dx"], rec["res_dresidual"])
    same(rb["dweight"], rec["res_dweight"], 4 * max(1.0, n_rows ** 0.5))


def test_rmsnorm_case_inputs_are_stable():
    case = make_golden.rmsnorm_case_list()[0]
    a = make_golden.make_rmsnorm_inputs(case, 0)
    b = make_golden.make_rmsnorm_inputs(case, 0)
    assert all(torch.equal(a[k], b[k]) for k in ("x", "residual", "weight", "dy", "dres"))
    assert len({c["name"] for c in make_golden.rmsnorm_case_list()}) == len(make_golden.rmsnorm_case_list())


# ---- host-side validation: the reference's messages, raised before any library call ----------------
def test_cpu_tensors_are_rejected_like_the_reference():
    with pytest.raises(ValueError, match="x must be a CUDA tensor"):
        norm_ops.rmsnorm(torch.randn(2, 8), torch.randn(8))
    with pytest.raises(ValueError, match="x must be a CUDA tensor"):
        norm_ops.residual_rmsnorm(torch.randn(2, 8), torch.randn(2, 8), torch.randn(8))
    with pytest.raises(ValueError, match="x must be a CUDA tensor"):
        norm_ops.rmsnorm_backward(torch.randn(2, 8), torch.randn(2, 8), torch.randn(8))


def test_next_pow2_limit():
    assert norm_ops._next_pow2(1) == 1 and norm_ops._next_pow2(65536) == 65536 and norm_ops._next_pow2(65537) == 131072
