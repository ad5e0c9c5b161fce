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


# ---- the launch plan (host arithmetic of the library; no device needed) ------------------------------
import ctypes  # noqa: E402

from helion_b200 import _lib  # noqa: E402

RING, REGISTER, WIDE = 0, 1, 2
ELEM = {_lib.DTYPE_BF16: 2, _lib.DTYPE_F16: 2, _lib.DTYPE_F32: 4}


def _plan(n_rows, hidden, dtype, op, aligned=1, sm_count=148):
    out = (ctypes.c_int64 * 8)()
    assert _lib.lib().lce_rmsnorm_plan(n_rows, hidden, dtype, op, aligned, sm_count, out) == 0
    return dict(zip(("form", "vpt", "threads", "rows", "ctas", "stages", "smem", "grid"), out))


@pytest.mark.parametrize("dtype", [_lib.DTYPE_BF16, _lib.DTYPE_F32])
@pytest.mark.parametrize("op", [0, 1, 2, 3])
def test_launch_plan_invariants(dtype, op):
    """For every width the reference's tests use and a sweep around the form boundaries: the threads of a
    CTA cover the row, the ring fits the shared memory of an SM with at least two stages, the backward never
    launches more CTAs than it has partial dweight rows, and the workspace covers them."""
    L = _lib.lib()
    vec = 16 // ELEM[dtype]
    n_streams = (1, 2, 2, 3)[op]
    widths = [8, 64, 100, 256, 520, 1024, 1536, 2048, 2560, 3072, 3584, 4096, 5120, 6144, 8192, 11008, 16384, 16392,
              32768, 65536]
    for hidden in widths:
        for n_rows in (1, 7, 128, 4097, 16384, 1 << 20):
            p = _plan(n_rows, hidden, dtype, op)
            nvec = -(-hidden // vec)
            assert p["threads"] % 32 == 0 and 32 <= p["threads"] <= 256
            assert 1 <= p["grid"] <= n_rows
            if p["form"] == WIDE:
                assert nvec > 8 * 256
                continue
            assert p["vpt"] in (1, 2, 4, 8) and p["vpt"] * p["threads"] >= nvec and p["rows"] in (1, 2, 4, 8)
            if p["form"] == RING:
                assert hidden % vec == 0 and 2 <= p["stages"] <= 4 and 2 <= p["ctas"] <= 8
                assert p["smem"] == p["stages"] * p["rows"] * n_streams * hidden * ELEM[dtype] <= 100 * 1024
                assert p["ctas"] * (p["smem"] + 3 * 1024) <= 228 * 1024  # what an SM has, static and reserved included
                assert p["grid"] <= 148 * p["ctas"]
            if op >= 2:
                assert p["grid"] <= 592
                ws = L.lce_rmsnorm_backward_workspace_bytes(n_rows, hidden, dtype)
                assert ws >= p["grid"] * hidden * 4 + n_rows * 4


def test_launch_plan_forms():
    bf16 = _lib.DTYPE_BF16
    # plain forward: the ring from 8 KB rows and 16 MiB of input, registers below; the residual form never
    assert _plan(16384, 4096, bf16, 0)["form"] == RING and _plan(16384, 2048, bf16, 0)["form"] == REGISTER
    assert _plan(1024, 4096, bf16, 0)["form"] == REGISTER and _plan(16384, 4096, bf16, 1)["form"] == REGISTER
    # backward: the ring whenever 16-byte copies are legal
    assert _plan(1, 1024, bf16, 2)["form"] == RING and _plan(16384, 4096, bf16, 3)["form"] == RING
    assert _plan(16, 100, bf16, 2)["form"] == REGISTER and _plan(16, 1024, bf16, 2, aligned=0)["form"] == REGISTER
    # rows beyond 256 threads x 8 vectors
    assert _plan(4, 16392, bf16, 0)["form"] == WIDE and _plan(4, 11008, _lib.DTYPE_F32, 2)["form"] == WIDE
    # Llama-3 width: 256 threads x 2 vectors; 4 KB rows with several tensors streaming in: 128 x 2
    p = _plan(16384, 4096, bf16, 2)
    assert (p["vpt"], p["threads"], p["rows"], p["ctas"], p["stages"]) == (2, 256, 2, 2, 3)
    assert (_plan(32768, 2048, bf16, 2)["vpt"], _plan(32768, 2048, bf16, 2)["threads"]) == (2, 128)
    assert (_plan(32768, 2048, bf16, 0)["vpt"], _plan(32768, 2048, bf16, 0)["threads"]) == (1, 256)
    out = (ctypes.c_int64 * 8)()
    assert _lib.lib().lce_rmsnorm_plan(0, 1024, bf16, 0, 1, 148, out) == 1  # invalid argument
    assert _lib.lib().lce_rmsnorm_plan(4, 1024, 9, 0, 1, 148, out) == 1
