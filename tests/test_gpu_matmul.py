"""matmul / matmul_vec on the GEMM cores: the reference's tests restated (tests/tritium/test_matmul.py)
plus LM-sized and split-K shapes. GPU only."""

from __future__ import annotations

import pytest
import torch

import helion_b200
from _helpers import reference_tolerances, scaled_max_err

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]
DEV = "cuda"


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


def _close(got, ref, dtype, accumulated=False, k=1):
    """The reference's tolerances (its tests/_utils.py:14-29). For fp32 its 1e-5 is an absolute bound on sums
    of k products of unit-variance numbers (magnitude ~ sqrt(k)): two correct fp32 evaluations with different
    summation orders differ by about eps * k, so the absolute part grows with k beyond the reference's sizes."""
    rtol, atol = reference_tolerances(dtype, accumulated)
    if dtype == torch.float32:
        atol *= max(1.0, k / 64)
    torch.testing.assert_close(got, ref, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(("m", "n", "k"), [(16, 16, 16), (64, 64, 64), (128, 256, 32), (33, 17, 9)])
def test_matmul_forward(dtype, m, n, k):
    a = torch.randn(m, k, device=DEV, dtype=dtype)
    b = torch.randn(k, n, device=DEV, dtype=dtype)
    _close(helion_b200.matmul(a, b), torch.matmul(a.float(), b.float()).to(dtype), dtype, k=k)


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_accepts_non_contiguous_second_input(dtype):
    a = torch.randn(64, 64, device=DEV, dtype=dtype)
    b = torch.randn(64, 64, device=DEV, dtype=dtype).T
    assert not b.is_contiguous()
    _close(helion_b200.matmul(a, b), torch.matmul(a.float(), b.float()).to(dtype), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(("n", "k"), [(16, 16), (96, 64), (1024, 384), (65, 33)])
def test_matmul_vec_forward(dtype, n, k):
    a = torch.randn(k, device=DEV, dtype=dtype)
    b = torch.randn(k, n, device=DEV, dtype=dtype)
    _close(helion_b200.matmul_vec(a, b), torch.matmul(a.float(), b.float()).to(dtype), dtype, k=k)
    bt = torch.randn(n, k, device=DEV, dtype=dtype).T
    _close(helion_b200.matmul_vec(a, bt), torch.matmul(a.float(), bt.float()).to(dtype), dtype, k=k)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(("m", "n", "k"), [(16, 16, 16), (64, 32, 48), (33, 17, 9)])
def test_matmul_autograd(dtype, m, n, k):
    a = torch.randn(m, k, device=DEV, dtype=dtype, requires_grad=True)
    b = torch.randn(k, n, device=DEV, dtype=dtype, requires_grad=True)
    dc = torch.randn(m, n, device=DEV, dtype=dtype)
    helion_b200.matmul(a, b).backward(dc)
    ar = a.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True)
    torch.matmul(ar, br).backward(dc.float())
    _close(a.grad, ar.grad.to(dtype), dtype, accumulated=True)
    _close(b.grad, br.grad.to(dtype), dtype, accumulated=True)


def test_matmul_vec_autograd_and_no_grad_path():
    a = torch.randn(64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(64, 96, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    helion_b200.matmul_vec(a, b).sum().backward()
    assert a.grad.shape == (64,) and b.grad.shape == (64, 96)
    with torch.no_grad():
        assert not helion_b200.matmul(a[None], b).requires_grad


def test_matmul_rejects_bad_inputs():
    with pytest.raises(ValueError, match="CUDA tensor"):
        helion_b200.matmul(torch.randn(4, 4), torch.randn(4, 4))
    a = torch.randn(4, 5, device=DEV)
    with pytest.raises(ValueError, match="Shape mismatch"):
        helion_b200.matmul(a, torch.randn(4, 5, device=DEV))
    with pytest.raises(ValueError, match="Dtype mismatch"):
        helion_b200.matmul(a, torch.randn(5, 4, device=DEV, dtype=torch.float16))
    with pytest.raises(ValueError, match="Shape mismatch"):
        helion_b200.matmul_vec(torch.randn(4, device=DEV), torch.randn(5, 4, device=DEV))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(("m", "n", "k"), [(512, 4096, 4096), (100, 264, 12800), (2048, 1000, 520), (1, 8192, 4096),
                                           (300, 72, 1000)])
def test_larger_shapes_all_operand_layouts(dtype, m, n, k):
    """LM-sized products, a short-M / long-K product (split along K), and unaligned pitches (CUDA cores)."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    b = torch.randn(k, n, generator=g).to(dtype).to(DEV)
    ref = a.float() @ b.float()
    for av in (a, a.t().contiguous().t()):
        for bv in (b, b.t().contiguous().t()):
            out = helion_b200.matmul(av, bv)
            assert out.dtype == dtype and scaled_max_err(out, ref) <= 8e-3
    assert torch.equal(helion_b200.matmul(a, b), helion_b200.matmul(a, b))  # fixed summation order


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(("m", "n", "k", "ldc"), [(70, 100, 64, 104), (300, 189, 128, 192), (129, 64, 72, 64), (31, 7, 64, 8)])
def test_output_pitch_wider_than_the_row_through_the_c_abi(dtype, m, n, k, ldc):
    """The C ABI takes the output pitch separately: rows of n values, ldc apart, n not a multiple of the 8 values
    a 16-byte store holds. The line-wide epilogue stores must write n values per row and leave the gap alone."""
    from helion_b200 import _lib

    L = _lib.lib()
    code = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F16
    g = torch.Generator().manual_seed(m * n + k)
    a = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    b = torch.randn(n, k, generator=g).to(dtype).to(DEV)  # given as [n][k]: b_mn_major = 0
    c = torch.full((m, ldc), 7.0, dtype=dtype, device=DEV)
    ws_bytes = L.lce_matmul_workspace_bytes(m, n, k, code, 0)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=DEV)
    _lib.check(L.lce_matmul(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, 0, k, 0, k, ldc, code, ws.data_ptr(),
                            ws_bytes, 0, torch.cuda.current_stream().cuda_stream), "lce_matmul")
    torch.cuda.synchronize()
    ref = a.float() @ b.float().T
    assert scaled_max_err(c[:, :n], ref) <= 8e-3
    assert torch.all(c[:, n:] == 7.0), "values beyond the row's end were overwritten"
