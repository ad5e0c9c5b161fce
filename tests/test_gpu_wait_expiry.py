"""A bounded device wait is made to run out, and the kernel must come back with a code, not hang.

Every mbarrier wait in the kernels has a time limit; past it the role records a code in the device status
word, the producer lets its copies land, tensor memory is freed and the kernel returns. Here the limit is
shortened to a few milliseconds and the producer announces 16 bytes more on its first barrier than its
copies deliver: every copy lands, the barrier never completes, no tensor-core instruction is ever issued,
and nothing is in flight when the kernel exits. Nothing traps or faults; the context stays usable, which
the test proves by running the same launches normally afterwards. GPU only."""

from __future__ import annotations

import pytest
import torch

from helion_b200 import _lib, norm_ops, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
LIMIT_NS = 3_000_000  # 3 ms


@pytest.fixture
def short_waits():
    L = _lib.lib()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    _lib.check(L.lce_debug_wait_test(LIMIT_NS, 16), "lce_debug_wait_test")
    try:
        yield
    finally:
        _lib.check(L.lce_debug_wait_test(0, 0), "lce_debug_wait_test")
        _lib.device_status()  # leave the status word clear for the tests that follow


def test_gemm_wait_runs_out_with_a_status_code_and_the_next_launch_is_fine(short_waits):
    g = torch.Generator().manual_seed(1)
    a = torch.randn(128, 64, generator=g).bfloat16().to(DEV)
    b = torch.randn(256, 64, generator=g).bfloat16().to(DEV)
    ops.debug_gemm(a, b, False, False, one_cta=True)  # one tile, one k block, cta_group::1
    torch.cuda.synchronize()  # returns: the waits gave up after 3 ms each
    # whichever role's timer ran out first has its code in the word: producer 101, issuer 102, epilogue 103
    assert _lib.device_status(clear=False) in (101, 102, 103)
    assert _lib.device_status() in (101, 102, 103)  # read and clear
    assert _lib.device_status() == 0
    _lib.check(_lib.lib().lce_debug_wait_test(0, 0), "lce_debug_wait_test")
    out = ops.debug_gemm(a, b, False, False, one_cta=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(out, a.float() @ b.float().T, rtol=1e-5, atol=1e-4)
    assert _lib.device_status() == 0


def test_rmsnorm_ring_wait_runs_out_with_code_111(short_waits):
    # the RMSNorm backward streams its rows through the shared-memory ring (the plain forward of rows this wide
    # runs on the one-row-per-CTA kernel, which has no waits)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2048, 4096, generator=g).bfloat16().to(DEV)
    dy = torch.randn(2048, 4096, generator=g).bfloat16().to(DEV)
    w = torch.randn(4096, generator=g).bfloat16().to(DEV)
    norm_ops.rmsnorm_backward(dy, x, w)
    torch.cuda.synchronize()
    assert _lib.device_status() == 111
    assert _lib.device_status() == 0
    _lib.check(_lib.lib().lce_debug_wait_test(0, 0), "lce_debug_wait_test")
    dx, dweight = norm_ops.rmsnorm_backward(dy, x, w)
    torch.cuda.synchronize()
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(dim=-1, keepdim=True) + 1e-6) * wr).backward(dy.float())
    torch.testing.assert_close(dx.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dweight.float(), wr.grad, rtol=2e-2, atol=0.5)
    assert _lib.device_status() == 0
