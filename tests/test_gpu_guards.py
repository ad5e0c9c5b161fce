"""Memory-safety check without a sanitizer: every output and the workspace of a C-ABI call sit between guard
zones filled with a byte pattern; the call gets the exact sizes the library asks for, and afterwards the
guards must be untouched. Ragged shapes, both kernel families. GPU only."""

from __future__ import annotations

import pytest
import torch

from helion_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda"
GUARD = 4096
PATTERN = 0x5A
CODES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16, torch.float32: _lib.DTYPE_F32}


class Guarded:
    """`nbytes` of device memory (256-byte aligned) with GUARD pattern bytes on either side."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        body = (self.nbytes + 255) // 256 * 256
        self.raw = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device=DEV)
        assert self.raw.data_ptr() % 256 == 0
        self.ptr = self.raw.data_ptr() + GUARD

    def view(self, dtype: torch.dtype, shape) -> torch.Tensor:
        return self.raw[GUARD:GUARD + self.nbytes].view(dtype).view(shape)

    def intact(self) -> bool:
        head = self.raw[:GUARD]
        tail = self.raw[GUARD + self.nbytes:]  # includes the round-up slack behind the payload
        return bool((head == PATTERN).all()) and bool((tail == PATTERN).all())


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("dtype,flags", [(torch.bfloat16, 0), (torch.bfloat16, _lib.FLAG_FORCE_SIMT), (torch.float32, 0)])
@pytest.mark.parametrize("shape", [(129, 64, 257), (1, 72, 1000), (300, 128, 4100)])
def test_fused_loss_forward_and_backward_stay_inside_their_buffers(dtype, flags, shape):
    n, h, v = shape
    if h % 8 and dtype != torch.float32 and flags == 0:
        flags = _lib.FLAG_FORCE_SIMT  # the tensor-core path needs 16-byte row pitches
    L = _lib.lib()
    code = CODES[dtype]
    elem = torch.empty((), dtype=dtype).element_size()
    x = torch.randn(n, h, device=DEV).to(dtype)
    w = (torch.randn(v, h, device=DEV) * 0.1).to(dtype)
    t = torch.randint(0, v, (n,), device=DEV)
    lse, loss = Guarded(n * 4), Guarded(4)
    ws = Guarded(L.lce_forward_loss_workspace_bytes(n, h, v, code, flags))
    _lib.check(L.lce_forward_loss(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, n, h, v, code, -100, _lib.REDUCTION_MEAN,
                                  lse.ptr, loss.ptr, None, ws.ptr, ws.nbytes, flags, stream()), "lce_forward_loss")
    go = torch.tensor(1.0, device=DEV)
    dx, dw = Guarded(n * h * elem), Guarded(v * h * elem)
    bws = Guarded(L.lce_backward_workspace_bytes(n, h, v, code, flags, 0))
    _lib.check(L.lce_backward(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, lse.ptr, go.data_ptr(), n, h, v, 0, code,
                              -100, _lib.REDUCTION_MEAN, dx.ptr, dw.ptr, bws.ptr, bws.nbytes, flags, 0, None, None,
                              None, stream()), "lce_backward")
    tok, lp = Guarded(n * 8), Guarded(n * 4)
    gws = Guarded(L.lce_forward_workspace_bytes(n, h, v, code, flags))
    _lib.check(L.lce_greedy_head(x.data_ptr(), w.data_ptr(), n, h, v, 0, code, tok.ptr, lp.ptr, None, gws.ptr,
                                 gws.nbytes, flags, stream()), "lce_greedy_head")
    torch.cuda.synchronize()
    for name, buf in (("lse", lse), ("loss", loss), ("forward workspace", ws), ("dx", dx), ("dw", dw),
                      ("backward workspace", bws), ("token", tok), ("logprob", lp), ("greedy workspace", gws)):
        assert buf.intact(), name
    assert torch.isfinite(loss.view(torch.float32, ())) and torch.isfinite(dx.view(dtype, (n, h)).float()).all()
    assert int(tok.view(torch.int64, (n,)).max()) < v
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(5, 17), (130, 100), (37, 1024), (4100, 4096), (3, 11008), (2, 20000)])
def test_rmsnorm_stays_inside_its_buffers(dtype, shape):
    n, h = shape
    L = _lib.lib()
    code = CODES[dtype]
    elem = torch.empty((), dtype=dtype).element_size()
    x, r, dy = (torch.randn(n, h, device=DEV).to(dtype) for _ in range(3))
    w = torch.randn(h, device=DEV).to(dtype)
    out, z, rstd = Guarded(n * h * elem), Guarded(n * h * elem), Guarded(n * 4)
    _lib.check(L.lce_rmsnorm_forward(x.data_ptr(), r.data_ptr(), w.data_ptr(), out.ptr, z.ptr, rstd.ptr, n, h, 1e-6, code,
                                     stream()), "lce_rmsnorm_forward")
    out2 = Guarded(n * h * elem)
    _lib.check(L.lce_rmsnorm_forward(x.data_ptr(), None, w.data_ptr(), out2.ptr, None, None, n, h, 1e-6, code, stream()),
               "lce_rmsnorm_forward")
    dx, dwt = Guarded(n * h * elem), Guarded(h * elem)
    ws = Guarded(L.lce_rmsnorm_backward_workspace_bytes(n, h, code))
    _lib.check(L.lce_rmsnorm_backward(dy.data_ptr(), z.ptr, w.data_ptr(), rstd.ptr, r.data_ptr(), dx.ptr, dwt.ptr, n, h,
                                      0.0, code, ws.ptr, ws.nbytes, stream()), "lce_rmsnorm_backward")
    torch.cuda.synchronize()
    for name, buf in (("out", out), ("residual_out", z), ("rstd", rstd), ("plain out", out2), ("dx", dx),
                      ("dweight", dwt), ("workspace", ws)):
        assert buf.intact(), name
    assert torch.isfinite(dx.view(dtype, (n, h)).float()).all() and torch.isfinite(dwt.view(dtype, (h,)).float()).all()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 17), (64, 1000), (9, 40000)])
def test_plain_cross_entropy_stays_inside_its_buffers(dtype, shape):
    n, v = shape
    L = _lib.lib()
    code = CODES[dtype]
    elem = torch.empty((), dtype=dtype).element_size()
    z = torch.randn(n, v, device=DEV).to(dtype)
    t = torch.randint(0, v, (n,), device=DEV)
    lse, loss, dz = Guarded(n * 4), Guarded(4), Guarded(n * v * elem)
    ws = Guarded(L.lce_ce_workspace_bytes(n, v, code))
    _lib.check(L.lce_ce_forward(z.data_ptr(), t.data_ptr(), 1, n, v, code, -100, _lib.REDUCTION_MEAN, lse.ptr, loss.ptr,
                                None, ws.ptr, ws.nbytes, stream()), "lce_ce_forward")
    go = torch.tensor(1.0, device=DEV)
    _lib.check(L.lce_ce_backward(z.data_ptr(), t.data_ptr(), 1, lse.ptr, go.data_ptr(), n, v, code, -100,
                                 _lib.REDUCTION_MEAN, dz.ptr, ws.ptr, ws.nbytes, stream()), "lce_ce_backward")
    torch.cuda.synchronize()
    for name, buf in (("lse", lse), ("loss", loss), ("dlogits", dz), ("workspace", ws)):
        assert buf.intact(), name
    assert torch.isfinite(loss.view(torch.float32, ()))
