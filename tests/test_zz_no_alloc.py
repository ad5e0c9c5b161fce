"""lce_forward_stats_static: the forward-statistics entry point for hosts that cannot provide scratch.

Some processes that embed this library have given away all of their device memory before the first
loss is computed (one big arena handed to their own allocator at start-up) or run the loss from a thread
that must never stall on an allocation. For them the library carries a fixed 16 MiB scratch array of
its own, and this entry point uses it instead of a caller-supplied workspace. The test drives it through
the C ABI exactly as such a host would (inputs and the output tensor exist beforehand; the call gets
no workspace) and requires the same numbers as lce_forward_stats on two calls in a row, the second on a
different problem so that whatever the first call left in the shared array is still there.

The file name sorts last on purpose: if this test fails, every other test has already run.
"""

from __future__ import annotations

import pytest
import torch

from helion_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _problem(n, h, v, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, h, generator=g).to(dtype).to(DEV)
    w = (torch.randn(v, h, generator=g) * 0.1).to(dtype).to(DEV)
    t = torch.randint(0, v, (n,), generator=g).to(DEV)
    return x, w, t


def _with_workspace(x, w, t, code, flags=0):
    L = _lib.lib()
    n, h = x.shape
    v = w.shape[0]
    stats = torch.empty(3, n, device=DEV)
    ws = torch.empty(L.lce_forward_workspace_bytes(n, h, v, code, flags), dtype=torch.uint8, device=DEV)
    _lib.check(L.lce_forward_stats(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, n, h, v, 0, code, stats.data_ptr(),
                                   ws.data_ptr(), ws.numel(), flags, torch.cuda.current_stream().cuda_stream),
               "lce_forward_stats")
    return stats


def _static(x, w, t, code, stats, flags=0):
    n, h = x.shape
    return _lib.lib().lce_forward_stats_static(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, n, h, w.shape[0], 0, code,
                                               stats.data_ptr(), flags, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype,code,flags", [(torch.bfloat16, _lib.DTYPE_BF16, 0),
                                              (torch.float32, _lib.DTYPE_F32, 0),
                                              (torch.float16, _lib.DTYPE_F16, _lib.FLAG_FORCE_SIMT)])
def test_static_scratch_entry_point_matches_the_workspace_entry_point_twice(dtype, code, flags):
    # second problem is smaller in both directions: stale entries of the first call surround it
    first = _problem(700, 256, 5000, dtype, seed=21)
    second = _problem(130, 136, 900, dtype, seed=22)
    for x, w, t in (first, second):
        expected = _with_workspace(x, w, t, code, flags)
        got = torch.full((3, x.shape[0]), float("nan"), device=DEV)  # output exists before the call
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert _static(x, w, t, code, got, flags) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels, same order of operations: identical up to the loss tolerance of this suite
        torch.testing.assert_close(got, expected, rtol=1e-6, atol=0.0)
    assert _lib.device_status() == 0


def test_static_scratch_entry_point_rejects_problems_beyond_its_array():
    L = _lib.lib()
    assert L.lce_forward_stats_static_capacity() == 16 << 20
    x, w, t = _problem(64, 64, 512, torch.bfloat16, seed=23)
    stats = torch.empty(3, 8192, device=DEV)
    launches = L.lce_launch_count()
    # claim the Llama-3 head shape: 501 tiles x 3 x 8192 rows x 4 bytes = 49 MB of partials > 16 MiB
    rc = L.lce_forward_stats_static(x.data_ptr(), w.data_ptr(), t.data_ptr(), 1, 8192, 4096, 128256, 0,
                                    _lib.DTYPE_BF16, stats.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 7 and L.lce_launch_count() == launches  # refused before anything was launched
    assert b"16 MiB" in L.lce_strerror(rc)
