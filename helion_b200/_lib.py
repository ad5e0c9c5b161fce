"""ctypes binding of libhelion_lce.so (C ABI: include/helion_lce.h).

There is no fallback: if the shared library cannot be loaded (or built), every op raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint, c_void_p
from functools import lru_cache

from . import build as _build

DTYPE_BF16, DTYPE_F16, DTYPE_F32 = 0, 1, 2
REDUCTION_NONE, REDUCTION_MEAN, REDUCTION_SUM = 0, 1, 2
FLAG_FORCE_SIMT, FLAG_FORCE_TC, FLAG_DX_F32, FLAG_NO_DX, FLAG_NO_DW, FLAG_ONE_CTA = 1, 2, 4, 8, 16, 32

REDUCTIONS = {"none": REDUCTION_NONE, "mean": REDUCTION_MEAN, "sum": REDUCTION_SUM}

# name -> (restype, argtypes); mirrors include/helion_lce.h declaration by declaration
SIGNATURES = {
    "lce_version": (c_int, []),
    "lce_strerror": (c_char_p, [c_int]),
    "lce_last_cuda_error": (c_char_p, []),
    "lce_launch_count": (ctypes.c_ulonglong, []),
    "lce_device_status": (c_int, [ctypes.POINTER(c_int), c_int]),
    "lce_forward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_uint]),
    "lce_forward_stats": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                                  c_int, c_void_p, c_void_p, c_size_t, c_uint, c_void_p]),
    "lce_forward_stats_static_capacity": (c_size_t, []),
    "lce_forward_stats_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                                         c_int, c_void_p, c_uint, c_void_p]),
    "lce_finalize_workspace_bytes": (c_size_t, [c_int64]),
    "lce_finalize": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_size_t, c_void_p]),
    "lce_forward_loss_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_uint]),
    "lce_forward_loss": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int64,
                                 c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_uint, c_void_p]),
    "lce_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_uint, c_size_t]),
    "lce_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                             c_int64, c_int64, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
                             c_uint, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lce_dx_reduce_gather": (c_int, [c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "lce_dx_reduce_slice": (c_int, [c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "lce_backward_plan": (c_int, [c_int64, c_int64, c_int64, c_int, c_uint, c_size_t, c_void_p, c_void_p,
                                  ctypes.POINTER(c_int64)]),
    "lce_ce_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "lce_ce_forward": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lce_ce_backward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64,
                                c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lce_matmul_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_uint]),
    "lce_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int64, c_int, c_int64,
                           c_int64, c_int, c_void_p, c_size_t, c_uint, c_void_p]),
    "lce_adamw_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, ctypes.c_float, ctypes.c_float,
                               ctypes.c_float, ctypes.c_float, ctypes.c_float, c_int64, c_void_p, c_void_p]),
    "lce_sumsq_workspace_bytes": (c_size_t, []),
    "lce_sumsq": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "lce_greedy_head": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_size_t, c_uint, c_void_p]),
    "lce_topk_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_uint]),
    "lce_topk_head": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, ctypes.c_float,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_uint, c_void_p]),
    "lce_rmsnorm_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                    ctypes.c_float, c_int, c_void_p]),
    "lce_rmsnorm_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "lce_rmsnorm_plan": (c_int, [c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "lce_rmsnorm_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int64, ctypes.c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "lce_set_tuning": (None, [c_int, c_int, c_int]),
    "lce_debug_wait_test": (c_int, [ctypes.c_ulonglong, c_uint]),
    "lce_debug_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int,
                               c_uint, c_void_p]),
}


class PeerScatter(ctypes.Structure):
    """``lce_peer_scatter`` of include/helion_lce.h."""

    _fields_ = [("staging", c_void_p * 8), ("rank", c_int), ("world", c_int)]


class LceError(RuntimeError):
    """A nonzero status from the C ABI."""


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    try:
        path = _build.build_library()
    except Exception as exc:  # noqa: BLE001 - surfaced verbatim: there is no other code path
        raise RuntimeError(
            "helion_b200: libhelion_lce.so is missing and could not be built; "
            "this package has no fallback path"
        ) from exc
    handle = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().lce_strerror(code).decode()
        if code == 5:  # LCE_ERR_CUDA: say which CUDA error
            msg += f" [{lib().lce_last_cuda_error().decode()}]"
        raise LceError(f"{what} failed: {msg} (code {code})")


def device_status(clear: bool = True) -> int:
    out = c_int(0)
    check(lib().lce_device_status(ctypes.byref(out), 1 if clear else 0), "lce_device_status")
    return out.value
