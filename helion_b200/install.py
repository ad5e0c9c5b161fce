"""Swap this package's op into an importable reference ``tritium`` package.

The reference's callers (``examples/common.py:125``, ``benchmarks/bench_linear_cross_entropy.py:67,114``,
its tests) look ``linear_cross_entropy`` / ``linear_cross_entropy_backward`` up on the module at call
time, so rebinding the attribute on the three modules that export the names
(``tritium/__init__.py:18-19``, ``tritium/ops/__init__.py:8-9``, ``tritium/ops/cross_entropy.py``) is
enough to make training scripts, examples and tests run on the sm_100a kernels unchanged.
"""

from __future__ import annotations

import importlib
import sys
from types import ModuleType

from . import ce_ops, matmul_ops, norm_ops, ops, optim_ops

# the fused op (the path this package exists for), the plain op of the same reference file, and the
# matrix product that runs on the same GEMM cores
NAMES = ("linear_cross_entropy", "linear_cross_entropy_backward", "cross_entropy", "cross_entropy_backward",
         "matmul", "matmul_vec", "adamw_step", "rmsnorm", "residual_rmsnorm", "rmsnorm_backward")
_IMPL = {
    "adamw_step": optim_ops.adamw_step,
    "rmsnorm": norm_ops.rmsnorm,
    "residual_rmsnorm": norm_ops.residual_rmsnorm,
    "rmsnorm_backward": norm_ops.rmsnorm_backward,
    "matmul": matmul_ops.matmul,
    "matmul_vec": matmul_ops.matmul_vec,
    "linear_cross_entropy": ops.linear_cross_entropy,
    "linear_cross_entropy_backward": ops.linear_cross_entropy_backward,
    "cross_entropy": ce_ops.cross_entropy,
    "cross_entropy_backward": ce_ops.cross_entropy_backward,
}
MODULES = ("tritium", "tritium.ops", "tritium.ops.cross_entropy", "tritium.ops.matmul", "tritium.ops.adamw",
           "tritium.ops.rmsnorm")

_saved: dict[tuple[str, str], object] = {}


def _targets(root: ModuleType | None) -> list[ModuleType]:
    # `tritium.ops.cross_entropy` as an attribute is the re-exported plain cross_entropy FUNCTION
    # (tritium/ops/__init__.py), so the submodules are taken from the import system, not via getattr.
    base = MODULES[0] if root is None else root.__name__
    mods = [importlib.import_module(base) if root is None else root]
    # (the same holds for `tritium.ops.matmul` and `tritium.ops.rmsnorm`)
    for suffix in (".ops", ".ops.cross_entropy", ".ops.matmul", ".ops.adamw", ".ops.rmsnorm"):
        name = base + suffix
        mod = sys.modules.get(name)
        if mod is None:
            try:
                mod = importlib.import_module(name)
            except ImportError:
                continue
        mods.append(mod)
    return mods


def install(tritium_module: ModuleType | None = None) -> list[str]:
    """Rebind the cross-entropy and matmul names on ``tritium`` and its op modules; returns the rebound
    ``module.name`` list. (On ``tritium.ops`` the attribute ``cross_entropy`` is the function, which
    shadows the submodule of the same name; it is the function that gets replaced.)"""
    rebound = []
    for mod in _targets(tritium_module):
        for name in NAMES:
            if not hasattr(mod, name):
                continue
            key = (mod.__name__, name)
            if key not in _saved:
                _saved[key] = getattr(mod, name)
            setattr(mod, name, _IMPL[name])
            rebound.append(f"{mod.__name__}.{name}")
    return rebound


def uninstall(tritium_module: ModuleType | None = None) -> None:
    """Put back whatever ``install`` replaced."""
    for mod in _targets(tritium_module):
        for name in NAMES:
            key = (mod.__name__, name)
            if key in _saved:
                setattr(mod, name, _saved.pop(key))
