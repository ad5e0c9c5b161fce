"""Swap this package's op into an importable reference ``tritium`` package.

The reference's callers (``examples/common.py:125``, ``benchmarks/bench_linear_cross_entropy.py:67,114``,
its tests) look ``linear_cross_entropy`` / ``linear_cross_entropy_backward`` up on the module at call
time, so rebinding the attribute on the three modules that export the names
(``tritium/__init__.py:18-19``, ``tritium/ops/__init__.py:8-9``, ``tritium/ops/cross_entropy.py``) is
enough to make training scripts, examples and tests run on the sm_100a kernels unchanged.
"""

from __future__ import annotations

import importlib
from types import ModuleType

from . import ops

NAMES = ("linear_cross_entropy", "linear_cross_entropy_backward")
MODULES = ("tritium", "tritium.ops", "tritium.ops.cross_entropy")

_saved: dict[tuple[str, str], object] = {}


def _targets(root: ModuleType | None) -> list[ModuleType]:
    if root is not None:
        mods = [root]
        sub = getattr(root, "ops", None)
        if isinstance(sub, ModuleType):
            mods.append(sub)
            leaf = getattr(sub, "cross_entropy", None)
            if isinstance(leaf, ModuleType):
                mods.append(leaf)
        return mods
    return [importlib.import_module(name) for name in MODULES]


def install(tritium_module: ModuleType | None = None) -> list[str]:
    """Rebind the two names on ``tritium`` and its op modules; returns the rebound ``module.name`` list."""
    rebound = []
    for mod in _targets(tritium_module):
        for name in NAMES:
            if not hasattr(mod, name):
                continue
            key = (mod.__name__, name)
            if key not in _saved:
                _saved[key] = getattr(mod, name)
            setattr(mod, name, getattr(ops, name))
            rebound.append(f"{mod.__name__}.{name}")
    return rebound


def uninstall(tritium_module: ModuleType | None = None) -> None:
    """Put back whatever ``install`` replaced."""
    for mod in _targets(tritium_module):
        for name in NAMES:
            key = (mod.__name__, name)
            if key in _saved:
                setattr(mod, name, _saved.pop(key))
