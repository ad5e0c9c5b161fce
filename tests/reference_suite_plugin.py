"""pytest plugin for running the REFERENCE's own test files against this package: loaded with
``-p reference_suite_plugin`` by tests/test_gpu_reference_suite.py. It rebinds the reference's op names to
this package's ops before the reference's test modules are imported (``helion_b200.install()``), seeds torch
before every test (the reference's tests draw unseeded inputs) and reports how many of this library's kernels
ran, so that a pass cannot come from the reference's own Triton kernels."""

from __future__ import annotations

import pytest


def pytest_configure(config):
    import helion_b200

    config._helion_rebound = helion_b200.install()


@pytest.fixture(autouse=True)
def _seed():
    import torch

    torch.manual_seed(20240607)


def pytest_terminal_summary(terminalreporter):
    from helion_b200 import _lib

    terminalreporter.write_line(f"helion_b200 rebound {len(terminalreporter.config._helion_rebound)} names; "
                                f"library kernels launched: {_lib.lib().lce_launch_count()}")
