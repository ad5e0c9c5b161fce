"""The reference's own test files for the ops this package replaces (linear / plain cross-entropy, matmul,
AdamW step, RMSNorm), collected UNCHANGED with the op names rebound by ``install()``: the acceptance test of the
drop-in. The files are not part of this repository; ``__graft_entry__.build()`` stages them next to the
reference install under baseline/_ref where a reference checkout exists. Skipped where they are absent."""

from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
SUITE = ROOT / "baseline" / "_ref" / "reference_tests"


@pytest.mark.parametrize("name", ["test_cross_entropy.py", "test_matmul.py", "test_adamw.py", "test_rmsnorm.py"])
def test_reference_test_file_passes_unchanged_on_the_rebound_ops(name):
    path = SUITE / "tritium" / name
    if not path.exists():
        pytest.skip("the reference's test files are not staged under baseline/_ref/reference_tests")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT / "tests"), str(ROOT), env.get("PYTHONPATH", "")])
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "reference_suite_plugin", "-p", "no:cacheprovider",
                           str(path)], cwd=str(SUITE), env=env, capture_output=True, text=True, timeout=900)
    tail = proc.stdout[-3000:] + proc.stderr[-1500:]
    assert proc.returncode == 0, tail
    passed = re.search(r"(\d+) passed", proc.stdout)
    launched = re.search(r"library kernels launched: (\d+)", proc.stdout)
    assert passed and int(passed.group(1)) > 0, tail
    assert "skipped" not in proc.stdout.splitlines()[-2] + proc.stdout.splitlines()[-1], tail
    assert launched and int(launched.group(1)) > 0, tail
