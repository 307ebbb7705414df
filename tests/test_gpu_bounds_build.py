"""The bounds-checking build of the extension (LPLB_B200_DEBUG_BOUNDS=1) on the small cases."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_small_cases_are_clean_and_a_violation_is_recorded_not_trapped():
    env = dict(os.environ, LPLB_B200_DEBUG_BOUNDS="1")
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "tests", "bounds_worker.py")],
        env=env, capture_output=True, text=True, timeout=1500, cwd=ROOT,
    )
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    assert "BOUNDS_BUILD_OK" in proc.stdout
