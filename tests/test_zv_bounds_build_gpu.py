"""The -DNB_BOUNDS=1 build of the kernel library: indices read from memory are tested against their extent, a failed
test is reported through the device status word and the access is skipped (no fault)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bounds_checked_build_reports_and_skips():
    env = dict(os.environ, NOEIRA_B200_BOUNDS="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "mp", "bounds_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert "BOUNDS_WORKER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
