"""The checks variant of the device library (-DPSDEV_CHECKS): the dense kernel verifies every
index against the table, the owner's state arrays and the arena, the sparse kernels every slot
index against the store's capacity and every value offset against the request buffers; a bad
index is recorded as PSDEV_ERR_BOUNDS and the access is skipped instead of performed.  The
variant is chosen per process, so the test
body runs in a child (tests/checks_build_child.py).  Nothing here touches memory outside an
allocation: the refused indices are made by telling the kernel that the table is shorter than
it really is."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_checks_build_is_silent_when_right_and_refuses_when_wrong(cuda_device):
    env = dict(os.environ, PSB200_DEVICE_CHECKS="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "checks_build_child.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "CHECKS_OK" in r.stdout, (r.stdout + r.stderr)[-4000:]
