"""The kernels of a call are launched with programmatic dependent launch (each one's set-up under the tail of the one
before; the dQ kernel runs beside the dK/dV kernel's last wave).  None of that may change a single bit: the same
forward + backward calls with every launch made the ordinary way (MCA_NO_PDL) must give identical outputs."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def _digest(no_pdl):
    env = dict(os.environ)
    env.pop("MCA_NO_PDL", None)
    if no_pdl:
        env["MCA_NO_PDL"] = "1"
    out = subprocess.run([sys.executable, str(Path(__file__).with_name("pdl_probe.py"))], env=env, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("DIGEST ")]
    assert len(lines) == 1, out.stdout[-2000:]
    return lines[0]


def test_dependent_launches_change_no_bit():
    assert _digest(False) == _digest(True)
