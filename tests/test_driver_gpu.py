"""GPU test of the main()-like driver (the reference's src/main.cu flow on top of the library):
it must print the reference's TIME line and report zero verification errors."""
import os
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

DRIVER = os.path.join(ROOT, "flash-attn-rtx5060_b200", "flash_driver")


@pytest.mark.parametrize("args", [
    [],                                                  # the reference's own configuration: B2 H8 N2048 d64, U(0,10)
    ["1", "4", "1024", "128", "1", "-1", "0", "1", "26"],  # causal, N(0,1)
    ["1", "4", "1024", "128", "1", "256", "0", "1", "26"],  # causal + window
    ["2", "3", "640", "64", "0", "-1", "1", "1", "7"],      # ALiBi
])
def test_driver_runs_and_verifies(args):
    if not os.path.exists(DRIVER):
        pytest.fail(f"{DRIVER} has not been built (make -C flash-attn-rtx5060_b200/csrc)")
    proc = subprocess.run([DRIVER] + args, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout
    assert "TIME:" in proc.stdout
    assert "finish,error:0" in proc.stdout
