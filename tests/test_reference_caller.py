"""The drop-in shown on the reference's own caller: the reference's unmodified src/main.cu (its
`#include "flash_forward.h"` at line 13, its call of run_flash_attention at line 99, its CPU attention
and its `verify`, lines 134-268) built against include/reference_shim/flash_forward.h and
libflashfwd_b200.so instead of the reference's header and kernel.

Building needs the reference sources, so that half runs where they are present (it is skipped
elsewhere); the binary lands in oracle/_ref/ and travels to the GPU machine with the other built
files, where the second half runs it."""
import os
import subprocess

import pytest

from conftest import ROOT

REFERENCE = "/root/reference"
BINARY = os.path.join(ROOT, "oracle", "_ref", "ref_main_dropin")


@pytest.mark.skipif(not os.path.isfile(os.path.join(REFERENCE, "src", "main.cu")), reason="reference sources not present")
def test_reference_main_builds_against_the_shim(pkg):
    if os.path.exists(BINARY):
        os.remove(BINARY)
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "_ref/ref_main_dropin", f"REFERENCE={REFERENCE}"],
                          stdout=subprocess.DEVNULL)
    assert os.path.isfile(BINARY)
    syms = subprocess.run(["nm", "-D", "--undefined-only", BINARY], capture_output=True, text=True, check=True).stdout
    assert "run_flash_attention_c" in syms  # the call at src/main.cu:99 lands in the library
    defined = subprocess.run(["nm", "-C", "--defined-only", BINARY], capture_output=True, text=True, check=True).stdout
    assert "forward_kernel" not in defined  # none of the reference's own kernel was compiled in
    assert "attention_forward_cpu" in defined and "verify" in defined  # its oracle and check were


@pytest.mark.gpu
def test_reference_main_runs_and_verifies():
    """The reference's main(): U(0,10) inputs seeded 26, B2 H8 N2048 d64, its CPU attention, its 6 % check
    (src/main.cu:21-132). Expected output: the entry point's "TIME:" line and verify's "finish,error:0"."""
    if not os.path.isfile(BINARY):
        pytest.skip("oracle/_ref/ref_main_dropin was not built (reference sources absent at build time)")
    r = subprocess.run([BINARY], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "TIME:" in r.stdout
    assert "finish,error:0" in r.stdout, r.stdout[-2000:]
