"""A bounded device-side wait is made to run out, on purpose and only in a test build of the library
(tests/_build/libflashfwd_waittest.so: same sources, waits give up after about 2 ms instead of 1 s, and
`variant` bit 1 of flash_forward_ex makes CTA 0 skip one K/V load). Nothing faults or hangs: the tensor-core
issuer of CTA 0 waits for the tile, gives up, raises the CTA's abort flag, every other role of the CTA sees the
flag and leaves its loop, the producer lets loads in flight land, the CTA sets the device status word and
exits normally; all other CTAs finish their work. The host reads FA_DEVICE_TIMEOUT, and the next ordinary
call on the same device is correct.

What the reference does in the same situation: its mbarrier wait spins without a limit
(include/utils.h:115-130), i.e. the kernel never returns."""
import ctypes
import os

import numpy as np
import pytest

from conftest import ROOT, make_inputs

pytestmark = pytest.mark.gpu

WAITTEST = os.path.join(ROOT, "tests", "_build", "libflashfwd_waittest.so")


def test_wait_gives_up_and_the_device_stays_usable(pkg, ob):
    import torch

    if not os.path.isfile(WAITTEST):
        pytest.skip("tests/_build/libflashfwd_waittest.so was not built")
    L = ctypes.CDLL(WAITTEST)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.flash_forward_ex.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, i, i, vp]
    L.flash_forward_check.argtypes = [vp]
    L.flash_forward_last_error.restype = ctypes.c_char_p

    B, H, N, d = 1, 1, 512, 128   # two work items; CTA 0's first item has four kv tiles
    q, k, v = make_inputs(61, B, H, N, d)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    out = torch.zeros_like(tq)
    stream = torch.cuda.current_stream().cuda_stream
    want = ob.attention(q, k, v, causal=True)

    # the test build computes the same thing as long as nothing is withheld
    assert L.flash_forward_ex(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), B, H, N, d, 0.0, 1, -1, -1,
                              stream, 0, 0, None) == pkg.FA_OK
    assert L.flash_forward_check(stream) == pkg.FA_OK
    mx, mean, nans = ob.abs_error(out.cpu().numpy(), want)
    assert nans == 0 and mx <= 2e-3 and mean <= 2e-4

    # withhold one tile in CTA 0: the launch returns, the check reports the time-out
    out.zero_()
    assert L.flash_forward_ex(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), B, H, N, d, 0.0, 1, -1, -1,
                              stream, 0, 2, None) == pkg.FA_OK
    assert L.flash_forward_check(stream) == pkg.FA_DEVICE_TIMEOUT
    assert b"ran out of time" in L.flash_forward_last_error()
    assert L.flash_forward_check(stream) == pkg.FA_OK      # the status word was consumed
    assert torch.cuda.current_stream().query()              # nothing is left running

    # the same library and the product library both work on this device afterwards
    for lib in (L, pkg.lib()):
        out.fill_(float("nan"))
        assert lib.flash_forward_ex(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), B, H, N, d, 0.0, 1, -1,
                                    -1, stream, 0, 0, None) == pkg.FA_OK
        assert lib.flash_forward_check(stream) == pkg.FA_OK
        mx, mean, nans = ob.abs_error(out.cpu().numpy(), want)
        assert nans == 0 and mx <= 2e-3 and mean <= 2e-4
