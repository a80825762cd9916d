"""CPU tests of the library's host side: the C ABI loads and exports what the header declares,
argument checks answer with status codes (the reference exits/aborts/throws instead,
include/utils.h:16-23, src/flash_forward.h:384-387, :588), the FLOP count and the tile plan."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "flash_forward_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b([a-z_0-9]+)\s*\(", text)) - {"defined"})


def test_library_exports_every_declared_symbol(pkg):
    names = declared_functions()
    assert "flash_forward" in names and "run_flash_attention_c" in names
    L = ctypes.CDLL(pkg.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} is declared in the header but not exported"
    assert sorted(pkg.EXPORTS) == names


def test_header_is_plain_c(pkg):
    # the ABI is plain C: the header must compile as C
    import subprocess
    import tempfile

    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "t.c")
        open(src, "w").write('#include "flash_forward_b200.h"\nint main(void){return FA_OK;}\n')
        subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", src,
                               "-o", os.path.join(td, "t.o")])


def test_argument_errors_are_status_codes(pkg):
    L = pkg.lib()
    p = ctypes.c_void_p(0x1000)
    assert L.flash_forward(None, p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None) == pkg.FA_INVALID_ARG
    assert L.flash_forward(p, p, p, p, 0, 1, 128, 64, 0.0, 0, -1, -1, None) == pkg.FA_INVALID_ARG
    assert L.flash_forward(p, p, p, p, 1, 1, 128, 96, 0.0, 0, -1, -1, None) == pkg.FA_UNSUPPORTED
    assert b"head_dim" in L.flash_forward_last_error()
    assert L.flash_forward(ctypes.c_void_p(0x1008), p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None) == pkg.FA_INVALID_ARG
    assert L.flash_forward_ex(p, p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None, 7, 0, None) == pkg.FA_INVALID_ARG
    # a softmax scale that is not finite, or so small that masked scores would come back into range
    for bad in (float("nan"), float("inf"), 1e-35):
        assert L.flash_forward(p, p, p, p, 1, 1, 128, 64, bad, 0, -1, -1, None) == pkg.FA_INVALID_ARG
        assert b"softmax_scale" in L.flash_forward_last_error()
    # dropout probability outside [0, 1]
    assert L.run_flash_attention_c(1, 1, 128, 64, p, p, p, p, None, None, 1, 0, 0, 0, 0, None, 1.5, None) == pkg.FA_INVALID_ARG
    assert L.flash_forward_dropout(p, p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None, -0.5, 0, None) == pkg.FA_INVALID_ARG
    # ALiBi without slopes is a caller error
    assert L.run_flash_attention_c(1, 1, 128, 64, p, p, p, p, None, None, 0, 0, 0, 1, 0, None, 0.0, None) == pkg.FA_INVALID_ARG
    assert L.flash_forward_alibi(p, p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None, None) == pkg.FA_INVALID_ARG
    # the log-sum-exp entry point needs its output buffer, 4-byte aligned
    assert L.flash_forward_lse(p, p, p, p, None, 1, 1, 128, 64, 0.0, 0, -1, -1, None, None) == pkg.FA_INVALID_ARG
    assert b"lse" in L.flash_forward_last_error()
    assert L.flash_forward_lse(p, p, p, p, ctypes.c_void_p(0x1002), 1, 1, 128, 64, 0.0, 0, -1, -1, None, None) == pkg.FA_INVALID_ARG
    with pytest.raises(pkg.FlashForwardError):
        pkg.run_flash_attention(1, 1, 128, 64, 0x1000, 0x1000, 0x1000, 0x1000, Is_dropout=True, dropout_prob=2.0)
    with pytest.raises(pkg.FlashForwardError):  # no slabs
        pkg.flash_forward_multi_gpu([], [], [], [], [], [], 128, 64)


def test_no_gpu_is_an_error_not_a_fallback(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    p = ctypes.c_void_p(0x1000)
    rc = pkg.lib().flash_forward(p, p, p, p, 1, 1, 128, 64, 0.0, 0, -1, -1, None)
    assert rc in (pkg.FA_CUDA_ERROR, pkg.FA_UNSUPPORTED)


def brute_pairs(N, causal, wl, wr):
    i = np.arange(N)[:, None]
    j = np.arange(N)[None, :]
    vis = np.ones((N, N), bool)
    if causal:
        vis &= j <= i
    if wl >= 0:
        vis &= j >= i - wl
    if wr >= 0:
        vis &= j <= i + wr
    return vis


def test_flops_formulas(pkg):
    # BASELINE figures: 4*B*H*N^2*d, halved for causal, window-adjusted for local
    assert pkg.flops(1, 4, 512, 64) == 4 * 4 * 512 * 512 * 64 == 268435456
    assert pkg.flops(4, 16, 2048, 64, True) == 2 * 64 * 2048 * 2048 * 64
    assert pkg.flops(2, 32, 8192, 128, True) == 2 * 64 * 8192 * 8192 * 128
    assert pkg.flops(4, 16, 16384, 128, True, 1024, -1) == 4.0 * 64 * 128 * 16268800
    assert pkg.flops(8, 64, 32768, 128, True) == 2.0 ** 47
    for (N, causal, wl, wr) in [(300, False, 17, 5), (257, True, 40, -1), (128, False, -1, 9)]:
        assert pkg.flops(1, 1, N, 64, causal, wl, wr) == 4.0 * 64 * brute_pairs(N, causal, wl, wr).sum()


@pytest.mark.parametrize("N,causal,wl,wr", [
    (512, False, -1, -1), (512, True, -1, -1), (1024, True, 256, -1), (1024, False, 100, 50), (1000, True, -1, -1),
    (333, False, -1, -1), (2048, True, 1024, -1), (640, False, 0, 0), (700, False, -1, 130), (900, True, 127, -1),
    (900, True, 128, -1), (900, True, 129, 7),
])
def test_tile_plan_matches_brute_force(pkg, N, causal, wl, wr):
    vis = brute_pairs(N, causal, wl, wr)
    for r0 in range(0, N, 128):
        r1 = min(r0 + 128, N) - 1
        lo, hi, masked = pkg.kv_range(N, causal, wl, wr, r0, r1)
        touched = [j for j in range((N + 127) // 128) if vis[r0:r1 + 1, j * 128:(j + 1) * 128].any()]
        assert touched == list(range(lo, hi)), (r0, lo, hi, touched)
        want_masked = 0
        for j in touched:
            blk = vis[r0:r1 + 1, j * 128:(j + 1) * 128]
            if blk.shape[1] < 128 or not blk.all():
                want_masked += 1
        assert masked == want_masked, (r0, masked, want_masked)


def test_windows_up_to_int_max(pkg):
    """Window arguments are legal up to INT_MAX: the host-side plan and the FLOP count treat a window that covers
    the sequence as no window instead of overflowing `row + window`."""
    big = 2 ** 31 - 1
    for N in (127, 1000, 2048):
        for causal in (False, True):
            assert pkg.flops(2, 3, N, 64, causal, big, big) == pkg.flops(2, 3, N, 64, causal, -1, -1)
            assert pkg.flops(2, 3, N, 64, causal, N, N + 5) == pkg.flops(2, 3, N, 64, causal, -1, -1)
            assert pkg.flops(2, 3, N, 64, causal, 10, big) == pkg.flops(2, 3, N, 64, causal, 10, -1)
            for r0 in range(0, N, 128):
                r1 = min(r0 + 128, N) - 1
                assert pkg.kv_range(N, causal, big, big, r0, r1) == pkg.kv_range(N, causal, -1, -1, r0, r1)
                assert pkg.kv_range(N, causal, 100, big, r0, r1) == pkg.kv_range(N, causal, 100, -1, r0, r1)
            assert pkg.head_group(64, N, 64, causal, big, big) == pkg.head_group(64, N, 64, causal, -1, -1)


def test_head_group_policy(pkg):
    # no mask: head-major order
    assert pkg.head_group(64, 8192, 128) == 1
    # BASELINE configs 2-5 (causal / causal + window), 148 SMs
    assert pkg.head_group(64, 2048, 64, True) == 16
    assert pkg.head_group(64, 8192, 128, True) == 16      # 64 MB / 4 MB per head
    assert pkg.head_group(40, 8192, 128, True) == 14      # 16 would leave a last group of 8: three even groups instead
    assert pkg.head_group(64, 16384, 128, True, 1024) == 16  # only the window span stays live
    assert pkg.head_group(512, 32768, 128, True) == 4
    assert pkg.head_group(0, 128, 64) == 0 and pkg.head_group(4, 128, 96) == 0
    for bh in (1, 2, 3, 7, 12, 64, 100, 512):
        for N in (128, 1000, 4096, 32768, 131072):
            for d in (64, 128):
                for wl in (-1, 0, 300):
                    g = pkg.head_group(bh, N, d, True, wl)
                    assert 1 <= g <= min(16, bh)
                    groups = -(-bh // g)
                    assert bh - (groups - 1) * g >= g - (groups - 1)  # the last group is not a stub
