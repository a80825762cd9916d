"""GPU test of flash_forward_noalloc, the entry point for callers that must not allocate device
memory (a process whose memory pool owns the whole GPU, a latency-critical loop that cannot take
cudaMalloc's device-wide synchronisation, a plug-in under an allocator hook). It runs the same
persistent kernel as flash_forward, with the kernel's scratch words in a fixed array inside the
library instead of memory from cudaMalloc.

The file name keeps it last in collection order, so a run that stops at the first failure has
already run every other test. The test works alone in a fresh process and after the other tests."""
import ctypes

import numpy as np
import pytest

from conftest import make_inputs

pytestmark = pytest.mark.gpu


def call_noalloc(pkg, q, k, v, o, B, H, N, d, causal, wl, wr, slot, wait=1):
    import torch

    stream = torch.cuda.current_stream().cuda_stream
    return pkg.lib().flash_forward_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, N, d, 0.0,
                                           int(causal), wl, wr, stream, slot, wait)


@pytest.mark.parametrize("B,H,N,d,causal,wl", [(2, 6, 1024, 128, True, -1), (1, 5, 777, 64, True, 200)])
def test_noalloc_matches_flash_forward_twice_in_a_row(pkg, ob, B, H, N, d, causal, wl):
    import torch

    q, k, v = make_inputs(41, B, H, N, d)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    want = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    want = want.cpu().numpy()
    oracle = ob.attention(q, k, v, causal=causal, window_left=wl, window_right=-1)
    for attempt in range(2):  # the second call finds the slot as the first one left it
        out = torch.full_like(tq, float("nan"))
        rc = call_noalloc(pkg, tq, tk, tv, out, B, H, N, d, causal, wl, -1, slot=3)
        assert rc == pkg.FA_OK, pkg.lib().flash_forward_last_error()
        got = out.cpu().numpy()
        mx, mean, nans = ob.abs_error(got, want)
        assert nans == 0 and mx <= 2e-3 and mean <= 2e-4, (attempt, mx, mean, nans)
        mx, mean, nans = ob.abs_error(got, oracle)
        assert nans == 0 and mx <= 2e-3 and mean <= 2e-4, (attempt, mx, mean, nans)


def test_noalloc_async_then_other_slot(pkg, ob):
    import torch

    B, H, N, d = 1, 4, 512, 128
    q, k, v = make_inputs(43, B, H, N, d)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    a = torch.empty_like(tq)
    b = torch.empty_like(tq)
    assert call_noalloc(pkg, tq, tk, tv, a, B, H, N, d, False, -1, -1, slot=0, wait=0) == pkg.FA_OK
    assert call_noalloc(pkg, tq, tk, tv, b, B, H, N, d, False, -1, -1, slot=15, wait=1) == pkg.FA_OK
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    want = ob.attention(q, k, v)
    mx, mean, nans = ob.abs_error(a.cpu().numpy(), want)
    assert nans == 0 and mx <= 2e-3 and mean <= 2e-4


def test_noalloc_in_a_cuda_graph_and_the_allocating_entry_point_refuses_capture(pkg, ob):
    # The entry point with a caller-chosen scratch slot is the one to capture: two launches (two slots) go into one
    # graph, the graph is replayed on new inputs in the same buffers, and every replay equals the eager result.
    # flash_forward itself answers FA_UNSUPPORTED while its stream is being captured, and leaves the capture intact.
    import torch

    B, H, N, d = 1, 6, 640, 128
    q, k, v = make_inputs(47, B, H, N, d)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    o1, o2 = torch.empty_like(tq), torch.empty_like(tq)
    assert call_noalloc(pkg, tq, tk, tv, o1, B, H, N, d, True, -1, -1, slot=4) == pkg.FA_OK  # first call: no capture yet
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            st = torch.cuda.current_stream().cuda_stream
            L = pkg.lib()
            rc_plain = L.flash_forward(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o1.data_ptr(), B, H, N, d, 0.0, 1,
                                       -1, -1, st)
            rc1 = L.flash_forward_noalloc(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o1.data_ptr(), B, H, N, d, 0.0,
                                          1, -1, -1, st, 4, 0)
            rc2 = L.flash_forward_noalloc(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o2.data_ptr(), B, H, N, d, 0.0,
                                          0, 100, 50, st, 5, 0)
    assert rc_plain == pkg.FA_UNSUPPORTED and b"graph" in pkg.lib().flash_forward_last_error()
    assert rc1 == pkg.FA_OK and rc2 == pkg.FA_OK
    for seed in (48, 49, 50):
        q, k, v = make_inputs(seed, B, H, N, d)
        for t, a in ((tq, q), (tk, k), (tv, v)):
            t.copy_(torch.from_numpy(a))
        o1.fill_(float("nan"))
        o2.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert pkg.lib().flash_forward_noalloc_check(None, 4) == pkg.FA_OK
        assert pkg.lib().flash_forward_noalloc_check(None, 5) == pkg.FA_OK
        want1 = pkg.attention_forward(tq, tk, tv, causal=True)
        want2 = pkg.attention_forward(tq, tk, tv, causal=False, window_left=100, window_right=50)
        torch.cuda.synchronize()
        assert torch.equal(o1, want1) and torch.equal(o2, want2), seed
    mx, mean, nans = ob.abs_error(o1.cpu().numpy(), ob.attention(q, k, v, causal=True))
    assert nans == 0 and mx <= 2e-3 and mean <= 2e-4


def test_noalloc_rejects_what_the_scratch_cannot_hold(pkg):
    import torch

    t = torch.zeros((1, 1, 128, 64), dtype=torch.float16, device="cuda")
    for slot in (-1, 16, 1000):
        rc = call_noalloc(pkg, t, t, t, t, 1, 1, 128, 64, False, -1, -1, slot=slot)
        assert rc == pkg.FA_INVALID_ARG
        assert b"slot" in pkg.lib().flash_forward_last_error()
    # more work items than the slot's 32-bit counter can number
    rc = pkg.lib().flash_forward_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 1 << 15, 1 << 15,
                                         1024, 64, 0.0, 0, -1, -1, None, 0, 1)
    assert rc == pkg.FA_INVALID_ARG
    assert b"work items" in pkg.lib().flash_forward_last_error()
    assert pkg.lib().flash_forward_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 1, 1, 128, 96, 0.0,
                                           0, -1, -1, None, 0, 1) == pkg.FA_UNSUPPORTED


_FRESH_PROCESS_SCRIPT = r"""
import ctypes, sys
import numpy as np
import torch
sys.path.insert(0, {root!r})
import __graft_entry__ as entry
pkg = entry.load_package()
L = pkg.lib()
rt = ctypes.CDLL("libcudart.so." + torch.version.cuda.split(".")[0], mode=ctypes.RTLD_GLOBAL)
def free_bytes():
    f, t = ctypes.c_size_t(), ctypes.c_size_t()
    assert rt.cudaMemGetInfo(ctypes.byref(f), ctypes.byref(t)) == 0
    return f.value
B, H, N, d = 1, 3, 640, 128
g = torch.Generator(device="cuda").manual_seed(5)
q, k, v = (torch.randn((B, H, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
outs = [torch.empty_like(q) for _ in range(4)]
torch.cuda.synchronize()
def call(o, slot, wait):
    return L.flash_forward_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, N, d, 0.0, 1, -1, -1,
                                   None, slot, wait)
assert call(outs[0], 2, 1) == 0          # first call on the device: one-time set-up
before = free_bytes()
assert call(outs[1], 2, 1) == 0
assert call(outs[2], 7, 0) == 0
assert L.flash_forward_noalloc_check(None, 7) == 0
assert call(outs[3], 2, 1) == 0
after = free_bytes()
assert before == after, (before, after)  # nothing was allocated on the device by any of the calls
for o in outs[1:]:
    assert torch.equal(o, outs[0])
# the ordinary entry point was never used in this process, so its scratch was never allocated either
ref = torch.softmax((q.float() @ k.float().transpose(-1, -2) / d ** 0.5).masked_fill(
    torch.triu(torch.ones(N, N, dtype=torch.bool, device="cuda"), 1), float("-inf")), -1) @ v.float()
assert (outs[0].float() - ref).abs().max().item() <= 4e-3
print("NOALLOC-OK")
"""


def test_noalloc_allocates_nothing_in_a_fresh_process(pkg):
    """The defining property, checked where nothing else can hide it: a new process that only ever calls
    flash_forward_noalloc (so the ordinary entry point's cudaMalloc never runs) sees the same free device memory
    before and after further calls, and the allocation-free status read works."""
    import subprocess
    import sys

    from conftest import ROOT

    r = subprocess.run([sys.executable, "-c", _FRESH_PROCESS_SCRIPT.format(root=ROOT)], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0 and "NOALLOC-OK" in r.stdout, r.stdout + r.stderr


def test_noalloc_on_a_second_device_and_after_shutdown(pkg):
    """The scratch address belongs to a device: a call on device 1 must look it up there, and a call after
    flash_forward_shutdown() must look it up again."""
    import torch

    B, H, N, d = 1, 2, 384, 64
    devices = [0] + ([1] if torch.cuda.device_count() > 1 else [])
    results = []
    for rep in range(2):
        for dev in devices:
            with torch.cuda.device(dev):
                g = torch.Generator(device=f"cuda:{dev}").manual_seed(9)
                q, k, v = (torch.randn((B, H, N, d), generator=g, device=f"cuda:{dev}", dtype=torch.float16)
                           for _ in range(3))
                o = torch.full_like(q, float("nan"))
                assert call_noalloc(pkg, q, k, v, o, B, H, N, d, True, -1, -1, slot=1) == pkg.FA_OK
                ref = pkg.attention_forward(q, k, v, causal=True)
                torch.cuda.synchronize()
                assert torch.equal(o, ref)
                results.append(o.cpu())
        torch.cuda.synchronize()
        assert pkg.lib().flash_forward_shutdown() == pkg.FA_OK
    for r in results[1:]:
        assert torch.equal(r, results[0])
