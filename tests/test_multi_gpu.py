"""flash_forward_multi_gpu: slabs of heads on one or several devices equal the single call bit for bit.
On a one-GPU machine both slabs run on device 0; with two or more GPUs every slab has its own device."""
import numpy as np
import pytest

from conftest import make_inputs

pytestmark = pytest.mark.gpu


def run_slabs(pkg, q, k, v, devices, cuts, causal, wl):
    import torch

    B, H, N, d = q.shape
    bh = B * H
    flat = [a.reshape(bh, N, d) for a in (q, k, v)]
    bounds = [0] + list(cuts) + [bh]
    tens, outs = [], []
    for i, dev in enumerate(devices):
        lo, hi = bounds[i], bounds[i + 1]
        tens.append([torch.from_numpy(np.ascontiguousarray(a[lo:hi])).to(f"cuda:{dev}") for a in flat])
        outs.append(torch.zeros((hi - lo, N, d), dtype=torch.float16, device=f"cuda:{dev}"))
    for dev in set(devices):
        torch.cuda.synchronize(dev)
    ptr = lambda t: t.data_ptr() if t.numel() else 0x10  # noqa: E731  (never dereferenced for an empty slab)
    pkg.flash_forward_multi_gpu(devices, [ptr(t[0]) for t in tens], [ptr(t[1]) for t in tens],
                                [ptr(t[2]) for t in tens], [ptr(o) for o in outs],
                                [bounds[i + 1] - bounds[i] for i in range(len(devices))], N, d, 0.0, causal, wl, -1,
                                None, True)
    return np.concatenate([o.cpu().numpy() for o in outs], axis=0).reshape(B, H, N, d)


@pytest.mark.parametrize("N,d,causal,wl", [(640, 128, True, -1), (1000, 64, True, 200), (512, 64, False, -1)])
def test_slabs_equal_single_call(pkg, N, d, causal, wl):
    import torch

    B, H = 2, 5
    q, k, v = make_inputs(900 + N, B, H, N, d)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    want = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    want = want.cpu().numpy()
    n_dev = torch.cuda.device_count()
    cur = torch.cuda.current_device()
    devices = [0, 1 % n_dev, 2 % n_dev]
    got = run_slabs(pkg, q, k, v, devices, cuts=(3, 3), causal=causal, wl=wl)  # slabs of 3, 0 and 7 heads
    assert torch.cuda.current_device() == cur
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    got = run_slabs(pkg, q, k, v, [d_ % n_dev for d_ in range(4)], cuts=(1, 4, 9), causal=causal, wl=wl)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_every_visible_device_gives_the_same_bits(pkg):
    """BASELINE config 3's per-head shape on every GPU of the machine: each device computes the same two
    heads; all results must be identical (no device-dependent state in the library)."""
    import torch

    n_dev = torch.cuda.device_count()
    N, d = 8192, 128
    q, k, v = make_inputs(77, 1, 2, N, d)
    outs = []
    for dev in range(n_dev):
        outs.append(run_slabs(pkg, q, k, v, [dev], cuts=(), causal=True, wl=-1))
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint16), outs[0].view(np.uint16))
    assert np.isfinite(outs[0].astype(np.float32)).all()
