"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle (the
restatement of the reference's attention_forward_cpu, src/main.cu:159-268) on the same seeded
fp16 inputs. Acceptance: max abs error <= 2e-3 and mean abs error <= 2e-4, fp16 outputs
compared in fp32."""
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR, golden_cases, make_inputs

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = 2e-3, 2e-4


def run_gpu(pkg, q, k, v, causal=False, wl=-1, wr=-1, kernel=0, scale=0.0):
    import torch

    tq, tk, tv = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, k, v))
    out = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl, window_right=wr, softmax_scale=scale,
                                kernel=kernel)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    return out.cpu().numpy()


def assert_close(ob, got, want, max_abs=MAX_ABS, mean_abs=MEAN_ABS):
    mx, mean, nans = ob.abs_error(got, want)
    assert nans == 0, f"{nans} NaNs in the GPU output"
    assert mx <= max_abs and mean <= mean_abs, f"max_abs={mx:.3e} mean_abs={mean:.3e}"
    return mx, mean


def fp16_ulp(x):
    """Spacing of fp16 numbers at |x| (subnormal spacing below 2^-14)."""
    a = np.abs(x.astype(np.float32))
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    return np.exp2(e - 10).astype(np.float32)


def exact_rows(q, k, v, b, h, rows, scale, causal, wl, wr):
    """fp64 attention of the given rows of one head (numpy): the error-free answer for those rows."""
    q64, k64, v64 = (a[b, h].astype(np.float64) for a in (q, k, v))
    n = k64.shape[0]
    out = np.empty((len(rows), v64.shape[1]))
    j = np.arange(n)
    for t, i in enumerate(rows):
        vis = np.ones(n, bool)
        if causal:
            vis &= j <= i
        if wl >= 0:
            vis &= j >= i - wl
        if wr >= 0 and not causal:
            vis &= j <= i + wr
        s = (k64[vis] @ q64[i]) * scale
        p = np.exp(s - s.max())
        out[t] = (p / p.sum()) @ v64[vis]
    return out


def assert_close_or_one_ulp(got, want, mean_abs=MEAN_ABS, exact=None):
    """The acceptance bar where 2e-3 is no longer more than the oracle's own rounding: every element is within
    2e-3 of the oracle, OR within one fp16 ulp of the oracle's value (3.9e-3 at |o| >= 4), OR - where `exact` is given
    - the element is one of the few on which the oracle itself is the noisy side: it rounds every p*v product to
    fp16, so a row whose terms reach 2..4 and cancel carries up to 2e-3 of noise at any |o|; such an element passes
    only if the kernel is within 1e-3 of the fp64 answer. `exact(b, h, rows)` returns fp64 rows. The mean bar is
    unchanged. Prints the worst distance in ulps beside the absolute one."""
    g32, w32 = got.astype(np.float32), want.astype(np.float32)
    assert np.isfinite(g32).all()
    diff = np.abs(g32 - w32)
    ulps = diff / fp16_ulp(want)
    worst = int(np.argmax(diff))
    print(f"max_abs={diff.max():.3e} at |o|={abs(w32.flat[worst]):.3f} ({ulps.flat[worst]:.2f} ulp of the oracle value); "
          f"mean_abs={diff.mean():.3e}")
    bad = np.argwhere((diff > MAX_ABS) & (ulps > 1.0))
    if len(bad) and exact is not None:
        assert len(bad) <= 16, f"{len(bad)} elements beyond both 2e-3 and one fp16 ulp"
        for b, h, i, c in bad:
            ex = exact(b, h, [i])[0, c]
            err_kernel, err_oracle = abs(g32[b, h, i, c] - ex), abs(w32[b, h, i, c] - ex)
            print(f"  element {(b, h, i, c)}: kernel {g32[b, h, i, c]:.5f} oracle {w32[b, h, i, c]:.5f} fp64 {ex:.5f}")
            assert err_kernel <= 1e-3 and err_kernel <= err_oracle, (err_kernel, err_oracle)
    else:
        assert len(bad) == 0, (f"{len(bad)} elements beyond both 2e-3 and one fp16 ulp; worst {diff.max():.3e} "
                               f"at |o|={abs(w32.flat[worst]):.3f}")
    assert diff.mean() <= mean_abs, f"mean_abs={diff.mean():.3e}"


def test_golden_alibi(pkg, ob):
    """The reference's ALiBi bias (src/mask.h:21-26, src/main.cu:200-207) against the golden vector made by its CPU
    function, through both the native entry point and the reference's positional one."""
    import torch

    z = np.load(os.path.join(GOLDEN_DIR, "case_n256d64_causal_alibi.npz"))
    q, k, v = (z[n].view(np.float16) for n in ("q", "k", "v"))
    want = z["out"].view(np.float16)
    B, H, N, d = q.shape
    tq, tk, tv = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, k, v))
    slopes = torch.from_numpy(z["slopes"]).cuda()
    out = pkg.attention_forward(tq, tk, tv, causal=True, alibi_slopes=slopes)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    assert_close(ob, out.cpu().numpy(), want)
    out2 = torch.empty_like(tq)
    torch.cuda.synchronize()
    pkg.run_flash_attention(B, H, N, d, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out2.data_ptr(), None, None,
                            False, True, False, True, 0, slopes.data_ptr())
    assert torch.equal(out, out2)


@pytest.mark.parametrize("N,d,causal,w", [(700, 128, False, -1), (1000, 64, True, 130), (512, 128, False, 64)])
def test_alibi_against_oracle(pkg, ob, N, d, causal, w):
    import torch

    H = 3
    q, k, v = make_inputs(77 + N, 2, H, N, d)
    slopes = np.array([-(2.0 ** (-8.0 / H * (i + 1))) for i in range(H)], dtype=np.float32)  # src/main.cu:41
    want = ob.attention(q, k, v, causal=causal, window_left=w, window_right=w, alibi_slopes=slopes)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    out = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=w, window_right=w,
                                alibi_slopes=torch.from_numpy(slopes).cuda())
    pkg.check(torch.cuda.current_stream().cuda_stream)
    assert_close_or_one_ulp(out.cpu().numpy(), want)  # the positive bias concentrates mass: |o| passes 4


@pytest.mark.parametrize("kernel", [0, 1])
@pytest.mark.parametrize("fname", [f for f in golden_cases() if "alibi" not in f])
def test_golden_vectors(pkg, ob, fname, kernel):
    z = np.load(os.path.join(GOLDEN_DIR, fname))
    q, k, v = (z[n].view(np.float16) for n in ("q", "k", "v"))
    w = int(z["window"])
    causal = bool(int(z["causal"]))
    got = run_gpu(pkg, q, k, v, causal, w, w, kernel)
    want = z["out"].view(np.float16)
    if "uniform" in fname:
        # The reference's own smoke distribution (src/main.cu:70): logits of ~200 and fp16-rounded
        # products of up to 100 make the CPU function itself noisy at the 1e-2 level, which is why
        # the reference checks this case with a 6 % relative tolerance (src/main.cu:107,149).
        # Same criterion here, plus a bound on the mean.
        g32, w32 = got.astype(np.float32), want.astype(np.float32)
        assert np.isfinite(g32).all()
        assert np.all(np.abs(g32 - w32) <= 0.06 * np.abs(w32))
        assert np.abs(g32 - w32).mean() <= 2e-2
    else:
        assert_close(ob, got, want)


# BASELINE configs 1 and 2, whole, against the oracle
@pytest.mark.parametrize("B,H,N,d,causal", [(1, 4, 512, 64, False), (4, 16, 2048, 64, True)])
def test_config_1_and_2_whole(pkg, ob, B, H, N, d, causal):
    q, k, v = make_inputs(26, B, H, N, d)
    got = run_gpu(pkg, q, k, v, causal)
    want = ob.attention(q, k, v, causal=causal)
    assert_close(ob, got, want)


def sampled_rows(N, wl):
    rng = np.random.default_rng(3)
    rows = [np.arange(0, min(N, 258)), np.arange(max(0, N - 128), N), rng.integers(0, N, 96)]
    for b in (127, 128, 129, 255, 256, 257):
        rows.append(np.array([b]))
    if wl >= 0:
        rows.append(np.arange(max(0, wl - 2), min(N, wl + 3)))
    return np.unique(np.concatenate(rows)).astype(np.int32)


# BASELINE configs 3, 4 and the per-GPU shape of config 5: full size on the GPU, oracle on sampled
# heads (first, last, one in the middle) and sampled rows (first 258, last 128, tile boundaries,
# the window edge, random rows)
@pytest.mark.parametrize("B,H,N,d,causal,wl", [
    (2, 32, 8192, 128, True, -1),
    (4, 16, 16384, 128, True, 1024),
    (1, 8, 32768, 128, True, -1),
])
def test_large_configs_sampled(pkg, ob, B, H, N, d, causal, wl):
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(26)
    q, k, v = (torch.randn((B, H, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    out = pkg.attention_forward(q, k, v, causal=causal, window_left=wl)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    rows = sampled_rows(N, wl)
    worst = (0.0, 0.0)
    for (b, h) in [(0, 0), (B - 1, H - 1), (B // 2, H // 2)]:
        hq, hk, hv, ho = (x[b, h].cpu().numpy() for x in (q, k, v, out))
        want = ob.attention_rows(hq, hk, hv, rows, causal=causal, window_left=wl, window_right=-1)
        mx, mean = assert_close(ob, ho[rows], want)
        worst = (max(worst[0], mx), max(worst[1], mean))
    # size-independent properties on the full output
    assert torch.isfinite(out).all()
    if causal:  # the first query sees only the first key: its output is v[0] exactly
        assert torch.equal(out[:, :, 0, :], v[:, :, 0, :])
    # linearity in V: a power-of-two factor commutes with every rounding except into fp16 subnormals
    out2 = pkg.attention_forward(q, k, v * 2, causal=causal, window_left=wl)
    assert (out2.float() - 2 * out.float()).abs().max().item() <= 2.0 ** -23


def test_very_long_sequence_and_very_many_heads(pkg, ob):
    """The two ends of the work-item space: one head of 131072 rows (512 q pairs, a 64 MB K/V working set, 1024 kv
    tiles for the last rows) and 6000 heads of 256 rows (one item per head, the dynamic work counter hands out
    ~5850 items). Sampled rows against the oracle for the long one, everything for the many."""
    import torch

    g = torch.Generator(device="cuda").manual_seed(131)
    N, d = 131072, 128
    q, k, v = (torch.randn((1, 1, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    out = pkg.attention_forward(q, k, v, causal=True)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    rows = np.unique(np.concatenate([np.arange(0, 130), np.arange(65530, 65540), np.arange(N - 64, N),
                                     np.random.default_rng(2).integers(0, N, 24)])).astype(np.int32)
    hq, hk, hv, ho = (x[0, 0].cpu().numpy() for x in (q, k, v, out))
    want = ob.attention_rows(hq, hk, hv, rows, causal=True, window_left=-1, window_right=-1)
    assert_close(ob, ho[rows], want)
    assert torch.isfinite(out).all()
    del q, k, v, out

    q, k, v = make_inputs(6000, 6000, 1, 256, 64)
    got = run_gpu(pkg, q, k, v, True, 100, -1)
    want = ob.attention(q, k, v, causal=True, window_left=100, window_right=-1)
    # 98 M outputs; the early causal rows are averages of a handful of N(0,1) values and some exceed 4, where one
    # fp16 ulp is 3.9e-3
    assert_close_or_one_ulp(got, want, exact=lambda b, h, rows: exact_rows(q, k, v, b, h, rows, 0.125, True, 100, -1))


@pytest.mark.parametrize("kernel", [0, 1])
@pytest.mark.parametrize("N,d,causal,wl,wr", [
    (1, 64, False, -1, -1), (5, 128, True, -1, -1), (127, 64, True, -1, -1), (129, 128, False, -1, -1),
    (333, 128, False, -1, -1), (1000, 64, True, -1, -1), (640, 64, False, 0, 0), (700, 128, False, -1, 130),
    (900, 64, True, 127, -1), (900, 128, True, 128, -1), (900, 64, True, 129, 7), (1024, 64, False, 100, 50),
    (1024, 128, True, 256, -1), (2048, 128, True, 1024, -1), (512, 64, False, 3, 3), (600, 128, False, 300, -1),
])
def test_edge_shapes_and_windows(pkg, ob, kernel, N, d, causal, wl, wr):
    q, k, v = make_inputs(N * 7 + d, 1, 3, N, d)
    got = run_gpu(pkg, q, k, v, causal, wl, wr, kernel)
    want = ob.attention(q, k, v, causal=causal, window_left=wl, window_right=wr)
    assert_close(ob, got, want)


@pytest.mark.parametrize("N,causal,wl,wr", [
    (512, False, -1, -1), (1024, True, -1, -1), (1000, True, -1, -1), (333, False, -1, -1), (1024, True, 256, -1),
    (700, False, 100, 50), (2048, True, 1024, -1), (129, True, -1, -1),
])
def test_cta_pair_kernel(pkg, ob, N, causal, wl, wr):
    """The cta_group::2 kernel (two CTAs share every K/V tile, one q tile per CTA, scores computed two kv tiles
    ahead; head_dim 128 only), flash_forward_ex(kernel=2)."""
    kernel = 2
    q, k, v = make_inputs(N * 3 + 1, 2, 3, N, 128)
    got = run_gpu(pkg, q, k, v, causal, wl, wr, kernel=kernel)
    want = ob.attention(q, k, v, causal=causal, window_left=wl, window_right=wr)
    assert_close(ob, got, want)
    ref = run_gpu(pkg, q, k, v, causal, wl, wr, kernel=0)
    mx, mean, nans = ob.abs_error(got, ref)
    assert nans == 0 and mx <= 2e-3


@pytest.mark.parametrize("B,H,N,causal,wl", [
    (1, 150, 512, True, -1),    # 300 items on 74 clusters: several short items (2 and 4 kv tiles) per cluster
    (3, 7, 2176, True, 300),    # windowed: items with odd numbers of kv tiles, ragged last pair
    (1, 40, 4096, False, -1),   # 16 long items of equal length per head
])
def test_cta_pair_kernel_many_items(pkg, ob, B, H, N, causal, wl):
    """The pair kernel streams the items of a cluster back to back (scores of the next item are issued while the
    last tiles of the current one are still in the softmax); every hand-off that is counted per item or per tile
    must survive short items. Two runs each, against the oracle on sampled heads and against the default kernel
    on everything."""
    import torch

    q, k, v = make_inputs(4000 + N + H, B, H, N, 128)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    ref = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl, kernel=0)
    for _ in range(2):
        got = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl, kernel=2)
        pkg.check(torch.cuda.current_stream().cuda_stream)
        assert float((got.float() - ref.float()).abs().max()) <= 2e-3
    heads = [0, H // 2, H - 1]
    want = ob.attention(q[:1, heads], k[:1, heads], v[:1, heads], causal=causal, window_left=wl, window_right=-1)
    assert_close(ob, got[:1, heads].cpu().numpy(), want)


def test_windows_up_to_int_max_are_unbounded(pkg, ob):
    """Any window value is legal; one that covers the whole sequence must give the unwindowed result bit for bit
    (the tile arithmetic works on `row - window_left` and `row + window_right`, so INT_MAX must not reach it)."""
    big = 2 ** 31 - 1
    q, k, v = make_inputs(91, 1, 2, 777, 64)   # ragged length: the tail tile is masked
    plain = run_gpu(pkg, q, k, v, False, -1, -1)
    assert np.array_equal(plain.view(np.uint16), run_gpu(pkg, q, k, v, False, big, big).view(np.uint16))
    assert np.array_equal(plain.view(np.uint16), run_gpu(pkg, q, k, v, False, big, -1).view(np.uint16))
    assert np.array_equal(plain.view(np.uint16), run_gpu(pkg, q, k, v, False, 777, 100000).view(np.uint16))
    causal = run_gpu(pkg, q, k, v, True, -1, -1)
    assert np.array_equal(causal.view(np.uint16), run_gpu(pkg, q, k, v, True, big, big).view(np.uint16))
    one_sided = run_gpu(pkg, q, k, v, False, 50, big)
    assert_close(ob, one_sided, ob.attention(q, k, v, window_left=50, window_right=-1))


def test_many_launches_on_two_streams(pkg):
    """More launches than the library has scheduler slots (64), alternating between two streams with nothing
    synchronising them: a launch that reuses a slot last used on the other stream must wait for that launch, or the
    two would share a work counter and rows would be left unwritten."""
    import torch

    g = torch.Generator(device="cuda").manual_seed(7)
    B, H, N, d = 1, 24, 1024, 64
    q, k, v = (torch.randn((B, H, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    want = pkg.attention_forward(q, k, v, causal=True)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.full_like(q, float("nan")) for _ in range(200)]
    for i, o in enumerate(outs):
        pkg.flash_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, N, d, is_causal=True,
                          stream=streams[i & 1].cuda_stream)
    for st in streams:
        pkg.check(st.cuda_stream)
    for o in outs:
        assert torch.equal(o, want)


def exact_attention(q, k, v, scale, causal):
    """fp64 attention of fp16 inputs (numpy), rounded once to fp16: the error-free answer."""
    q64, k64, v64 = (a.astype(np.float64) for a in (q, k, v))
    s = np.einsum("bhid,bhjd->bhij", q64, k64) * scale
    if causal:
        n = s.shape[-1]
        s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhij,bhjd->bhid", p, v64).astype(np.float16)


def test_explicit_scale_and_large_logits(pkg, ob):
    # Logit spread of ~20 makes the softmax nearly one-hot and exercises the rescale of the running
    # output. In this regime the oracle itself is noisy: it rounds every q*k product (up to ~16
    # here) to fp16, which moves logits by ~1e-2 and outputs by ~1e-2. So the kernel is held to the
    # tight bound against the exact fp64 answer and to a loose one against the oracle.
    q, k, v = make_inputs(11, 1, 2, 1024, 128)
    q = (q.astype(np.float32) * 4).astype(np.float16)
    exact = exact_attention(q, k, v, 0.5, True)
    want = ob.attention(q, k, v, causal=True, scale=0.5)
    for kernel in (0, 1):
        got = run_gpu(pkg, q, k, v, True, -1, -1, kernel, scale=0.5)
        assert_close(ob, got, exact, max_abs=4e-3)  # |o| reaches 4+: one fp16 ulp there is 3.9e-3
        assert_close(ob, got, want, max_abs=5e-2, mean_abs=1e-3)


@pytest.mark.parametrize("scale", [1e-20, 1e-6])
def test_tiny_scale_keeps_hidden_keys_hidden(pkg, ob, scale):
    # The kernel hides a masked score by pushing it to about -3e38 BEFORE the scale is applied. With a scale near the
    # smallest the host accepts every visible key gets the same weight, so row i of a causal, left-windowed call is
    # the plain mean of V over its visible keys; a hidden key that leaked back in would show as a wrong mean.
    N, d, wl = 700, 64, 200
    q, k, v = make_inputs(17, 1, 2, N, d)
    got = run_gpu(pkg, q, k, v, True, wl, -1, 0, scale=scale).astype(np.float64)
    v64 = v.astype(np.float64)
    csum = np.concatenate([np.zeros((1, 2, 1, d)), np.cumsum(v64, axis=2)], axis=2)
    for i in (0, 1, 127, 128, 199, 200, 201, 333, 511, 512, 699):
        lo = max(0, i - wl)
        want = (csum[:, :, i + 1] - csum[:, :, lo]) / (i + 1 - lo)
        assert np.abs(got[:, :, i] - want).max() <= 2e-3, i


def test_growing_row_max_forces_rescale(pkg, ob):
    # keys ordered so that every later kv tile raises the row max by far more than the lazy threshold
    N, d = 1024, 64
    rng = np.random.default_rng(12)
    q = np.ones((1, 1, N, d), np.float16)
    k = (np.arange(N, dtype=np.float32)[:, None] / 8.0 * np.ones((1, d), np.float32) / d * 8).astype(np.float16)
    k = k.reshape(1, 1, N, d)
    v = rng.standard_normal((1, 1, N, d), dtype=np.float32).astype(np.float16)
    for kernel in (0, 1):
        got = run_gpu(pkg, q, k, v, False, -1, -1, kernel, scale=1.0)
        want = ob.attention(q, k, v, scale=1.0)
        assert_close_or_one_ulp(got, want)


def test_deterministic_and_kernels_agree(pkg, ob):
    q, k, v = make_inputs(13, 2, 4, 768, 128)
    a = run_gpu(pkg, q, k, v, True)
    b = run_gpu(pkg, q, k, v, True)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    c = run_gpu(pkg, q, k, v, True, kernel=1)
    mx, mean, nans = ob.abs_error(a, c)
    assert nans == 0 and mx <= 2e-3 and mean <= 5e-5


def test_head_shards_equal_full_call(pkg):
    # the multi-GPU partition: a slab of (batch, head) computed alone equals its slice of the full call
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    q, k, v = (torch.randn((2, 8, 1024, 128), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    full = pkg.attention_forward(q, k, v, causal=True).reshape(16, 1024, 128)
    qf, kf, vf = (x.reshape(1, 16, 1024, 128) for x in (q, k, v))
    for world in (2, 4, 8):
        per = 16 // world
        for r in range(world):
            sl = slice(r * per, (r + 1) * per)
            part = pkg.attention_forward(qf[:, sl].contiguous(), kf[:, sl].contiguous(), vf[:, sl].contiguous(),
                                         causal=True)
            assert torch.equal(part[0], full[sl])


def test_reference_entry_point_mapping(pkg, ob, capfd):
    # run_flash_attention(B, heads, S, d, Q, K, V, O, L, M, dropout, causal, local, alibi, window, ...)
    import torch

    q, k, v = make_inputs(17, 1, 2, 512, 64)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    to = torch.empty_like(tq)
    torch.cuda.synchronize()
    pkg.run_flash_attention(1, 2, 512, 64, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), to.data_ptr(), None, None,
                            False, True, True, False, 100)
    assert "TIME:" in capfd.readouterr().out
    want = ob.attention(q, k, v, causal=True, window_left=100, window_right=100)  # symmetric window + causal
    assert_close(ob, to.cpu().numpy(), want)
    pkg.run_flash_attention(1, 2, 512, 64, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), to.data_ptr(), None, None,
                            False, False, True, False, 64)
    want = ob.attention(q, k, v, causal=False, window_left=64, window_right=64)
    assert_close(ob, to.cpu().numpy(), want)
    with pytest.raises(pkg.FlashForwardError):
        pkg.run_flash_attention(1, 2, 512, 64, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), to.data_ptr(),
                                Has_alibi=True)


def test_host_buffer_entry_point(pkg, ob):
    import torch

    B, H, N, d = 2, 5, 640, 128
    q, k, v = make_inputs(19, B, H, N, d)
    hq, hk, hv = (torch.from_numpy(a).pin_memory() for a in (q, k, v))
    ho = torch.empty((B, H, N, d), dtype=torch.float16).pin_memory()
    chunk = 3  # 10 heads -> chunks of 3, 3, 3, 1
    nbytes = pkg.host_workspace_bytes(N, d, chunk)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    pkg.flash_forward_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(), B, H, N, d, ws.data_ptr(),
                           nbytes, chunk, is_causal=True)
    want = ob.attention(q, k, v, causal=True)
    assert_close(ob, ho.numpy(), want)
    dev = run_gpu(pkg, q, k, v, True)
    assert np.array_equal(dev.view(np.uint16), ho.numpy().view(np.uint16))
    with pytest.raises(pkg.FlashForwardError):
        pkg.flash_forward_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(), B, H, N, d, ws.data_ptr(),
                               nbytes - 1, chunk)
