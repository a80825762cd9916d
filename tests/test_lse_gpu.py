"""flash_forward_lse on the GPU: the log-sum-exp output against its definition evaluated in float64
on the same fp16 inputs, and O against the plain entry point. The reference never writes its L/M
outputs (src/flash_forward.h:602-603), so there are no reference vectors for this output; the
tolerance is 5e-4 absolute on ln-units (fp32 scores from the tensor cores, ex2/lg2 approximations)."""
import numpy as np
import pytest

from conftest import make_inputs

pytestmark = pytest.mark.gpu
LSE_TOL = 5e-4


def run(pkg, q, k, v, **kw):
    import torch

    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    slopes = kw.pop("alibi_slopes", None)
    ts = None if slopes is None else torch.from_numpy(slopes).cuda()
    out, lse = pkg.attention_forward(tq, tk, tv, alibi_slopes=ts, return_lse=True, **kw)
    plain = pkg.attention_forward(tq, tk, tv, alibi_slopes=ts, **kw)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    return out.cpu().numpy(), lse.cpu().numpy(), plain.cpu().numpy()


@pytest.mark.parametrize("N,d,causal,wl,wr", [
    (333, 128, False, -1, -1),    # ragged, one item per head
    (1000, 64, True, -1, -1),     # ragged causal
    (1024, 128, True, 256, -1),   # causal + left window
    (700, 64, False, 100, 50),    # two-sided window, ragged
    (2048, 64, False, -1, -1),    # many unmasked tiles: the running sum crosses lazy rescales
    (128, 64, True, 0, -1),       # every row sees exactly itself
])
def test_lse_matches_definition(pkg, ob, N, d, causal, wl, wr):
    q, k, v = make_inputs(500 + N + d, 2, 3, N, d)
    out, lse, plain = run(pkg, q, k, v, causal=causal, window_left=wl, window_right=wr)
    want = ob.log_sum_exp_fp64(q, k, causal=causal, window_left=wl, window_right=wr)
    assert np.isfinite(lse).all()
    assert np.abs(lse - want).max() <= LSE_TOL
    assert np.array_equal(out.view(np.uint16), plain.view(np.uint16))  # O does not depend on the lse output


def test_lse_with_alibi_and_scale(pkg, ob):
    import torch

    H, N, d = 4, 640, 128
    q, k, v = make_inputs(611, 1, H, N, d)
    slopes = np.array([-(2.0 ** (-8.0 / H * (i + 1))) for i in range(H)], dtype=np.float32)  # src/main.cu:41
    out, lse, plain = run(pkg, q, k, v, causal=True, alibi_slopes=slopes)
    want = ob.log_sum_exp_fp64(q, k, causal=True, alibi_slopes=slopes)
    assert np.abs(lse - want).max() <= 2e-3  # the bias reaches |slope| * N ~ 450 ln-units: fp32 spacing there is 3e-5
    assert np.array_equal(out.view(np.uint16), plain.view(np.uint16))

    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    _, lse2 = pkg.attention_forward(tq, tk, tv, softmax_scale=0.25, return_lse=True)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    want2 = ob.log_sum_exp_fp64(q, k, softmax_scale=0.25)
    assert np.abs(lse2.cpu().numpy() - want2).max() <= 2e-3  # logits of +-40


def test_lse_growing_row_max(pkg, ob):
    """Keys grow along the sequence, so the running max moves in every tile and the lazy threshold is
    crossed repeatedly; the final (max, sum) pair must still describe the whole row."""
    N, d = 1536, 64
    rng = np.random.default_rng(9)
    q = np.abs(rng.standard_normal((1, 2, N, d), dtype=np.float32)).astype(np.float16)
    ramp = np.linspace(0.05, 3.0, N, dtype=np.float32)[None, None, :, None]
    k = (np.abs(rng.standard_normal((1, 2, N, d), dtype=np.float32)) * ramp).astype(np.float16)
    v = rng.standard_normal((1, 2, N, d), dtype=np.float32).astype(np.float16)
    _, lse, _ = run(pkg, q, k, v, causal=False)
    want = ob.log_sum_exp_fp64(q, k)
    assert np.abs(lse - want).max() <= 2e-3


def test_lse_config_3_sampled(pkg, ob):
    """BASELINE config 3 (B2 H32 N8192 d128 causal): row 0 of every head sees one key, so its lse is the
    scaled dot product itself; sampled rows of the first and last head against the definition."""
    import torch

    B, H, N, d = 2, 32, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn((B, H, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    out, lse = pkg.attention_forward(q, k, v, causal=True, return_lse=True)
    pkg.check(torch.cuda.current_stream().cuda_stream)
    lse = lse.cpu().numpy()
    assert np.isfinite(lse).all()
    dot0 = (q[:, :, 0].double() * k[:, :, 0].double()).sum(-1).cpu().numpy() / np.sqrt(d)
    assert np.abs(lse[:, :, 0] - dot0).max() <= 1e-4
    rows = np.unique(np.concatenate([np.arange(0, 260), np.arange(4090, 4100), np.arange(N - 130, N),
                                     np.random.default_rng(1).integers(0, N, 64)]))
    for b, h in ((0, 0), (B - 1, H - 1)):
        qq, kk = (t[b:b + 1, h:h + 1].cpu().numpy() for t in (q, k))
        want = ob.log_sum_exp_fp64(qq, kk, causal=True, rows=rows)[0, 0]
        assert np.abs(lse[b, h, rows] - want).max() <= LSE_TOL
