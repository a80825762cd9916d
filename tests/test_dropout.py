"""Dropout on the attention probabilities: the reference's Is_dropout / dropout_prob (src/flash_forward.h:248-265,
src/init_curand_states.h:7-14). The reference skips its own check when dropout is on (src/main.cu:103) and its
random stream cannot be reproduced (one curand state per q tile, shared by every thread of the CTA), so this
feature is pinned by construction instead: the keep mask is Philox-4x32-10 on (seed, head, row, column), the
generator is held to the published known-answer vectors, the oracle applies the same mask inside the reference's
CPU arithmetic, and the kernel must agree with that oracle at the usual 2e-3 / 2e-4 bar."""
import ctypes

import numpy as np
import pytest

from conftest import make_inputs


def test_philox_known_answers(ob):
    """Philox-4x32-10 known-answer vectors of the Random123 distribution (counter, key -> output)."""
    fn = ob.port().oracle_philox4x32_10
    cases = [
        ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
         (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for ctr, key, want in cases:
        c = (ctypes.c_uint32 * 4)(*ctr)
        fn(ctypes.c_uint32(key[0]), ctypes.c_uint32(key[1]), c)
        assert tuple(c) == want


def test_keep_probability_is_quantised_to_256ths(pkg):
    kp = pkg.lib().flash_forward_dropout_keep_probability
    assert kp(0.0) == 1.0 and kp(0.001) == 1.0          # below 1/512: nothing is dropped
    assert kp(0.5) == 0.5 and kp(0.25) == 0.75 and kp(0.003) == 255 / 256
    assert kp(0.1) == 230 / 256 and kp(1.0) == 0.0
    assert kp(-0.1) == -1.0 and kp(1.5) == -1.0


def test_oracle_mask_statistics(ob):
    """Kept fraction of the oracle's mask within binomial bounds, and no visible structure along rows or columns."""
    for p, thr in ((0.1, 230), (0.5, 128), (0.9, 25)):
        n = 40000
        rng = np.random.default_rng(3)
        rows, cols = rng.integers(0, 4096, n), rng.integers(0, 4096, n)
        kept = sum(ob.dropout_keep(77, 5, int(r), int(c), thr) for r, c in zip(rows, cols))
        q = thr / 256
        assert abs(kept / n - q) < 5 * np.sqrt(q * (1 - q) / n)
    # neighbouring columns (same Philox block) and neighbouring rows are uncorrelated
    a = np.array([[ob.dropout_keep(1, 0, r, c, 128) for c in range(256)] for r in range(64)], dtype=np.float64)
    assert abs(np.corrcoef(a[:, :-1].ravel(), a[:, 1:].ravel())[0, 1]) < 0.03
    assert abs(np.corrcoef(a[:-1].ravel(), a[1:].ravel())[0, 1]) < 0.03
    # another seed or another head gives another mask
    b = np.array([[ob.dropout_keep(2, 0, r, c, 128) for c in range(256)] for r in range(64)], dtype=np.float64)
    c2 = np.array([[ob.dropout_keep(1, 1, r, c, 128) for c in range(256)] for r in range(64)], dtype=np.float64)
    assert 0.4 < (a != b).mean() < 0.6 and 0.4 < (a != c2).mean() < 0.6


def test_oracle_dropout_zero_is_plain_attention(ob):
    q, k, v = make_inputs(3, 1, 2, 200, 64)
    assert np.array_equal(ob.attention_dropout(q, k, v, 0.0, 9, causal=True).view(np.uint16),
                          ob.attention(q, k, v, causal=True).view(np.uint16))


def run_dropout(pkg, q, k, v, p, seed, causal=False, wl=-1, wr=-1, slopes=None):
    import torch

    tq, tk, tv = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, k, v))
    out = pkg.attention_forward(tq, tk, tv, causal=causal, window_left=wl, window_right=wr, dropout_p=p, seed=seed,
                                alibi_slopes=None if slopes is None else torch.from_numpy(slopes).cuda())
    pkg.check(torch.cuda.current_stream().cuda_stream)
    return out.cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("N,d,causal,wl,p", [
    (512, 64, False, -1, 0.1), (777, 128, True, -1, 0.5), (1024, 128, True, 200, 0.25), (300, 64, True, -1, 0.9),
])
def test_kernel_matches_oracle_with_the_same_mask(pkg, ob, N, d, causal, wl, p):
    q, k, v = make_inputs(500 + N, 2, 3, N, d)
    seed = 0x123456789abcdef0 + N
    got = run_dropout(pkg, q, k, v, p, seed, causal, wl, -1)
    want = ob.attention_dropout(q, k, v, p, seed, causal=causal, window_left=wl, window_right=-1)
    mx, mean, nans = ob.abs_error(got, want)
    # the kept probabilities are scaled by up to 1/(1-p): the absolute bar scales with them
    scale = 1.0 / max(pkg.lib().flash_forward_dropout_keep_probability(p), 1 / 256)
    assert nans == 0 and mx <= 2e-3 * max(1.0, scale) and mean <= 2e-4 * max(1.0, scale), (mx, mean, nans)
    # a wrong mask would show as errors of the size of the outputs themselves
    plain = ob.attention(q, k, v, causal=causal, window_left=wl, window_right=-1)
    assert ob.abs_error(got, plain)[1] > 20 * mean


@pytest.mark.gpu
def test_dropout_properties(pkg, ob):
    import torch

    q, k, v = make_inputs(71, 1, 4, 640, 128)
    plain = run_dropout(pkg, q, k, v, 0.0, 1, True)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    ref = pkg.attention_forward(tq, tk, tv, causal=True).cpu().numpy()
    assert np.array_equal(plain.view(np.uint16), ref.view(np.uint16))           # p = 0 is the plain forward, bit for bit
    a = run_dropout(pkg, q, k, v, 0.3, 42, True)
    b = run_dropout(pkg, q, k, v, 0.3, 42, True)
    c = run_dropout(pkg, q, k, v, 0.3, 43, True)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))                 # same seed, same bits
    assert not np.array_equal(a.view(np.uint16), c.view(np.uint16))             # another seed, another mask
    # V = 1 makes every output the kept, rescaled probability mass of its row: mean 1, spread of a binomial draw
    ones = np.ones_like(v)
    mass = run_dropout(pkg, q, k, ones, 0.5, 7, False).astype(np.float32)[..., 0]
    assert abs(mass.mean() - 1.0) < 0.02
    assert 0.02 < mass.std() < 0.5
    # everything dropped
    zero = run_dropout(pkg, q, k, v, 1.0, 7, True)
    assert np.all(zero == 0)
    # ALiBi and dropout together
    slopes = np.array([-(2.0 ** (-8.0 / 4 * (i + 1))) for i in range(4)], dtype=np.float32)
    got = run_dropout(pkg, q, k, v, 0.2, 5, True, slopes=slopes)
    want = ob.attention_dropout(q, k, v, 0.2, 5, causal=True, alibi_slopes=slopes)
    mx, mean, nans = ob.abs_error(got, want)
    assert nans == 0 and mx <= 4e-3 and mean <= 3e-4, (mx, mean)


@pytest.mark.gpu
def test_reference_entry_point_takes_dropout(pkg, capfd):
    """run_flash_attention(..., Is_dropout=true, ..., dropout_prob, states) of the reference (src/main.cu:99)."""
    import torch

    q, k, v = make_inputs(73, 1, 2, 512, 64)
    tq, tk, tv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    o1, o2 = torch.empty_like(tq), torch.empty_like(tq)
    torch.cuda.synchronize()
    for o in (o1, o2):
        pkg.run_flash_attention(1, 2, 512, 64, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), None, None,
                                True, True, False, False, 0, None, 0.25, None)
    assert "TIME:" in capfd.readouterr().out
    assert torch.isfinite(o1).all() and not torch.equal(o1, o2)   # the stream moves on from call to call
    plain = pkg.attention_forward(tq, tk, tv, causal=True)
    assert 1e-3 < (o1.float() - plain.float()).abs().mean().item() < 1.0
