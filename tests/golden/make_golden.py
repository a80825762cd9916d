"""Generates the golden attention vectors in this directory from the REFERENCE's own CPU attention.

Run where the reference sources are available and `make -C oracle` has produced
oracle/_ref/libref_attention.so (the reference's src/main.cu compiled unmodified):

    python tests/golden/make_golden.py

Each case_*.npz holds the fp16 bits of q, k, v and of the reference output, plus the call's
parameters. The tests then check the C restatement (and, on a GPU, the CUDA kernels) against
these files on machines where the reference sources do not exist.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as ob  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name, B, H, N, d, causal, window (symmetric, -1 = none), alibi, input distribution
CASES = [
    ("c1_b1h4n512d64_full", 1, 4, 512, 64, 0, -1, 0, "normal"),          # BASELINE config 1, whole
    ("n256d64_full", 1, 1, 256, 64, 0, -1, 0, "normal"),
    ("n256d128_causal", 1, 2, 256, 128, 1, -1, 0, "normal"),
    ("n384d64_causal_w128", 1, 1, 384, 64, 1, 128, 0, "normal"),          # causal + window, as config 4 combines them
    ("n256d64_w100", 1, 1, 256, 64, 0, 100, 0, "normal"),                 # symmetric window, not a multiple of 128
    ("n256d128_causal_w37", 1, 1, 256, 128, 1, 37, 0, "normal"),
    ("n256d64_causal_alibi", 1, 2, 256, 64, 1, -1, 1, "normal"),          # the reference's ALiBi bias (flash_forward_alibi / Has_alibi)
    ("n256d64_uniform0_10", 1, 1, 256, 64, 0, -1, 0, "uniform"),          # the reference's own smoke distribution
]


def inputs(seed, B, H, N, d, dist):
    rng = np.random.default_rng(seed)
    if dist == "normal":
        return [rng.standard_normal((B, H, N, d), dtype=np.float32).astype(np.float16) for _ in range(3)]
    return [rng.uniform(0.0, 10.0, (B, H, N, d)).astype(np.float32).astype(np.float16) for _ in range(3)]


def main():
    if not ob.ref_available():
        raise SystemExit("oracle/_ref/libref_attention.so is missing: run `make -C oracle` where the reference exists")
    for idx, (name, B, H, N, d, causal, w, alibi, dist) in enumerate(CASES):
        q, k, v = inputs(26 + idx, B, H, N, d, dist)
        slopes = None
        if alibi:  # the reference's slope formula, src/main.cu:41
            slopes = np.array([-(2.0 ** (-8.0 / H * (i + 1))) for i in range(H)], dtype=np.float32)
        out = ob.reference_attention(q, k, v, bool(causal), w, alibi_slopes=slopes)
        np.savez(os.path.join(HERE, f"case_{name}.npz"), q=q.view(np.uint16), k=k.view(np.uint16), v=v.view(np.uint16),
                 out=out.view(np.uint16), causal=causal, window=w, alibi=alibi,
                 slopes=slopes if slopes is not None else np.zeros(0, np.float32))
        print(name, "written; |out| max", float(np.abs(out.astype(np.float32)).max()))


if __name__ == "__main__":
    main()
