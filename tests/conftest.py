import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


def _has_gpu():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pkg():
    """The product package; its shared library must exist (no fallback)."""
    p = entry.load_package()
    p.lib()
    return p


@pytest.fixture(scope="session")
def ob():
    """The CPU oracle bindings (test infrastructure)."""
    b = entry.load_oracle()
    if not os.path.exists(b.PORT_PATH):
        entry._run(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle_attn.so"], ROOT)
    b.port()
    return b


def make_inputs(seed, B, H, N, d, dist="normal"):
    """Seeded fp16 Q, K, V as numpy arrays: i.i.d. N(0,1) (the benchmark's distribution) or
    U(0,10) (the reference's own smoke distribution, src/main.cu:70)."""
    rng = np.random.default_rng(seed)
    if dist == "normal":
        return [rng.standard_normal((B, H, N, d), dtype=np.float32).astype(np.float16) for _ in range(3)]
    return [rng.uniform(0.0, 10.0, (B, H, N, d)).astype(np.float32).astype(np.float16) for _ in range(3)]


GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def golden_cases():
    return sorted(f for f in os.listdir(GOLDEN_DIR) if f.startswith("case_") and f.endswith(".npz"))
