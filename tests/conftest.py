import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on a B200)')


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


def seeded_weight(k: int, n: int, seed: int = 0, std: float = 0.02, dtype=np.float16) -> np.ndarray:
    """W ~ N(0, std^2), drawn in float32 and cast, as the benchmark configurations describe."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((k, n), dtype=np.float32) * np.float32(std)).astype(dtype)


def seeded_activation(m: int, k: int, seed: int = 1, dtype=np.float16) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.standard_normal((m, k), dtype=np.float32).astype(dtype)


@pytest.fixture(scope='session')
def oracle_lib():
    import oracle

    return oracle
