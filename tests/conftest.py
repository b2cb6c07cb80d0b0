import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "reference_cases.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def seeded():
    """Committed CPU-oracle vectors of small seeded layers (tests/golden/make_golden.py)."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "seeded_cases.npz")
    with np.load(path) as z:
        return {k: z[k] for k in z.files}
