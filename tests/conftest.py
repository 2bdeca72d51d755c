import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))



def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def weight_files(tmp_path_factory):
    """Factory: (recipe, seed) -> (path of a synthetic SHLDV001 file, its tensors); generated once per session."""
    from shield_sisa_b200 import weights as W

    cache = {}
    base = tmp_path_factory.mktemp("weights")

    def get(recipe="W3", seed=1):
        key = (recipe, seed)
        if key not in cache:
            path = base / f"{recipe.lower()}_s{seed}.weights"
            cache[key] = (path, W.synth_weight_file(path, seed, recipe))
        return cache[key]

    return get
