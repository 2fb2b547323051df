import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # The file whose name starts with test_zz runs last.
    items.sort(key=lambda item: (Path(str(item.fspath)).name.startswith("test_zz"),))


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny model folders written by the tests' own writer: name -> (folder, config, numpy weights)."""
    import tiny_models

    out = {}
    base = tmp_path_factory.mktemp("models")
    for tag, cfg, seed, scale in (("A", tiny_models.TINY_A, 11, 4.0), ("B", tiny_models.TINY_B, 12, 4.0),
                                  ("C", tiny_models.TINY_C, 13, 4.0), ("D", tiny_models.TINY_D, 14, 4.0),
                                  ("E", tiny_models.TINY_E, 15, 2.0)):
        weights = tiny_models.numpy_weights(cfg, seed, scale=scale, bf16_exact=True)
        folder = tiny_models.write_folder(base / tag, cfg, weights)
        out[tag] = (folder, cfg, weights)
    return out
