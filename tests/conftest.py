import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def scenes(pkg):
    from gradoom_b200 import scene as gdscene

    cache = {}

    def get(name, ray_tables=None):
        key = (name, ray_tables is not None)
        if key not in cache:
            sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[name])
            cache[key] = (sc, gdscene.pack_scene(sc, ray_table_override=ray_tables))
        return cache[key]

    return get


def load_golden(name):
    path = os.path.join(GOLDEN, f"golden_{name}.npz")
    if not os.path.exists(path):
        pytest.skip(f"fixture {path} not generated")
    return np.load(path)


def pad_things(things, k):
    out = np.zeros((things.shape[0], k, 4), dtype=np.int32)
    out[:, : things.shape[1]] = things
    return out
