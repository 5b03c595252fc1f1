import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


class RefOps:
    """Vectors produced by running the reference's own hot-path functions
    (tests/golden/make_golden.py)."""

    def __init__(self):
        self.z = np.load(GOLDEN / "ref_ops.npz")
        specs = json.loads(bytes(self.z["specs_json"]).decode())
        self.rulebooks = specs["rulebooks"]
        self.features = specs["features"]

    def get(self, key):
        return self.z[key]

    def has(self, key):
        return key in self.z.files

    def rb(self, name, key):
        return self.z[f"rb/{name}/{key}"]

    def rb_has(self, name, key):
        return f"rb/{name}/{key}" in self.z.files


@pytest.fixture(scope="session")
def ref_ops():
    return RefOps()


def rulebook_case_names():
    z = np.load(GOLDEN / "ref_ops.npz")
    specs = json.loads(bytes(z["specs_json"]).decode())
    return sorted(specs["rulebooks"].keys())


def feature_case_names():
    z = np.load(GOLDEN / "ref_ops.npz")
    specs = json.loads(bytes(z["specs_json"]).decode())
    return sorted(specs["features"].keys())
