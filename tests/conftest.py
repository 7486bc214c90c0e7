import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (its directory name has a hyphen, hence import_module)."""
    return importlib.import_module("odm-kv_b200")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure only)."""
    from oracle import odmkv_oracle
    odmkv_oracle.build_c()
    return odmkv_oracle


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    gdir = os.path.join(ROOT, "tests", "golden")
    return {name[:-4]: np.load(os.path.join(gdir, name)) for name in os.listdir(gdir) if name.endswith(".npz")}


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    importlib.import_module("odm-kv_b200")._lib.lib()  # fail loudly if the library is missing
    return torch.device("cuda:0")
