import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu); everything else runs on CPU")


@pytest.fixture(scope="session")
def golden_small():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "small_cases.npz"))


@pytest.fixture(scope="session")
def golden_config1():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "config1_samples.npz"))


@pytest.fixture(scope="session")
def golden_conv1d():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "conv1d_cases.npz"))


@pytest.fixture(scope="session")
def oracle():
    from oracle import nectar_oracle
    nectar_oracle.build()
    return nectar_oracle


@pytest.fixture(scope="session")
def lib():
    from nectarml_b200 import build, _lib
    build.build()
    return _lib.load()
