import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    return json.loads((ROOT / "tests" / "golden" / "encoding_words.json").read_text())


@pytest.fixture(scope="session")
def host_codec():
    """Context without a GPU: table metadata and ELF helpers only."""
    import cubit_b200
    return cubit_b200.Codec(devices=())


@pytest.fixture(scope="session")
def codec():
    """Context on cuda:0.  Fails (does not skip) when the CUDA library cannot run."""
    import cubit_b200
    return cubit_b200.Codec(devices=(0,))
