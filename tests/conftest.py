import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu); everything else runs on CPU")


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(ROOT / "tests" / "golden" / "reference_vectors.pt", weights_only=True)


@pytest.fixture(scope="session")
def lib():
    from feather_ops_b200 import _lib

    return _lib.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test ran without a CUDA device: the kernels have no fallback")
    return torch.device("cuda:0")
