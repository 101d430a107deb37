import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "golden.pt")
    return torch.load(path, map_location="cpu", weights_only=True)


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def dry_backend(tmp_path_factory):
    """The backend registered for CPU tensors in dry-run mode: sources are emitted and built
    with nvcc exactly as on a GPU, nothing is launched."""
    import shutil

    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available")
    os.environ["IXB_CACHE_DIR"] = str(tmp_path_factory.mktemp("ixbcache"))
    import inductor_x_b200  # noqa: F401
    from inductor_x_b200 import config
    from inductor_x_b200.prebuild import _dry_cpu_backend

    old_dir = config.cache_dir
    config.cache_dir = os.environ["IXB_CACHE_DIR"]
    with _dry_cpu_backend(False):
        yield
    config.cache_dir = old_dir
