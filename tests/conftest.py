import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for path in (ROOT, HERE):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def no_index_check_failed(request):
    """In the debug build (TORCHLET_B200_DEBUG=1) every GPU test also asserts that no kernel's index
    check has fired: page ids, positions, slots and token ids stayed inside their ranges."""
    yield
    if "gpu" not in request.keywords:
        return
    from torchlet_b200.csrc.build import DEBUG_BUILD

    if DEBUG_BUILD:
        import torch

        from torchlet_b200 import ops

        torch.cuda.synchronize()
        assert ops.debug_errors() == []
