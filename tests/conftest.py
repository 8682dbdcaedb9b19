import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA GPU (B200)")
    config.addinivalue_line("markers", "multigpu: needs two or more GPUs (also marked gpu)")


def _gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:  # noqa: BLE001
        return 0


def pytest_collection_modifyitems(config, items):
    n = _gpu_count()
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no GPU"))
        need = item.get_closest_marker("multigpu")
        if need is not None:
            want = need.args[0] if need.args else 2
            if n < want:
                item.add_marker(pytest.mark.skip(reason=f"needs {want} GPUs, have {n}"))


@pytest.fixture(scope="session")
def native_lib():
    from yali_b200 import _native
    return _native.lib()


@pytest.fixture(scope="session")
def free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port
