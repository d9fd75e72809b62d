import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# Rendez-vous on the loopback interface: the container host name may not resolve.
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multi_gpu(n): needs at least n CUDA devices")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    try:
        import torch

        n_gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:  # pragma: no cover
        n_gpus = 0
    for item in items:
        if "gpu" in item.keywords and n_gpus == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        marker = item.get_closest_marker("multi_gpu")
        if marker is not None:
            need = marker.args[0] if marker.args else 2
            if n_gpus < need:
                item.add_marker(pytest.mark.skip(reason=f"needs {need} CUDA devices, found {n_gpus}"))
