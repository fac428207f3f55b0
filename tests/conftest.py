import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs at least one CUDA device (B200)')
    config.addinivalue_line('markers', 'multigpu: needs two or more CUDA devices')


def pytest_collection_modifyitems(config, items):
    import torch
    num_gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if 'gpu' in item.keywords and num_gpus == 0:
            item.add_marker(pytest.mark.skip(reason='no CUDA device'))
        if 'multigpu' in item.keywords and num_gpus < 2:
            item.add_marker(pytest.mark.skip(reason='needs >= 2 CUDA devices'))


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


@pytest.fixture
def master_port():
    return free_port()
