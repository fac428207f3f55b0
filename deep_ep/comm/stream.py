"""The process-wide communication stream (reference: `deep_ep/comm/stream.py:9-12`)."""
from typing import Any

import torch

from .._C_loader import _C


def get_comm_stream(buffer: Any = None) -> torch.cuda.Stream:
    """Return the single high-priority stream on which bucket collectives run; `buffer` is ignored."""
    stream_id, device_index, device_type = _C.get_comm_stream()
    return torch.cuda.Stream(stream_id=stream_id, device_index=device_index, device_type=device_type)
