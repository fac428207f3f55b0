"""Device barrier over a buffer's communication context (reference: `deep_ep/comm/barrier.py:7-12`)."""
from typing import Any, Optional

import torch.distributed as dist

from .._C_loader import _C


def barrier(buffer: Any, wait_comm_stream: bool = True, with_cpu_sync: bool = False,
            sequential: bool = True, context_idx: Optional[int] = None) -> None:
    """Cross-rank barrier on the current stream; optionally joins the communication stream and the host."""
    context = buffer.context if context_idx is None else buffer.contexts[context_idx]
    if isinstance(context, _C.Context):
        _C.barrier(context, with_cpu_sync, sequential, wait_comm_stream)
    else:  # CPU simulation contexts
        dist.barrier(buffer.group if context_idx is None else buffer.groups[context_idx])
