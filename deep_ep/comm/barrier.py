"""Device barrier over a buffer's communication context (reference: `deep_ep/comm/barrier.py:7-12`).

On GPUs this launches the one-warp barrier kernel of the context on the current stream: every rank adds itself to a
phase counter in every peer's signal block and waits, with the context's time limit, until its own counter is complete;
a wait that runs out raises `EPException` naming the rank that stayed away (with `with_cpu_sync`, otherwise at the next
status check). CPU stand-in contexts (gloo ranks) use the process group's own barrier.
"""
from typing import Any, Optional

import torch.distributed as dist

from .._C_loader import _C


def _context_of(buffer: Any, context_idx: Optional[int]):
    """The buffer's only context, or one of the contexts of a buffer registered with several groups."""
    return buffer.context if context_idx is None else buffer.contexts[context_idx]


def _group_of(buffer: Any, context_idx: Optional[int]):
    return buffer.group if context_idx is None else buffer.groups[context_idx]


def barrier(buffer: Any, wait_comm_stream: bool = True, with_cpu_sync: bool = False,
            sequential: bool = True, context_idx: Optional[int] = None, *, repeats: int = 1) -> None:
    """Cross-rank barrier on the current stream; optionally joins the communication stream and the host.

    `repeats` > 1 runs that many barriers inside ONE kernel launch (every rank must pass the same number): the way to
    time the barrier itself rather than the host's launch rate (`benchmarks/comm_micro.py`).
    """
    assert repeats >= 1
    context = _context_of(buffer, context_idx)
    if _C is not None and isinstance(context, _C.Context):
        _C.barrier(context, with_cpu_sync, sequential, wait_comm_stream, repeats)
        return
    # CPU stand-in contexts: the process group's barrier, once per requested repeat
    for _ in range(repeats):
        dist.barrier(_group_of(buffer, context_idx))
