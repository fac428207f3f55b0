"""`EventOverlap`: wait for a recorded event, then run a one-shot deferred epilogue.

Reference: `deep_ep/utils/event.py:8-94`. `EventHandle` is the native CUDA event wrapper of the
extension; on a machine without CUDA a no-op stand-in keeps the CPU test tier running.
"""
from typing import Any, Callable, Optional, Tuple

import torch

from .._C_loader import _C

EventHandle = _C.EventHandle


class EventOverlap:
    """Holds an event plus at most one hook that runs after the first wait.

    Attributes:
        event: the recorded event (or `None` once released).
        extra_tensors: tensors kept alive for as long as this object lives.
    """

    def __init__(self, event: Optional[EventHandle] = None,
                 extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self.hook_after_wait: Optional[Callable[[], Any]] = None
        self._release_on_exit = False

    def current_stream_wait(self, release_handle: bool = False) -> Any:
        """Make the current stream wait for the event; run and clear the hook; return its result."""
        assert self.event is not None, 'the event handle has already been released'
        self.event.current_stream_wait()
        hook, self.hook_after_wait = self.hook_after_wait, None
        result = hook() if hook is not None else None
        if release_handle:
            self.event = None
        return result

    def wait(self) -> Any:
        return self.current_stream_wait()

    def register_hook_after_wait(self, hook_after_wait: Callable[[], Any]) -> None:
        assert self.hook_after_wait is None, 'A hook is already registered on this `EventOverlap`'
        self.hook_after_wait = hook_after_wait

    def __call__(self, release_handle: bool = False) -> 'EventOverlap':
        """`with event_overlap(release_handle=True): ...` — configures the exit behaviour."""
        self._release_on_exit = release_handle
        return self

    def __enter__(self) -> 'EventOverlap':
        return self

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        release, self._release_on_exit = self._release_on_exit, False
        if self.event is not None:
            self.current_stream_wait(release_handle=release)
