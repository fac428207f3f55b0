"""Tiny semantic helpers shared by the Python API layer."""
from typing import Any, Optional


def value_or(value: Optional[Any], default: Any) -> Any:
    """Return `value` unless it is `None` (reference: deep_ep/utils/semantic.py:4-5)."""
    return value if value is not None else default


def nvtx_range(name: str):
    """Decorator: with `EP_NVTX=1` in the environment at import time, the call runs inside an NVTX range of that name
    (visible in Nsight Systems / `torch.profiler` timelines); otherwise the function is returned unchanged, so the
    default path pays nothing. The reference brackets its kernels with device trace stamps under a build flag
    (`deep_ep/include/deep_ep/impls/ep/dispatch.hpp:643-653`); ranges on the host side are the CUDA counterpart."""
    import functools
    import os

    def decorate(fn):
        if os.environ.get('EP_NVTX', '0') != '1':
            return fn

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            import torch
            if not torch.cuda.is_available():
                return fn(*args, **kwargs)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        return wrapper
    return decorate
