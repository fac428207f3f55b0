"""Tiny semantic helpers shared by the Python API layer."""
from typing import Any, Optional


def value_or(value: Optional[Any], default: Any) -> Any:
    """Return `value` unless it is `None` (reference: deep_ep/utils/semantic.py:4-5)."""
    return value if value is not None else default
