"""B200-native implementation of EOQ's inference hot path (see include/eoq_b200.h)."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
