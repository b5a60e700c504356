"""velox_b200: sm_100a decode-step library for Velox models (C ABI in include/velox_b200.h)."""
from . import lib  # noqa: F401
from .modelspec import ModelSpec, SPECS  # noqa: F401

__all__ = ["lib", "ModelSpec", "SPECS"]
