"""Carrier types and plumbing used by the routers (counterpart of ``brt.runtime``)."""
from .registry import Registry  # noqa: F401
from . import log  # noqa: F401
