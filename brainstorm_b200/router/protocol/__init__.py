"""Routing protocols: gate scores -> int32 hot mask."""
from . import swin_moe, switch, threshold, topk  # noqa: F401  (registration side effects)
from .base import ProtocolBase, make_protocol, register_protocol

__all__ = ["make_protocol", "ProtocolBase", "register_protocol"]
