"""Fabrics: move cells according to a hot mask."""
from . import distributed, distributed_slots, fused, generic  # noqa: F401  (registration)
from .base import FabricBase, make_fabric, register_fabric

__all__ = ["FabricBase", "make_fabric", "register_fabric"]
