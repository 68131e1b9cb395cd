"""Fabrics: move cells according to a hot mask."""
from . import distributed, fused, generic  # noqa: F401  (registration side effects)
from .base import FabricBase, make_fabric, register_fabric

__all__ = ["FabricBase", "make_fabric", "register_fabric"]
