"""Routers: ScatterRouter / GatherRouter and their protocols and fabrics
(counterpart of the reference's ``brt.router`` package)."""
from .base import RouterBase, is_router, make_router, register_router
from .fabric.base import reset_router_stats, switch_capture
from .gather import GatherRouter
from .scatter import ScatterRouter, SwinMoEScatterRouter, TaskScatterRouter

__all__ = ["RouterBase", "is_router", "make_router", "register_router", "reset_router_stats",
           "switch_capture", "GatherRouter", "ScatterRouter", "SwinMoEScatterRouter",
           "TaskScatterRouter"]
