"""Router base class and registry (counterpart of python/brt/router/base.py).

The reference wraps router classes with its fx-tracing ``trace_init``; tracing is outside the
routing path, so registration here only records the type name.
"""
import inspect
from typing import Any, Callable, Dict

import torch.nn as nn

from ..runtime import Registry
from .utils import make_kwargs

__all__ = ["RouterBase", "register_router", "make_router", "is_router"]


class RouterBase(nn.Module):
    def __init__(self):
        super().__init__()


def register_router(router_type: str) -> Callable:
    register = Registry.register_sub_cls(router_type, RouterBase)

    def decorator(router_cls):
        if not (inspect.isclass(router_cls) and issubclass(router_cls, RouterBase)):
            raise ValueError(f"{router_cls} is not a subclass of RouterBase")
        router_cls._router_type = router_type
        return register(router_cls)

    return decorator


def make_router(router_type: str, kwargs: Dict[str, Any]) -> RouterBase:
    router_cls = Registry.get_sub_cls(router_type, RouterBase)
    if router_cls is None:
        raise ValueError(f"Router type: {router_type} is not registered.")
    return router_cls(**make_kwargs(kwargs))


def is_router(cls_or_instance) -> bool:
    router_cls = cls_or_instance if inspect.isclass(cls_or_instance) else type(cls_or_instance)
    return Registry.sub_cls_exists_and_registered(router_cls, RouterBase)
