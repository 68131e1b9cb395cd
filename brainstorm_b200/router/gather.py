"""Gather router: combine fabric only (counterpart of python/brt/router/gather.py:19-54)."""
from typing import Any, Dict

from .base import RouterBase, register_router
from .fabric import make_fabric

__all__ = ["GatherRouter"]


@register_router("gather")
class GatherRouter(RouterBase):
    def __init__(self, fabric_type: str = "combine", fabric_kwargs: Dict[str, Any] = None):
        """fabric kwargs: reduction ("add"), transform (scale by score), max_path_padding,
        ever_padded, index_format."""
        super().__init__()
        self.fabric_type = fabric_type
        self.fabric_kwargs = {"flow_num": 1, "reduction": "add", "sparse": False} \
            if "combine" in fabric_type else {}
        self.fabric_kwargs.update(fabric_kwargs or {})
        self.fabric = make_fabric(fabric_type, self.fabric_kwargs)

    def forward(self, in_flows, residual_flows=None, score=None):
        return self.fabric(in_flows, residual_flows, score)
