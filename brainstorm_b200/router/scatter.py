"""Scatter routers: protocol (scores -> hot mask) + dispatch fabric
(counterpart of python/brt/router/scatter.py:20-255)."""
from typing import Any, Dict

import torch

from .base import RouterBase, register_router
from .fabric import make_fabric
from .protocol import make_protocol

__all__ = ["ScatterRouter", "SwinMoEScatterRouter", "TaskScatterRouter"]

_PROTOCOL_DEFAULTS = {
    "topk": {"top_k": 1},
    "threshold": {"threshold": 0.0, "residual_path": -1},
}


def _dispatch_defaults(dispatch_score: bool) -> Dict[str, Any]:
    if dispatch_score:
        # second flow: the score matrix itself, routed element-wise (path e gets score[t, e])
        return {"flow_num": 2, "route_logic": ["1d", "2d"], "transform": [False, False]}
    return {"flow_num": 1, "route_logic": "1d", "transform": False}


class _FabricIndexRules:
    """(supported_capacities, capacity_padding, path_wise_padding) of a dispatch fabric, read
    when called (the capacities are a buffer that moves with the module).  A plain object, so
    that the protocol holding it does not register the fabric as a submodule of its own."""

    def __init__(self, fabric):
        self.fabric = fabric

    def __call__(self):
        f = self.fabric
        return f.supported_capacities, bool(f.capacity_padding), bool(f.path_wise_padding)


class _ScoreScatterBase(RouterBase):
    def __init__(self, dispatch_score=False, protocol_type: str = "topk",
                 fabric_type: str = "dispatch", protocol_kwargs: Dict[str, Any] = None,
                 fabric_kwargs: Dict[str, Any] = None):
        super().__init__()
        self.dispatch_score = dispatch_score
        self.protocol_type = protocol_type
        self.protocol_kwargs = dict(_PROTOCOL_DEFAULTS.get(protocol_type, {}))
        self.protocol_kwargs.update(protocol_kwargs or {})
        self.protocol = make_protocol(protocol_type, self.protocol_kwargs)
        self.fabric_type = fabric_type
        self.fabric_kwargs = _dispatch_defaults(dispatch_score) if "dispatch" in fabric_type \
            else {}
        self.fabric_kwargs.update(fabric_kwargs or {})
        self.fabric = make_fabric(fabric_type, self.fabric_kwargs)
        if hasattr(self.fabric, "capacity_padding") and \
                hasattr(self.protocol, "index_rules_of"):
            # the fabric scans the hot mask for seat indices under these rules: a protocol that
            # runs the library's gate kernel does that scan in the same launch
            self.protocol.index_rules_of = _FabricIndexRules(self.fabric)

    def _route(self, in_flows, score):
        hot_mask = self.protocol(score)
        if self.dispatch_score:
            in_flows = in_flows + [score] if isinstance(in_flows, list) else [in_flows, score]
        return self.fabric(in_flows, hot_mask, None, score)


@register_router("scatter")
class ScatterRouter(_ScoreScatterBase):
    """protocol_type: "topk" (top_k) | "threshold" (threshold, residual_path) | any registered
    protocol; fabric_type: "dispatch" | "fused_dispatch" | "distributed_fused_dispatch" ...;
    dispatch_score additionally routes the score matrix as a second flow."""

    def forward(self, in_flows, score: torch.Tensor):
        out_flows, _ = self._route(in_flows, score)
        return out_flows


@register_router("task_scatter")
class TaskScatterRouter(_ScoreScatterBase):
    """Same as ScatterRouter but also returns the score handed back by the fabric (task ids
    for the task-locality variant of the distributed fabric)."""

    def forward(self, in_flows, score: torch.Tensor):
        return self._route(in_flows, score)


@register_router("swin_moe_scatter")
class SwinMoEScatterRouter(RouterBase):
    ALLOWED_PROTOCOL_TYPES = ["swin_moe"]

    def __init__(self, protocol_type: str = "swin_moe", fabric_type: str = "dispatch",
                 protocol_kwargs: Dict[str, Any] = None, fabric_kwargs: Dict[str, Any] = None):
        super().__init__()
        assert protocol_type in self.ALLOWED_PROTOCOL_TYPES, \
            f"protocol_type {protocol_type} is not supported by SwinMoEScatterRouter"
        self.protocol_type = protocol_type
        self.protocol_kwargs = {
            "top_k": 1, "capacity_factor": 0, "gate_noise": 0.0, "group": None,
            "is_postscore": True, "batch_prioritized_routing": False, "normalize_gate": True,
            "is_gshard_loss": True, "alignment": 1,
        }
        self.protocol_kwargs.update(protocol_kwargs or {})
        self.protocol = make_protocol(protocol_type, self.protocol_kwargs)
        self.fabric_type = fabric_type
        self.fabric_kwargs = {"flow_num": 1, "route_logic": ["1d"], "transform": [False]}
        self.fabric_kwargs.update(fabric_kwargs or {})
        self.fabric = make_fabric(fabric_type, self.fabric_kwargs)
        if hasattr(self.fabric, "capacity_padding"):
            self.protocol.index_rules = (bool(self.fabric.capacity_padding),
                                         bool(self.fabric.path_wise_padding))

    def forward(self, in_flows, score, logits_wo_noise=None, logits=None):
        hot_mask, runtime_capacities, new_score, _loss = self.protocol(score, logits_wo_noise,
                                                                       logits)
        if self.fabric.max_path_load == 0:
            # every path has the same runtime capacity; known on the host without a sync
            self.fabric.max_path_load = self.protocol.runtime_capacity(score.size(0),
                                                                       score.size(1))
        return self.fabric(in_flows, hot_mask, runtime_capacities, new_score)
