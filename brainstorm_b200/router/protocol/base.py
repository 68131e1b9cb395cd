"""Protocol base class: a protocol maps gate scores to an int32 hot mask [cells, paths]
(counterpart of python/brt/router/protocol/base.py)."""
import os
from typing import Any, Callable, Dict

import torch
import torch.nn as nn

from ...runtime import Registry
from ..utils import make_kwargs

__all__ = ["ProtocolBase", "register_protocol", "make_protocol"]


class ProtocolBase(nn.Module):
    def __init__(self, **kwargs):
        super().__init__()
        self.debug = os.environ.get("BRT_DEBUG", "False").lower() in ("true", "1")
        # Set by a scatter router that owns this protocol and a seat-index dispatch fabric: a
        # callable returning (supported_capacities, capacity_padding, path_wise_padding) of
        # that fabric.  A protocol whose decision comes out of the library's gate kernel then
        # lets the same launch scan the mask and leaves (indices, loads) on the mask it
        # returns (``_brt_routes``); the fabric skips its own index scan.
        self.index_rules_of = None

    def _gate_with_indices(self, score: torch.Tensor, decision: str, **gate):
        """The hot mask of ``score`` with its seat indices and loads attached, all from one
        launch, or None when no fabric asked for them or the scores do not fit the kernel."""
        from ..._C import router as c_router

        if self.index_rules_of is None or not c_router.route_scores_supported(score):
            return None
        caps, cpad, pwise = self.index_rules_of()
        if caps is not None and not caps.is_cuda:
            return None
        try:
            indices, loads, hot_mask = c_router.route_scores(
                score, decision, output="seat_indices", supported_capacities=caps,
                capacity_padding=cpad, path_wise_padding=pwise, with_mask=True, **gate)
        except NotImplementedError:  # more scores than one launch takes
            return None
        hot_mask._brt_routes = (indices, loads, caps, cpad, pwise)
        return hot_mask

    def forward(self, score: torch.Tensor, *args, **kwargs):
        decisions = self.make_route_decision(score, *args, **kwargs)
        if self.debug:
            self.check_decision(decisions, score)
        return decisions

    def make_route_decision(self, score, **kwargs):
        raise NotImplementedError("make_route_decision has to be implemented by user")

    def check_decision(self, decisions, scores: torch.Tensor) -> None:
        hot_mask = decisions[0] if isinstance(decisions, (tuple, list)) else decisions
        assert hot_mask.size(0) == scores.size(0), \
            "indices and scores should have the same size in the first dimension"

    def check_compatibility(self, kwargs: Dict[str, Any]) -> None:
        pass


def register_protocol(protocol_type: str) -> Callable:
    return Registry.register_sub_cls(protocol_type, ProtocolBase)


def make_protocol(protocol_type: str, kwargs: Dict[str, Any]) -> ProtocolBase:
    protocol_cls = Registry.get_sub_cls(protocol_type, ProtocolBase)
    if protocol_cls is None:
        raise ValueError(f"Protocol type: {protocol_type} is not registered.")
    return protocol_cls(**make_kwargs(kwargs))
