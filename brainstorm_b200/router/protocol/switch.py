"""Switch top-1 protocol (python/brt/router/protocol/switch.py:13-33): the gate already produced a
(capacity-masked) one-hot matrix; the protocol only flattens and casts it."""
import torch

from .base import ProtocolBase, register_protocol

__all__ = ["SwitchTop1Protocol"]


@register_protocol("switch_top1")
class SwitchTop1Protocol(ProtocolBase):
    def __init__(self):
        super().__init__()

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        return score.reshape(-1, score.shape[-1]).to(torch.int32)

    def update(self, supported_capacities):
        self.supported_capacities = supported_capacities
