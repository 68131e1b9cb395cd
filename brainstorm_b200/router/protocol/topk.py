"""Top-k protocol (python/brt/router/protocol/topk.py:13-31): ones at the k best-scored paths
of every cell."""
import torch

from .base import ProtocolBase, register_protocol

__all__ = ["TopKProtocol"]


@register_protocol("topk")
class TopKProtocol(ProtocolBase):
    def __init__(self, top_k: int = 1):
        super().__init__()
        self.top_k = top_k

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        picks = torch.topk(score, self.top_k, dim=1).indices
        mask = torch.zeros(score.shape, dtype=torch.int32, device=score.device)
        return mask.scatter_(1, picks, 1)
