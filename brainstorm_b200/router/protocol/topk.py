"""Top-k protocol (python/brt/router/protocol/topk.py:13-31): ones at the k best-scored paths
of every cell.  Contiguous fp32 CUDA scores over a multiple of 4 (at most 256) paths take the
library's single-launch gate; anything else the same torch ops as the reference.  Equal scores
go to the lower path in the gate kernel; the reference leaves them to ``torch.topk``."""
import torch

from ..._C import router as c_router
from .base import ProtocolBase, register_protocol

__all__ = ["TopKProtocol"]


@register_protocol("topk")
class TopKProtocol(ProtocolBase):
    def __init__(self, top_k: int = 1):
        super().__init__()
        self.top_k = top_k

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        if c_router.route_scores_supported(score) and 1 <= self.top_k <= score.size(1):
            fused = self._gate_with_indices(score, "topk", top_k=self.top_k)
            if fused is not None:
                return fused
            try:
                return c_router.route_scores(score, "topk", self.top_k, output="mask")[0]
            except NotImplementedError:  # more scores than one launch takes
                pass
        picks = torch.topk(score, self.top_k, dim=1).indices
        mask = torch.zeros(score.shape, dtype=torch.int32, device=score.device)
        return mask.scatter_(1, picks, 1)
