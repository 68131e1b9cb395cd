"""Threshold protocols (python/brt/router/protocol/threshold.py:14-94)."""
import torch

from ..._C import router as c_router
from .base import ProtocolBase, register_protocol

__all__ = ["ThresholdProtocol", "ResidualThresholdProtocol", "BinaryThresholdProtocol"]


@register_protocol("threshold")
class ThresholdProtocol(ProtocolBase):
    """A cell goes to every path whose score exceeds ``threshold``; with ``residual_path >= 0``
    cells that would go nowhere are sent to that path."""

    def __init__(self, threshold: float = 0.0, residual_path: int = -1, **kwargs):
        super().__init__(**kwargs)
        self.threshold = threshold
        self.residual_path = residual_path

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        if c_router.route_scores_supported(score) and self.residual_path < score.size(1):
            fused = self._gate_with_indices(score, "threshold", threshold=self.threshold,
                                            residual_path=self.residual_path)
            if fused is not None:
                return fused
            try:  # the library's single-launch gate
                return c_router.route_scores(score, "threshold", threshold=self.threshold,
                                             residual_path=self.residual_path, output="mask")[0]
            except NotImplementedError:
                pass
        mask = (score > self.threshold).to(torch.int32)
        if self.residual_path >= 0:
            nowhere = (mask.sum(dim=1) == 0).to(torch.int32)
            mask[:, self.residual_path] += nowhere
        return mask


@register_protocol("residual_threshold")
class ResidualThresholdProtocol(ProtocolBase):
    """Two paths; cells whose scores sum below ``threshold`` take ``residual_path``."""

    def __init__(self, threshold: float = 0.0, residual_path: int = 0, **kwargs):
        super().__init__(**kwargs)
        if residual_path not in (0, 1):
            raise ValueError("residual_path should be 0 or 1")
        self.threshold = threshold
        self.residual_path = residual_path

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        low = (score.sum(dim=1, keepdim=True) < self.threshold).to(torch.int64)
        if self.residual_path == 0:
            base = torch.ones((score.size(0), 2), dtype=torch.int32, device=score.device)
            return base.scatter_(1, low, 0)
        base = torch.zeros((score.size(0), 2), dtype=torch.int32, device=score.device)
        return base.scatter_(1, low, 1)


@register_protocol("binary_threshold")
class BinaryThresholdProtocol(ProtocolBase):
    """Two paths; decided by whether the largest softmax probability reaches ``threshold``."""

    def __init__(self, threshold: float = 0.0, selected_path: int = 0, **kwargs):
        super().__init__(**kwargs)
        if selected_path not in (0, 1):
            raise ValueError("selected_path should be 0 or 1 for a binary threshold protocol")
        self.threshold = threshold
        self.selected_path = selected_path

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        confident = (torch.softmax(score, dim=1).max(dim=1).values >= self.threshold)
        confident = confident.long().unsqueeze(-1)
        if self.selected_path == 0:
            base = torch.ones((score.size(0), 2), dtype=torch.int32, device=score.device)
            return base.scatter_(1, confident, 0)
        base = torch.zeros((score.size(0), 2), dtype=torch.int32, device=score.device)
        return base.scatter_(1, confident, 1)
