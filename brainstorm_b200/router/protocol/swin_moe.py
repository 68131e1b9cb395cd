"""Swin-MoE gate protocol (python/brt/router/protocol/swin_moe.py:47-144,193-204).

``make_route_decision`` keeps the reference's behaviour: the hot mask holds the *first* of the
top-k picks of every cell, throttled to ``top_k * int(capacity_factor * ceil(T / E))`` cells per
path, optionally in order of decreasing best score (batch-prioritised routing).
``renormalised_topk_score`` is the gate renormalisation of the reference's legacy decision
path, exposed on its own because benchmarks use it to build combine weights.
"""
import torch
import torch.distributed as dist

from ..._C import router as c_router
from .base import ProtocolBase, register_protocol

__all__ = ["SwinMoEProtocol", "process_mask", "renormalised_topk_score", "topk_hot_mask"]


def process_mask(hot_mask, prefix_base, capacity, score_sorted=False, score=None):
    """Throttle ``hot_mask`` to ``capacity`` cells per path on top of ``prefix_base``."""
    if not score_sorted:
        return c_router.throttle_hotmask(hot_mask, prefix_base, capacity)
    order = (-score.max(dim=1).values).argsort(dim=0)
    throttled, prefix_base = c_router.throttle_hotmask(hot_mask[order].contiguous(), prefix_base,
                                                       capacity)
    return throttled[order.argsort(dim=0)], prefix_base


def topk_hot_mask(score: torch.Tensor, top_k: int) -> torch.Tensor:
    if c_router.route_scores_supported(score) and 1 <= top_k <= score.size(1):
        try:
            return c_router.route_scores(score, "topk", top_k, output="mask")[0]
        except NotImplementedError:
            pass
    picks = torch.topk(score, top_k, dim=1).indices
    return torch.zeros(score.shape, dtype=torch.int32, device=score.device).scatter_(1, picks, 1)


def renormalised_topk_score(score: torch.Tensor, top_k: int) -> torch.Tensor:
    """Scores of the top-k paths divided by their sum (clamped at eps), zero elsewhere."""
    if c_router.route_scores_supported(score) and 1 <= top_k <= score.size(1):
        try:
            return c_router.route_scores(score, "topk", top_k, output="mask", with_gates=True)[2]
        except NotImplementedError:
            pass
    vals, picks = torch.topk(score, top_k, dim=1)
    denom = torch.clamp(vals.sum(dim=1, keepdim=True), min=torch.finfo(score.dtype).eps)
    return torch.zeros_like(score).scatter_(1, picks, vals / denom)


@register_protocol("swin_moe")
class SwinMoEProtocol(ProtocolBase):
    def __init__(self, top_k=2, capacity_factor=0, gate_noise=0.0, group: dist.group = None,
                 is_postscore=True, batch_prioritized_routing=False, normalize_gate=True,
                 is_gshard_loss=True, alignment=1, **kwargs):
        super().__init__(**kwargs)
        self.top_k = top_k
        self.capacity_factor = capacity_factor
        self.gate_noise = gate_noise
        self.group = group
        self.is_postscore = is_postscore
        self.batch_prioritized_routing = batch_prioritized_routing
        self.normalize_gate = normalize_gate
        self.is_gshard_loss = is_gshard_loss
        self.alignment = alignment
        # (capacity_padding, path_wise_padding) of the dispatch fabric that follows, set by the
        # router that owns both: the gate kernel then hands the fabric its seat indices and
        # loads along with the hot mask, and the fabric skips its own index scan
        self.index_rules = None

    def runtime_capacity(self, cell_num: int, path_num: int) -> int:
        if self.capacity_factor <= 0:
            raise NotImplementedError("capacity_factor must be greater than 0")
        per_path = (int(cell_num) + path_num - 1) // path_num
        return self.top_k * int(self.capacity_factor * per_path)

    def make_route_decision(self, score, logits_wo_noise=None, logits=None):
        T, E = score.shape
        if not self.batch_prioritized_routing and c_router.route_scores_supported(score):
            # first pick and throttle in one launch of the library's gate kernel
            cap = self.runtime_capacity(T, E)
            runtime_capacities = torch.full((E,), cap, dtype=torch.int32, device=score.device)
            prefix = torch.zeros((E,), dtype=torch.int32, device=score.device)
            try:
                if self.index_rules is not None:
                    # gate, throttle and index scan in one launch; the mask comes with it
                    cpad, pwise = self.index_rules
                    indices, loads, _, hot_mask = c_router.route_scores(
                        score, "topk", 1, output="throttled_seat_indices", prefix=prefix,
                        throttle_capacity=runtime_capacities,
                        supported_capacities=runtime_capacities, capacity_padding=cpad,
                        path_wise_padding=pwise, with_mask=True)
                    hot_mask._brt_routes = (indices, loads, runtime_capacities, cpad, pwise)
                else:
                    hot_mask, _ = c_router.route_scores(score, "topk", 1,
                                                        output="throttled_mask", prefix=prefix,
                                                        throttle_capacity=runtime_capacities)
                loss = self.generate_auxiliary(score, logits_wo_noise, logits, None)
                return hot_mask, runtime_capacities, score, loss
            except NotImplementedError:
                pass
        first_pick = torch.topk(score, self.top_k, dim=1).indices[:, :1]
        hot_mask = torch.zeros((T, E), dtype=torch.int32, device=score.device)
        hot_mask.scatter_(1, first_pick, 1)
        cap = self.runtime_capacity(T, E)
        runtime_capacities = torch.full((E,), cap, dtype=torch.int32, device=score.device)
        prefix = torch.zeros((E,), dtype=torch.int32, device=score.device)
        hot_mask, _ = process_mask(hot_mask, prefix, runtime_capacities,
                                   self.batch_prioritized_routing, score)
        loss = self.generate_auxiliary(score, logits_wo_noise, logits, None)
        return hot_mask, runtime_capacities, score, loss

    def generate_auxiliary(self, score, logits_wo_noise, logits, topk_ids):
        return None
