"""Switch top-1 protocol (python/brt/router/protocol/switch.py:13-33): the gate already produced a
(capacity-masked) one-hot matrix; the protocol only flattens and casts it."""
import torch

from .base import ProtocolBase, register_protocol

from ..._C import router as c_router

__all__ = ["SwitchTop1Protocol", "switch_top1_capacity_mask"]


def switch_top1_capacity_mask(router_probs: torch.Tensor, expert_capacity: int) -> torch.Tensor:
    """The capacity-masked one-hot matrix a Switch gate hands to this protocol
    (benchmark/switch_moe/switch_transformer.py:240-254 in the reference: argmax -> one-hot ->
    cumsum over the tokens of a group -> ``<= expert_capacity``), from the gate kernel in one
    launch per group: a top-1 decision throttled at ``expert_capacity``.  ``router_probs`` is
    ``[tokens, experts]`` or ``[groups, tokens, experts]``; the result has its shape, int32.
    Equal probabilities go to the lower expert index, as ``torch.argmax`` does."""
    probs = router_probs if router_probs.dim() == 3 else router_probs.unsqueeze(0)
    E = probs.size(-1)
    out = []
    for group in probs:
        g = group.float().contiguous()
        if c_router.route_scores_supported(g):
            cap = torch.full((E,), int(expert_capacity), dtype=torch.int32, device=g.device)
            try:
                mask, _ = c_router.route_scores(
                    g, "topk", 1, output="throttled_mask",
                    prefix=torch.zeros((E,), dtype=torch.int32, device=g.device),
                    throttle_capacity=cap)
                out.append(mask)
                continue
            except NotImplementedError:
                pass
        one_hot = torch.nn.functional.one_hot(torch.argmax(g, dim=-1), num_classes=E)
        out.append((one_hot * (torch.cumsum(one_hot, dim=-2) <= expert_capacity)).to(torch.int32))
    mask = torch.stack(out)
    return mask if router_probs.dim() == 3 else mask[0]


@register_protocol("switch_top1")
class SwitchTop1Protocol(ProtocolBase):
    def __init__(self):
        super().__init__()

    def make_route_decision(self, score: torch.Tensor) -> torch.Tensor:
        return score.reshape(-1, score.shape[-1]).to(torch.int32)

    def update(self, supported_capacities):
        self.supported_capacities = supported_capacities
