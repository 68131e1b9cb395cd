"""Fused fabrics (counterpart of python/brt/router/fabric/fused.py:18-123): all paths stay in
one tensor ordered by path; the route indices and loads travel on the GridTensor's stacks from
the scatter to the gather."""
from typing import List, Tuple, Union

import torch

from ..._C import router as c_router
from ...runtime.grid_tensor import GridTensor, init_grid_tensor, to_torch_tensor
from .base import register_fabric
from .generic import CombineFabric, DispatchFabric

__all__ = ["FusedDispatchFabric", "FusedCombineFabric"]


@register_fabric("fused_dispatch")
class FusedDispatchFabric(DispatchFabric):
    def __init__(self, flow_num: int, route_logic: Union[str, List[str]] = "1d",
                 transform: Union[bool, List[bool]] = False, **kwargs):
        kwargs["index_format"] = "seat_index"
        super().__init__(flow_num, route_logic=route_logic, transform=transform, **kwargs)

    def dispatch(self, in_flows: List[GridTensor], route_indices: torch.Tensor,
                 loads: torch.Tensor, score: torch.Tensor) -> Tuple[List[GridTensor], torch.Tensor]:
        all_out_flows = []
        for flow_idx, flow in enumerate(in_flows):
            data, tag_stack, load_stack, extra = to_torch_tensor(flow, retrieve_attr=True)
            flow_tag = tag_stack[-1]
            assert flow_tag is None
            (routed,) = self._route(data, route_indices, loads, score, flow_idx, flow_tag)
            all_out_flows.append(init_grid_tensor(
                routed, tag_stack[:-1] + [route_indices], load_stack[:-1] + [loads], extra))
        return all_out_flows, score


@register_fabric("fused_combine")
class FusedCombineFabric(CombineFabric):
    def __init__(self, flow_num, reduction="add", transform=False, **kwargs) -> None:
        kwargs["index_format"] = "seat_index"
        super().__init__(flow_num=flow_num, reduction=reduction, transform=transform, **kwargs)

    def combine(self, in_flows: List[GridTensor], residual_flows: List[GridTensor],
                score: torch.Tensor) -> List[GridTensor]:
        out_flows = []
        for flow_idx, flow in enumerate(in_flows):
            data, tag_stack, load_stack, extra = to_torch_tensor(flow, retrieve_attr=True)
            residual = residual_flows[flow_idx] if residual_flows is not None else None
            tag_stack, load_stack = list(tag_stack), list(load_stack)
            route_indices = tag_stack.pop()
            loads = load_stack.pop()
            (out,) = c_router.combine_with_indices_and_loads(
                data, route_indices, loads, score if self.transform else None, residual,
                max_path_padding=self.max_path_padding, ever_padded=self.ever_padded)
            out_flows.append(init_grid_tensor(out, tag_stack, load_stack, extra))
        return out_flows
