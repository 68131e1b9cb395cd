"""Per-path dispatch and combine fabrics (counterpart of
python/brt/router/fabric/generic.py:17-313).

``DispatchFabric`` turns a hot mask into seat indices and loads, dispatches every flow with
one fused kernel launch and hands back one GridTensor view per path.  With the default
``index_format="tag_index"`` the dispatch also emits, for every output row, the tag of the cell
it came from; ``CombineFabric`` then merges the paths by tag (sum of the rows that share a
tag).  With ``index_format="seat_index"`` the route indices themselves ride on the tag stack.
"""
from typing import List, Tuple, Union

import torch

from ..._C import router as c_router
from ...runtime.grid_tensor import GridTensor, init_grid_tensor, to_torch_tensor
from .base import FabricBase, register_fabric

__all__ = ["DispatchFabric", "CombineFabric"]


def _per_flow(value, flow_num, kind, allowed=None):
    values = [value] * flow_num if isinstance(value, kind) else value
    assert isinstance(values, list) and len(values) == flow_num
    assert all(isinstance(v, kind) and (allowed is None or v in allowed) for v in values)
    return values


@register_fabric("dispatch")
class DispatchFabric(FabricBase):
    def __init__(self, flow_num: int, route_logic: Union[str, List[str]] = "1d",
                 transform: Union[bool, List[bool]] = False, **kwargs):
        """route_logic: "1d" (route whole cells) or "2d" (path e takes element e of a cell), per
        flow; transform: scale routed cells by the score, per flow.  Other kwargs:
        index_format, supported_capacities, capacity_padding, path_wise_padding,
        max_path_padding, max_path_load."""
        index_format = kwargs.pop("index_format", "tag_index")
        supported_capacities = kwargs.pop("supported_capacities", None)
        self_capacity_padding = kwargs.pop("capacity_padding", False)
        path_wise_padding = kwargs.pop("path_wise_padding", False)
        max_path_padding = kwargs.pop("max_path_padding", False)
        max_path_load = kwargs.pop("max_path_load", 0)
        super().__init__(flow_num=flow_num, index_format=index_format, **kwargs)
        self.route_logics = _per_flow(route_logic, flow_num, str, ("1d", "2d"))
        self.transforms = _per_flow(transform, flow_num, bool)
        self.capacity_padding = self_capacity_padding
        if supported_capacities is not None:
            if isinstance(supported_capacities, int):
                supported_capacities = [supported_capacities]
            assert isinstance(supported_capacities, list) and all(
                isinstance(c, int) for c in supported_capacities)
            self.register_buffer("supported_capacities",
                                 torch.tensor(supported_capacities, dtype=torch.int32))
            self.path_wise_padding = path_wise_padding
        else:
            self.register_buffer("supported_capacities", None)
            self.path_wise_padding = False
        self.max_path_padding = max_path_padding
        self.max_path_load = max_path_load

    def forward(self, in_flow, hot_mask: torch.Tensor, runtime_capacities: torch.Tensor = None,
                score: torch.Tensor = None):
        capacities = runtime_capacities if runtime_capacities is not None \
            else self.supported_capacities
        routes = getattr(hot_mask, "_brt_routes", None)
        if routes is not None and routes[2] is capacities and \
                routes[3:] == (self.capacity_padding, self.path_wise_padding):
            # the gate kernel that made this mask already scanned it under the same rules
            route_indices, loads = routes[0], routes[1]
        else:
            route_indices, loads = c_router.generate_indices_and_loads(
                hot_mask, supported_capacities=capacities,
                capacity_padding=self.capacity_padding,
                path_wise_padding=self.path_wise_padding, is_tag_index=False)
        in_flows = [in_flow] if self.flow_num == 1 else in_flow
        self.capture_flow_stats(in_flows, route_indices, loads)
        all_out_flows, score = self.dispatch(in_flows, route_indices, loads, score)
        if self.flow_num == 1:
            all_out_flows = all_out_flows[0]
        return all_out_flows, score

    def _route(self, flow_data, route_indices, loads, score, flow_idx, flow_tag):
        # positional layout of the operator: (data, indices, loads, gates, tag_generating, tags,
        # max_path_padding, max_path_load, is_1d_routing)
        return c_router.dispatch_with_indices_and_loads(
            flow_data, route_indices, loads, score if self.transforms[flow_idx] else None,
            self.is_tag_index, flow_tag, self.max_path_padding, self.max_path_load,
            self.route_logics[flow_idx] == "1d")

    def dispatch(self, in_flows: List[GridTensor], route_indices: torch.Tensor,
                 loads: torch.Tensor, score: torch.Tensor
                 ) -> Tuple[List[List[GridTensor]], torch.Tensor]:
        all_out_flows = []
        path_num = route_indices.size(1)
        for flow_idx in range(self.flow_num):
            data, tag_stack, load_stack, extra = to_torch_tensor(in_flows[flow_idx],
                                                                 retrieve_attr=True)
            flow_tag = tag_stack[-1]
            tag_stack, load_stack = tag_stack[:-1], load_stack[:-1]
            routed = self._route(data, route_indices, loads, score, flow_idx, flow_tag)
            if self.is_tag_index:
                routed_data, routed_tags = routed
                datas, split_loads, split_tags = c_router.split_fused_cells_to_paths(
                    routed_data, loads, self.max_path_padding, is_load_split=True,
                    is_tag_split=True, tags=routed_tags)
                out_flows = [
                    init_grid_tensor(datas[i], tag_stack + [split_tags[i]],
                                     load_stack + [split_loads[i]], extra)
                    for i in range(path_num)]
            else:
                (datas,) = c_router.split_fused_cells_to_paths(
                    routed[0], loads, self.max_path_padding, is_load_split=False,
                    is_tag_split=False)
                out_flows = [
                    init_grid_tensor(datas[i], tag_stack + [route_indices], load_stack + [loads],
                                     extra)
                    for i in range(path_num)]
            all_out_flows.append(out_flows)
        return all_out_flows, score


@register_fabric("combine")
class CombineFabric(FabricBase):
    def __init__(self, flow_num: int, reduction="add", transform=False, **kwargs):
        index_format = kwargs.pop("index_format", "tag_index")
        max_path_padding = kwargs.pop("max_path_padding", False)
        ever_padded = kwargs.pop("ever_padded", False)
        super().__init__(flow_num=flow_num, index_format=index_format, **kwargs)
        self.max_path_padding = max_path_padding
        self.ever_padded = ever_padded or max_path_padding
        self.reduction = reduction
        self.transform = transform

    def forward(self, in_flows, residual_flows=None, score: torch.Tensor = None):
        if self.flow_num == 1:
            in_flows = [in_flows]
            residual_flows = [residual_flows] if residual_flows is not None else None
        self.capture_flow_stats(in_flows)
        out_flows = self.combine(in_flows, residual_flows, score)
        return out_flows[0] if self.flow_num == 1 else out_flows

    def combine(self, in_flows: List[List[GridTensor]], residual_flows: List[GridTensor],
                score: torch.Tensor) -> List[GridTensor]:
        out_flows = []
        for flow_idx in range(self.flow_num):
            residual = residual_flows[flow_idx] if residual_flows is not None else None
            datas, tags, loads = [], [], []
            tag_stack = load_stack = extra = None
            for flow in in_flows[flow_idx]:
                data, tag_stack, load_stack, extra = to_torch_tensor(flow, retrieve_attr=True)
                datas.append(data)
                tags.append(tag_stack[-1])
                loads.append(load_stack[-1])
            if len(datas) == 1 and tags[0] is None:
                # a single un-routed flow passes through with fresh tags
                data = datas[0]
                tag_stack[-1] = torch.arange(1, data.shape[0] + 1, dtype=torch.int32,
                                             device=data.device)
                load_stack[-1] = torch.tensor([data.shape[0]], dtype=torch.int32,
                                              device=data.device)
                out_flows.append(init_grid_tensor(data, tag_stack, load_stack, extra))
                continue
            if self.is_tag_index:
                fused, fused_tags, route_indices = c_router.fuse_split_cells_from_paths(
                    datas, is_tag_fuse=True, loads=loads, tags=tags)
                fused_loads = None
            else:
                (fused,) = c_router.fuse_split_cells_from_paths(datas)
                fused_loads, route_indices, fused_tags = loads[0], tags[0], None
            result = c_router.combine_with_indices_and_loads(
                fused, route_indices, fused_loads, score if self.transform else None, residual,
                max_path_padding=self.max_path_padding, ever_padded=self.ever_padded,
                is_tag_index=self.is_tag_index, tags=fused_tags)
            if self.is_tag_index:
                out_data, out_tag, out_load = result
            else:
                (out_data,), out_tag, out_load = result, None, None
            out = init_grid_tensor(out_data, tag_stack[:-1], load_stack[:-1], extra)
            out_flows.append(out.pack(out_tag, out_load))
        return out_flows
