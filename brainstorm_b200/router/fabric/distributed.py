"""Expert-parallel fused fabrics (counterpart of python/brt/router/fabric/distributed.py:14-158).

Dispatch: local fused dispatch in global-expert order, then the packed variable-size
all-to-all that regroups rows as [local expert][source rank].  Combine: the inverse exchange,
then the local weighted combine.  Without an initialised process group both exchanges are the
identity, which is how single-GPU runs use these fabrics.

``device_sizes=True`` (dispatch fabric; not in the reference) keeps the exchange's size tensors
on the device: no host synchronisation, so a layer built from these fabrics can be captured in
a CUDA graph inside ``brt_dist.replayable_exchanges()``.  The flow the experts get is then the
whole landing half seen as rows, of which the first ``loads.sum()`` are theirs, and ``loads``
is a device tensor.  Peer-memory transport only.
"""
import os
from typing import List, Tuple, Union

import torch
import torch.distributed as dist

from ..._C import router as c_router
from ...runtime import distributed as brt_dist
from ...runtime.grid_tensor import GridTensor, init_grid_tensor, to_torch_tensor
from .base import register_fabric
from .fused import FusedCombineFabric, FusedDispatchFabric

__all__ = ["DistributedFusedDispatchFabric", "DistributedFusedCombineFabric"]


@register_fabric("distributed_fused_dispatch")
class DistributedFusedDispatchFabric(FusedDispatchFabric):
    def __init__(self, flow_num: int, capacity_padding=False,
                 route_logic: Union[str, List[str]] = "1d",
                 transform: Union[bool, List[bool]] = False, task_locality: bool = False,
                 device_sizes: bool = False, **kwargs):
        self.task_locality = task_locality
        self.device_sizes = device_sizes
        if device_sizes and task_locality:
            raise ValueError("task_locality needs the sizes on the host")
        super().__init__(flow_num=flow_num, capacity_padding=capacity_padding,
                         route_logic=route_logic, transform=transform, **kwargs)

    def dispatch(self, in_flows: List[GridTensor], route_indices: torch.Tensor,
                 loads: torch.Tensor, score: torch.Tensor) -> Tuple[List[GridTensor], torch.Tensor]:
        all_out_flows = []
        for flow_idx in range(self.flow_num):
            data, tag_stack, load_stack, extra = to_torch_tensor(in_flows[flow_idx],
                                                                 retrieve_attr=True)
            fused = None
            plain = not self.transforms[flow_idx] and self.route_logics[flow_idx] == "1d"
            if self.device_sizes and dist.is_initialized():
                if plain and getattr(route_indices, c_router._DENSE, None) is not None:
                    fused = brt_dist.dispatch_group_sparse_a2a_device(
                        data, route_indices, loads, self.max_path_padding, self.max_path_load)
                else:
                    (routed,) = self._route(data, route_indices, loads, score, flow_idx, None)
                    fused = brt_dist.group_sparse_a2a_device(
                        routed, loads, self.max_path_padding, self.max_path_load)
            elif plain:
                # dispatch and exchange as one kernel over peer memory when that is possible
                fused = brt_dist.dispatch_group_sparse_a2a(
                    data, route_indices, loads, self.max_path_padding, self.max_path_load)
            if fused is not None:
                out_data, out_loads, in_loads = fused
            else:
                (routed,) = self._route(data, route_indices, loads, score, flow_idx, None)
                out_data, out_loads, in_loads = brt_dist.group_sparse_a2a(
                    routed, loads, self.max_path_padding, self.max_path_load)
            if self.task_locality:
                # hand back, per received row, the global id of the local expert ("task") it
                # belongs to, in place of the score
                world_size = dist.get_world_size() if dist.is_initialized() else 1
                world_rank = dist.get_rank() if dist.is_initialized() else 0
                local_tasks = out_loads.numel() // world_size
                per_task = out_loads.reshape(local_tasks, world_size).sum(dim=1).to(
                    out_data.device)
                ids = torch.arange(local_tasks, device=out_data.device) + world_rank * local_tasks
                score = torch.repeat_interleave(ids, per_task.to(torch.int64),
                                                output_size=out_data.size(0))
                all_out_flows.append(out_data)
                continue
            out_flow = init_grid_tensor(out_data, tag_stack, load_stack, extra)
            out_flow.pack(route_indices, out_loads, in_loads=in_loads)
            all_out_flows.append(out_flow)
        return all_out_flows, score


@register_fabric("distributed_fused_combine")
class DistributedFusedCombineFabric(FusedCombineFabric):
    def __init__(self, flow_num, reduction="add", transform=False, task_locality: bool = False,
                 pull_combine: bool = None, **kwargs) -> None:
        self.task_locality = task_locality
        # Inverse exchange and combine as ONE kernel that pulls the expert outputs from the
        # peers (not in the reference).  Off by default: on the NVLink boxes it was measured
        # on, the two kernels (rows pushed back, then combined locally) finish a little sooner.
        self.pull_combine = (os.environ.get("BRT_P2P_PULL_COMBINE", "0") == "1"
                             if pull_combine is None else bool(pull_combine))
        super().__init__(flow_num=flow_num, reduction=reduction, transform=transform, **kwargs)

    def combine(self, in_flows: List[GridTensor], residual_flows: List[GridTensor],
                score: torch.Tensor) -> List[GridTensor]:
        out_flows = []
        for idx, flow in enumerate(in_flows):
            flow, route_indices, in_loads, popped = flow.unpack("in_loads")
            out_loads = popped["in_loads"]
            data, tag_stack, load_stack, extra = to_torch_tensor(flow, retrieve_attr=True)
            residual = residual_flows[idx] if residual_flows is not None else None
            out = None
            if residual is None and self.pull_combine:
                # expert outputs that still sit in the arena (experts that work in place, or
                # that wrote into brt_dist.expert_output_buffer) are pulled by the combine
                # itself: inverse exchange and combine as one kernel
                out = brt_dist.combine_group_sparse_a2a(
                    data, route_indices, score if self.transform else None, in_loads,
                    out_loads, self.max_path_padding)
            if out is None:
                data = brt_dist.size_known_group_sparse_a2a(data, in_loads, out_loads,
                                                            self.max_path_padding)
                (out,) = c_router.combine_with_indices_and_loads(
                    data, route_indices, out_loads, score if self.transform else None, residual,
                    max_path_padding=self.max_path_padding, ever_padded=self.ever_padded)
            out_flows.append(init_grid_tensor(out, tag_stack, load_stack, extra))
        return out_flows
