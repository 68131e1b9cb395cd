"""Expert-parallel fabrics on the padded-slot exchange, with locality-aware and task-locality
variants (counterpart of python/brt/router/fabric/distributed_legacy.py:14-246, adapted to
the interface the current fabrics share; the reference file is written against an older one).

Dispatch: local fused dispatch into ``E`` slots of ``max_path_load`` rows, then
``group_asymmetry_all_to_all``: slot (i, j) of rank s lands in slot (s, j) of rank i.
Combine: ``size_known_group_asymmetry_all_to_all`` back into the same slots, then the local
combine.

``locality_aware``: the exchange also returns the greedy rank matching on the gathered load
matrix (``reorder_indices``).  The received rank-slices are permuted by it, and every rank
takes over the routing metadata (route indices, loads, score) of the rank it is matched with
(``batched_exchange``): on the way back the largest slice then stays on its rank, and the
combined cells of rank ``reorder_indices[k]`` come out on rank ``k``
(``brt_dist.get_reorder_indices()`` tells the caller).

``task_locality_aware`` (dispatch only): the useful rows of every local expert ("task") are
concatenated and handed back with the task id of each row in place of the score.
"""
from typing import List, Tuple, Union

import torch
import torch.distributed as dist

from ..._C import router as c_router
from ...runtime import distributed as brt_dist
from ...runtime.grid_tensor import GridTensor, init_grid_tensor, to_torch_tensor
from .base import register_fabric
from .distributed import DistributedFusedCombineFabric, DistributedFusedDispatchFabric
from .fused import FusedCombineFabric, FusedDispatchFabric

__all__ = ["DistributedSlotDispatchFabric", "DistributedSlotCombineFabric",
           "DistributedPlacementDispatchFabric", "DistributedPlacementCombineFabric"]


@register_fabric("distributed_slot_dispatch")
class DistributedSlotDispatchFabric(FusedDispatchFabric):
    def __init__(self, flow_num: int, capacity_padding=False,
                 route_logic: Union[str, List[str]] = "1d",
                 transform: Union[bool, List[bool]] = False, locality_aware: bool = False,
                 task_locality_aware: bool = False, **kwargs):
        self.locality_aware = locality_aware
        self.task_locality_aware = task_locality_aware
        kwargs["max_path_padding"] = True  # the exchange works on equal slots
        super().__init__(flow_num=flow_num, capacity_padding=capacity_padding,
                         route_logic=route_logic, transform=transform, **kwargs)

    def dispatch(self, in_flows: List[GridTensor], route_indices: torch.Tensor,
                 loads: torch.Tensor, score: torch.Tensor) -> Tuple[List[GridTensor], torch.Tensor]:
        if self.max_path_load <= 0:
            raise RuntimeError("the padded-slot fabric needs max_path_load (the slot size)")
        out_flows = []
        for flow_idx in range(self.flow_num):
            data, tag_stack, load_stack, extra = to_torch_tensor(in_flows[flow_idx],
                                                                 retrieve_attr=True)
            (routed,) = self._route(data, route_indices, loads, score, flow_idx, None)
            res = brt_dist.group_asymmetry_a2a(routed, loads, self.locality_aware)
            out, out_loads = res[0], res[1]
            m_indices, m_loads, m_score = route_indices, loads, score
            if self.locality_aware and dist.is_initialized():
                reorder = res[2]
                world = reorder.numel()
                out = out.reshape(world, -1).index_select(0, reorder.long()).reshape(out.shape)
                m_indices, m_loads, m_score = brt_dist.batched_exchange(
                    [route_indices, loads, score], reorder)
                brt_dist.set_reorder_indices(reorder)
            if self.task_locality_aware:
                world = dist.get_world_size() if dist.is_initialized() else 1
                rank = dist.get_rank() if dist.is_initialized() else 0
                tasks = out_loads.numel() // world
                cap = self.max_path_load
                counts = out_loads.reshape(world, tasks).cpu().tolist()
                parts, ids = [], []
                for j in range(tasks):
                    for i in range(world):
                        start = (i * tasks + j) * cap
                        parts.append(out[start:start + counts[i][j]])
                    ids.append(torch.full((sum(counts[i][j] for i in range(world)),),
                                          rank * tasks + j, dtype=torch.int64, device=out.device))
                out_flows.append(torch.cat(parts, dim=0))
                score = torch.cat(ids, dim=0)
                continue
            flow = init_grid_tensor(out, tag_stack, load_stack, extra)
            flow.pack(m_indices, out_loads, in_loads=m_loads, slot_score=m_score)
            out_flows.append(flow)
        return out_flows, score


@register_fabric("distributed_slot_combine")
class DistributedSlotCombineFabric(FusedCombineFabric):
    def __init__(self, flow_num, reduction="add", transform=False, locality_aware: bool = False,
                 **kwargs) -> None:
        self.locality_aware = locality_aware
        kwargs["max_path_padding"] = True
        super().__init__(flow_num=flow_num, reduction=reduction, transform=transform, **kwargs)

    def combine(self, in_flows: List[GridTensor], residual_flows: List[GridTensor],
                score: torch.Tensor) -> List[GridTensor]:
        out_flows = []
        for idx, flow in enumerate(in_flows):
            flow, route_indices, out_loads, popped = flow.unpack("in_loads", "slot_score")
            in_loads = popped["in_loads"]
            # with the locality matching this rank combines another rank's cells: the score
            # that travelled with the metadata is the one that belongs to them
            gates = popped["slot_score"] if popped["slot_score"] is not None else score
            data, tag_stack, load_stack, extra = to_torch_tensor(flow, retrieve_attr=True)
            residual = residual_flows[idx] if residual_flows is not None else None
            data = brt_dist.size_known_group_asymmetry_a2a(data, out_loads, in_loads)
            (out,) = c_router.combine_with_indices_and_loads(
                data, route_indices, in_loads, gates if self.transform else None, residual,
                max_path_padding=True, ever_padded=self.ever_padded)
            out_flows.append(init_grid_tensor(out, tag_stack, load_stack, extra))
        return out_flows


@register_fabric("distributed_placement_dispatch")
class DistributedPlacementDispatchFabric(DistributedFusedDispatchFabric):
    """The packed-bucket exchange under the name the placement experiments use
    (distributed_legacy.py:172-219); the experts' placement lives in the gate's row order
    (``brainstorm_b200.runtime.placement.reorder_gate_rows``), not in the fabric."""


@register_fabric("distributed_placement_combine")
class DistributedPlacementCombineFabric(DistributedFusedCombineFabric):
    """See ``DistributedPlacementDispatchFabric`` (distributed_legacy.py:222-246)."""
