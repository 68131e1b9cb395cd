"""Python-level wrappers around the distributed operators
(counterpart of python/brt/runtime/distributed.py:22-202).

Every wrapper degrades to the identity when ``torch.distributed`` is not initialised, which
is how single-GPU code runs the expert-parallel fabrics.  On first use with a process group
the library's own NCCL communicator is created from a unique id broadcast through
``torch.distributed``.
"""
from typing import List

import torch
import torch.distributed as dist

from .._C import distributed as C_dist
from . import p2p


class global_info:
    initialized = False
    reorder_indices = None
    group = None
    world_size = None
    world_rank = None


def _is_initialized() -> bool:
    return global_info.initialized


def is_nccl_activated(group: dist.ProcessGroup = None) -> bool:
    if not dist.is_initialized():
        return False
    if not global_info.initialized:
        global_info.group = group or dist.group.WORLD
        global_info.world_size = dist.get_world_size(group)
        global_info.world_rank = dist.get_rank(group)
        unique_id = C_dist.make_nccl_unique_id(global_info.world_rank)
        dist.broadcast(unique_id, 0, global_info.group)
        C_dist.init_nccl(unique_id, global_info.world_rank, global_info.world_size)
        # NVLink peer arena for the packed exchange (all ranks or none; BRT_P2P=0 disables)
        p2p.setup(global_info.group, global_info.world_rank, global_info.world_size)
        global_info.initialized = True
    return True


def get_reorder_indices():
    return global_info.reorder_indices


def set_reorder_indices(reorder_indices: torch.Tensor):
    global_info.reorder_indices = reorder_indices


def exchange(in_data: torch.Tensor, reorder_indices: torch.Tensor):
    return C_dist.exchange(in_data, reorder_indices) if is_nccl_activated() else in_data


def batched_exchange(in_datas: List[torch.Tensor], reorder_indices: torch.Tensor):
    return C_dist.batched_exchange(in_datas, reorder_indices) if is_nccl_activated() \
        else in_datas


def reverse_exchange(in_data: torch.Tensor, reorder_indices: torch.Tensor):
    return C_dist.reverse_exchange(in_data, reorder_indices) if is_nccl_activated() else in_data


def batched_reverse_exchange(in_datas: List[torch.Tensor], reorder_indices: torch.Tensor):
    return C_dist.batched_reverse_exchange(in_datas, reorder_indices) if is_nccl_activated() \
        else in_datas


def asymmetry_a2a(in_data: torch.Tensor, in_loads: torch.Tensor, locality_aware: bool = False):
    if is_nccl_activated():
        return C_dist.asymmetry_all_to_all(in_data, in_loads, locality_aware)
    assert locality_aware is False
    return in_data, in_loads


def group_asymmetry_a2a(in_data: torch.Tensor, in_loads: torch.Tensor,
                        locality_aware: bool = False):
    if is_nccl_activated():
        return C_dist.group_asymmetry_all_to_all(in_data, in_loads, locality_aware)
    assert locality_aware is False
    return in_data, in_loads


def batched_group_asymmetry_a2a(in_datas: List[torch.Tensor], in_loads: torch.Tensor,
                                locality_aware: bool = False):
    if is_nccl_activated():
        outs, out_loads, reorder = C_dist.batched_group_asymmetry_all_to_all(
            in_datas, in_loads, locality_aware)
        return (outs, out_loads, reorder) if locality_aware else (outs, out_loads)
    assert locality_aware is False
    return in_datas, in_loads


def size_known_group_asymmetry_a2a(in_data: torch.Tensor, in_loads: torch.Tensor,
                                   out_loads: torch.Tensor):
    if is_nccl_activated():
        return C_dist.size_known_group_asymmetry_all_to_all(in_data, in_loads, out_loads)
    return in_data


def batched_size_known_group_asymmetry_a2a(in_datas: List[torch.Tensor], in_loads: torch.Tensor,
                                           out_loads: torch.Tensor):
    if is_nccl_activated():
        return C_dist.batched_size_known_group_asymmetry_all_to_all(in_datas, in_loads,
                                                                    out_loads)
    return in_datas


def group_sparse_a2a(in_data: torch.Tensor, in_loads: torch.Tensor, max_path_padding=False,
                     max_path_load=0):
    if is_nccl_activated():
        return C_dist.group_sparse_all_to_all(in_data, in_loads, max_path_padding, max_path_load)
    return in_data, in_loads, in_loads


def dispatch_group_sparse_a2a(in_data: torch.Tensor, route_indices: torch.Tensor,
                              loads: torch.Tensor, max_path_padding=False, max_path_load=0):
    """Unweighted dispatch + ``group_sparse_a2a`` as one kernel when the peer-memory transport
    can take it, else ``None`` (the caller runs the two steps)."""
    if is_nccl_activated():
        return C_dist.dispatch_group_sparse_all_to_all(in_data, route_indices, loads,
                                                       max_path_padding, max_path_load)
    return None


def group_sparse_a2a_device(in_data: torch.Tensor, in_loads: torch.Tensor,
                            max_path_padding=False, max_path_load=0):
    """``group_sparse_a2a`` whose size tensors stay on the device (no host synchronisation;
    fit for ``replayable_exchanges`` and CUDA graph capture)."""
    is_nccl_activated()
    return C_dist.group_sparse_all_to_all_device(in_data, in_loads, max_path_padding,
                                                 max_path_load)


def dispatch_group_sparse_a2a_device(in_data: torch.Tensor, route_indices: torch.Tensor,
                                     loads: torch.Tensor, max_path_padding=False,
                                     max_path_load=0):
    """``dispatch_group_sparse_a2a`` whose size tensors stay on the device."""
    is_nccl_activated()
    return C_dist.dispatch_group_sparse_all_to_all_device(in_data, route_indices, loads,
                                                          max_path_padding, max_path_load)


def combine_group_sparse_a2a(in_data: torch.Tensor, route_indices: torch.Tensor, gates,
                             in_loads: torch.Tensor, out_loads: torch.Tensor,
                             max_path_padding=False):
    """``size_known_group_sparse_a2a`` + weighted combine as one kernel that pulls the expert
    outputs over NVLink when the peer-memory transport can take it, else ``None`` (the caller
    runs the two steps)."""
    if is_nccl_activated():
        return C_dist.combine_group_sparse_all_to_all(in_data, route_indices, gates, in_loads,
                                                      out_loads, max_path_padding)
    return None


expert_output_buffer = C_dist.expert_output_buffer
replayable_exchanges = C_dist.replayable_exchanges


def size_known_group_sparse_a2a(in_data: torch.Tensor, in_loads: torch.Tensor,
                                out_loads: torch.Tensor, max_path_padding=False):
    if is_nccl_activated():
        return C_dist.size_known_group_sparse_all_to_all(in_data, in_loads, out_loads,
                                                         max_path_padding)
    return in_data
