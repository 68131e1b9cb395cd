"""Small helpers shared by routers, protocols and fabrics
(counterpart of python/brt/router/utils.py)."""
from typing import List

import torch

__all__ = ["pad_to_max", "make_kwargs", "empty_flows", "assert_compatibility"]


def pad_to_max(tensors: List[torch.Tensor], pad_value=0):
    """Right-pad the flattened cells of every tensor to the widest cell, keeping that cell's
    shape."""
    widths = [t.numel() // t.size(0) for t in tensors]
    widest = max(range(len(tensors)), key=widths.__getitem__)
    shape = tensors[widest].shape[1:]
    out = []
    for t, w in zip(tensors, widths):
        flat = t.reshape(t.size(0), -1)
        flat = torch.nn.functional.pad(flat, (0, widths[widest] - w), value=pad_value)
        out.append(flat.view(t.size(0), *shape))
    return out


def make_kwargs(kwargs):
    if kwargs is None:
        return {}
    if isinstance(kwargs, dict) and all(isinstance(k, str) for k in kwargs):
        return kwargs
    raise ValueError(f"kwargs should be a dict of str to Any, but got {kwargs}")


def empty_flows(in_flows) -> bool:
    if isinstance(in_flows, list):
        return len(in_flows) == 0 or empty_flows(in_flows[0])
    return False


def assert_compatibility(instance, k, expected_v, given_v) -> None:
    assert expected_v == given_v, (
        f"compatibility check failed for {type(instance).__name__}, caused by keyword argument "
        f"{k}: expected {expected_v}, given {given_v}")
