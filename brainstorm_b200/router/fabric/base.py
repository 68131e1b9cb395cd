"""Fabric base class: a fabric moves cells according to a hot mask
(counterpart of python/brt/router/fabric/base.py).

Load/decision capture (used by the reference's offline placement search) is kept as an
opt-in feature controlled by the same environment variables: BRT_CAPTURE_STATS,
BRT_CAPTURE_MODE (avg|max|cum) and BRT_CAPTURED_FABRIC_TYPE.
"""
import os
from typing import Any, Callable, Dict, List

import numpy as np
import torch
import torch.nn as nn

from ..._C import router as c_router
from ...runtime import Registry
from ..utils import make_kwargs

__all__ = ["FabricBase", "register_fabric", "make_fabric", "switch_capture",
           "reset_router_stats"]


class FabricBase(nn.Module):
    def __init__(self, flow_num: int, index_format: str = None, **kwargs) -> None:
        super().__init__()
        self.flow_num = flow_num
        assert index_format in ("tag_index", "seat_index"), \
            f"index_format should be tag_index or seat_index, but got {index_format}"
        self.is_tag_index = index_format == "tag_index"
        if os.environ.get("BRT_CAPTURE_STATS", "False").lower() == "true":
            mode = os.environ.get("BRT_CAPTURE_MODE", "avg")
            assert mode in ("avg", "max", "cum"), f"Invalid capture mode: {mode}"
            self.enable_capture(mode=mode,
                                fabric_type=os.environ.get("BRT_CAPTURED_FABRIC_TYPE", "dispatch"))
        else:
            self.disable_capture()
        self.reset_flow_stats()

    def forward(self, *inputs: Any):
        raise NotImplementedError("FabricBase is an abstract class for Fabric")

    def check_compatibility(self, kwargs: Dict[str, Any]) -> None:
        pass

    # -- statistics ---------------------------------------------------------------------------
    def enable_capture(self, mode: str = "cum", fabric_type: str = "dispatch"):
        self.capturing = True
        self.capture_mode = mode
        self.captured_fabric_type = fabric_type.split(",") if isinstance(fabric_type, str) \
            else list(fabric_type)

    def disable_capture(self):
        self.capturing = False
        self.capture_mode = None
        self.captured_fabric_type = []

    def reset_flow_stats(self):
        self.history_len = 0
        self.cell_tag_base = 0
        self.load_history: np.ndarray = None
        self.cell_decision_history: List[np.ndarray] = None
        self.cell_grain_history: List[torch.Size] = None
        self.cell_dtype_history: List[torch.dtype] = None
        self.cell_device_history: List[torch.device] = None

    def copy_flow_stats_from(self, other: "FabricBase"):
        for name in ("history_len", "cell_tag_base", "load_history", "cell_decision_history",
                     "cell_grain_history", "cell_device_history"):
            setattr(self, name, getattr(other, name))

    def capture_flow_stats(self, in_flows, route_indices=None, loads=None):
        if not self.capturing:
            return
        kind = getattr(self, "brt_abs_type", "")
        wanted = ",".join(self.captured_fabric_type)
        if "dispatch" in kind and "dispatch" in wanted:
            self._capture_decisions(route_indices, loads)
            self._capture_cell_options(in_flows, is_dispatch=True)
            self._accumulate_load(loads.cpu().numpy().astype(np.float64))
        elif "combine" in kind and "combine" in wanted:
            if isinstance(in_flows, list) and len(in_flows) == 0:
                return
            self._capture_cell_options(in_flows, is_dispatch=False)
            flows = in_flows
            if all(isinstance(f, list) for f in flows):
                if not all(len(f) > 0 for f in flows):
                    return
                flows = flows[0]
            self._accumulate_load(np.array([f.size(0) for f in flows], dtype=np.float64))
        else:
            return
        self.history_len += 1

    def _accumulate_load(self, current: np.ndarray):
        if self.history_len == 0 or self.load_history is None:
            self.load_history = np.zeros_like(current, dtype=np.float64)
        if self.capture_mode == "avg":
            self.load_history = (self.load_history * self.history_len + current) / (
                self.history_len + 1.0)
        elif self.capture_mode == "max":
            self.load_history = np.maximum(self.load_history, current)
        elif self.capture_mode == "cum":
            self.load_history = self.load_history + current

    def _listing_flows(self, flows, is_dispatch=True):
        if is_dispatch:
            return [flows] if isinstance(flows, torch.Tensor) else flows
        if isinstance(flows, list) and flows and isinstance(flows[0], torch.Tensor):
            return [flows]
        return flows

    def _capture_cell_options(self, flows, is_dispatch=True):
        if self.cell_grain_history is not None:
            return
        flows = self._listing_flows(flows, is_dispatch)
        heads = flows if is_dispatch else [f[0] for f in flows]
        self.cell_grain_history = [h.shape for h in heads]
        self.cell_dtype_history = [h.dtype for h in heads]
        self.cell_device_history = [h.device for h in heads]

    def _capture_decisions(self, indices: torch.Tensor, loads: torch.Tensor):
        path_num = len(loads)
        tag_indices = indices
        if not self.is_tag_index:
            # flag semantics of the operator: False converts seat indices to tag indices
            tag_indices = c_router.convert_index_format(indices, loads, False)
        loads_host = loads.cpu().tolist()
        current = []
        for i in range(path_num):
            col = tag_indices[: int(loads_host[i]), i].cpu().numpy()
            current.append(col[col != 0] + self.cell_tag_base)
        if self.history_len == 0 or self.cell_decision_history is None:
            self.cell_decision_history = current
        else:
            self.cell_decision_history = [
                np.concatenate((old, new), axis=None)
                for old, new in zip(self.cell_decision_history, current)]
        for hist in self.cell_decision_history:
            if hist.size > 0:
                self.cell_tag_base = max(self.cell_tag_base, int(hist.max()))

    def check_cell_consistency(self, flows, is_dispatch=True) -> bool:
        if self.cell_grain_history is None:
            return self.history_len == 0
        heads = flows if is_dispatch else [f[0] for f in flows]
        for i, h in enumerate(heads):
            if (h.shape[1:] != self.cell_grain_history[i][1:]
                    or h.dtype != self.cell_dtype_history[i]
                    or h.device != self.cell_device_history[i]):
                return False
        return True


def register_fabric(fabric_type: str) -> Callable:
    return Registry.register_sub_cls(fabric_type, FabricBase)


def make_fabric(fabric_type: str, kwargs: Dict[str, Any]) -> FabricBase:
    fabric_cls = Registry.get_sub_cls(fabric_type, FabricBase)
    if fabric_cls is None:
        raise ValueError(f"Fabric type: {fabric_type} is not registered.")
    return fabric_cls(**make_kwargs(kwargs))


def switch_capture(m: nn.Module, capture=True, mode=None, fabric_type=None):
    for child in m.children():
        switch_capture(child, capture=capture, mode=mode, fabric_type=fabric_type)
    if isinstance(m, FabricBase):
        if capture:
            m.enable_capture(mode=mode or m.capture_mode or "cum",
                             fabric_type=fabric_type or ",".join(m.captured_fabric_type)
                             or "dispatch")
        else:
            m.disable_capture()
    return m


def reset_router_stats(m: nn.Module):
    for child in m.children():
        reset_router_stats(child)
    if isinstance(m, FabricBase):
        m.reset_flow_stats()
    return m
