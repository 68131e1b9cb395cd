"""Annotator: turns a tensor into a GridTensor whose leading dimension enumerates cells
(counterpart of python/brt/runtime/annotate.py:11-43)."""
from typing import List, Optional

import torch
import torch.nn as nn

from .grid_tensor import GridTensor, init_grid_tensor


class Annotator(nn.Module):
    def __init__(self, dims: List[int], cell_shape: Optional[List[int]] = None,
                 gridding: bool = True):
        super().__init__()
        assert isinstance(dims, list)
        self.dims = sorted(dims)
        assert cell_shape is None or isinstance(cell_shape, list)
        self.cell_shape = cell_shape
        self.gridding = gridding

    def forward(self, t: torch.Tensor):
        assert self.dims[-1] < t.dim()
        rest = [i for i in range(t.dim()) if i not in self.dims]
        cell_shape = self.cell_shape if self.cell_shape is not None else [t.shape[i] for i in rest]
        cells = t.permute(*self.dims, *rest).contiguous().reshape(-1, *cell_shape)
        if not self.gridding:
            return cells
        if isinstance(cells, GridTensor):
            return cells.pack(None, None)
        return init_grid_tensor(cells, [None], [None])
