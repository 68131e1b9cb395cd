"""GridTensor: a tensor that carries routing metadata between scatter and gather.

Counterpart of python/brt/runtime/grid_tensor.py:87-334 in the reference.  A GridTensor holds
two parallel stacks — tags (which source cell each row came from, or the route indices for
fused fabrics) and loads (rows per path) — plus a dict of extra attributes.  Results of torch
functions applied to a GridTensor inherit the stacks of the first GridTensor argument.
"""
import copy
from typing import Any, Dict, List, Optional, Tuple

import torch

__all__ = [
    "GridTensor", "init_grid_tensor", "init_grid_tensor_from", "deinit_grid_tensor",
    "to_grid_tensor", "to_torch_tensor", "collect_cell_attr", "attach_cell_attr",
]

_TAGS, _LOADS, _EXTRA = "cell_tag_stack", "cell_load_stack", "cell_extra_attr_dict"


def collect_cell_attr(args):
    """Stacks of the first GridTensor found in (possibly nested) ``args``; ``(None, None, None)``
    when there is none."""
    if isinstance(args, GridTensor):
        return args.tag_stack, args.load_stack, args.extra_attr_dict
    if isinstance(args, (tuple, list)):
        for a in args:
            tags, loads, extra = collect_cell_attr(a)
            if tags is not None and loads is not None:
                return tags, loads, extra
    return None, None, None


def attach_cell_attr(ret, tag_stack, load_stack, extra_attr_dict=None):
    if isinstance(ret, GridTensor):
        ret.deep_pack(tag_stack, load_stack, **(extra_attr_dict or {}))
    elif isinstance(ret, (tuple, list)):
        for r in ret:
            attach_cell_attr(r, tag_stack, load_stack, extra_attr_dict)
    return ret


class GridTensor(torch.Tensor):
    SHALLOW_TRANSPORT = True
    CHECK_TAGS = False

    # -- storage of the three attributes ------------------------------------------------------
    @property
    def cell_initilized(self) -> bool:  # (sic) spelling kept from the reference API
        d = self.__dict__
        return _TAGS in d and _LOADS in d and _EXTRA in d

    def init_cell(self):
        if not self.cell_initilized:
            self.__dict__[_TAGS] = []
            self.__dict__[_LOADS] = []
            self.__dict__[_EXTRA] = {}

    def _carry(self, value):
        return value if GridTensor.SHALLOW_TRANSPORT else copy.copy(value)

    @property
    def tag_stack(self) -> List[Optional[torch.Tensor]]:
        return self.__dict__[_TAGS]

    @tag_stack.setter
    def tag_stack(self, value):
        self.__dict__[_TAGS] = self._carry(value)

    @property
    def load_stack(self) -> List[Optional[torch.Tensor]]:
        return self.__dict__[_LOADS]

    @load_stack.setter
    def load_stack(self, value):
        self.__dict__[_LOADS] = self._carry(value)

    @property
    def extra_attr_dict(self) -> Dict[str, Any]:
        return self.__dict__[_EXTRA]

    @extra_attr_dict.setter
    def extra_attr_dict(self, value):
        self.__dict__[_EXTRA] = self._carry(value)

    @property
    def tag(self):
        return self.tag_stack[-1]

    @tag.setter
    def tag(self, value):
        self.tag_stack[-1] = value

    @property
    def load(self):
        return self.load_stack[-1]

    @load.setter
    def load(self, value):
        self.load_stack[-1] = value

    def set_extra_attr(self, key, value):
        assert key in self.extra_attr_dict
        self.extra_attr_dict[key] = self._carry(value)

    def get_extra_attr(self, key):
        assert key in self.extra_attr_dict
        return self.extra_attr_dict[key]

    @property
    def stack_size(self) -> int:
        return len(self.tag_stack)

    def annotation_empty(self) -> bool:
        return not self.tag_stack or not self.load_stack

    # -- push / pop ---------------------------------------------------------------------------
    def pack(self, tag, load, **extra):
        self.init_cell()
        self.tag_stack.append(tag)
        self.load_stack.append(load)
        for k, v in extra.items():
            assert k not in self.extra_attr_dict
            self.extra_attr_dict[k] = v
        return self

    def unpack(self, *extra_keys):
        assert self.cell_initilized and not self.annotation_empty()
        tag = self.tag_stack.pop()
        load = self.load_stack.pop()
        popped = {}
        for k in extra_keys:
            assert k in self.extra_attr_dict
            popped[k] = self.extra_attr_dict.pop(k)
        return self, tag, load, popped

    def deep_pack(self, tag_stack, load_stack, **extra):
        assert isinstance(tag_stack, list) and isinstance(load_stack, list), \
            "tag_stack and load_stack must be list for deep_pack"
        self.tag_stack = tag_stack
        self.load_stack = load_stack
        self.extra_attr_dict = {}
        for k, v in extra.items():
            self.extra_attr_dict[k] = v
        return self

    def deep_unpack(self):
        assert self.cell_initilized
        tags, loads, extra = self.tag_stack, self.load_stack, self.extra_attr_dict
        self.tag_stack, self.load_stack, self.extra_attr_dict = [], [], {}
        return self, tags, loads, extra

    def copy_cell_attr(self):
        assert self.cell_initilized
        return (self, self._carry(self.tag_stack), self._carry(self.load_stack),
                self._carry(self.extra_attr_dict))

    def __repr__(self):
        return (f"{super().__repr__()}\ntag_stack: {self.tag_stack}\n"
                f"load stack: {self.load_stack}\nextra_attr_dict: {self.extra_attr_dict}")

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        tags, loads, extra = collect_cell_attr(args)
        ret = super().__torch_function__(func, types, args, kwargs or {})
        if tags is not None and loads is not None:
            attach_cell_attr(ret, tags, loads, extra)
        return ret


def init_grid_tensor(tensor: torch.Tensor, tag_stack=None, load_stack=None,
                     extra_attr_dict=None) -> GridTensor:
    grid: GridTensor = tensor.as_subclass(GridTensor)
    if tag_stack and load_stack:
        grid.deep_pack(tag_stack, load_stack, **(extra_attr_dict or {}))
    else:
        grid.init_cell()
    return grid


def init_grid_tensor_from(tensor: torch.Tensor, from_grid_tensor: GridTensor) -> GridTensor:
    _, tags, loads, extra = to_torch_tensor(from_grid_tensor, True)
    return init_grid_tensor(tensor, tags, loads, extra)


def deinit_grid_tensor(grid_t: GridTensor, retrieve_attr: bool = True):
    if not retrieve_attr:
        return grid_t.as_subclass(torch.Tensor)
    grid_t, tags, loads, extra = grid_t.deep_unpack()
    return grid_t.as_subclass(torch.Tensor), tags, loads, extra


def to_grid_tensor(torch_t: torch.Tensor, tag_stack=None, load_stack=None,
                   extra_attr_dict=None) -> GridTensor:
    return init_grid_tensor(torch_t, tag_stack, load_stack, extra_attr_dict)


def to_torch_tensor(grid_t, retrieve_attr: bool = False):
    """Plain-tensor view of ``grid_t`` (so that router internals do not pay for
    ``__torch_function__``), optionally with its stacks."""
    if not retrieve_attr:
        return grid_t.as_subclass(torch.Tensor)
    if not isinstance(grid_t, GridTensor):
        grid_t = init_grid_tensor(grid_t, [None], [None])
    _, tags, loads, extra = grid_t.copy_cell_attr()
    return grid_t.as_subclass(torch.Tensor), tags, loads, extra
