"""Drop-in for the reference's ``brt._C.router`` extension.

Same function names, argument order, defaults, return shapes and error type
(``RuntimeError``) as the pybind module defined in src/backend/torch/router.cc:479-513 of
the reference.  Shape logic and output allocation live here (torch's caching allocator);
all device work goes through the C ABI in ``include/brt_b200.h``.  Differences that are
deliberate:

* bf16 is accepted wherever fp16 is (the reference raises for bf16);
* kernels are enqueued on the *current* stream (the reference uses the default stream;
  identical when the current stream is the default one);
* outputs are never pre-zeroed by a separate memset: the kernels write every byte.
"""
import os
from typing import List, Optional

import torch

from .. import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _check_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        # wording of CHECK_ON_CUDA, src/backend/torch/torch.h:20
        raise RuntimeError(f"{name} must be a CUDA tensor")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return _lib.raw_stream(device)


def _int32c(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be an int32 tensor, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _contig_rows(t: torch.Tensor, cell_size: int) -> torch.Tensor:
    flat = t.reshape(t.size(0), cell_size)
    return flat if flat.is_contiguous() else flat.contiguous()


class _ScratchPool:
    """One reusable scratch buffer per (purpose, device, stream).  Reuse is safe for calls
    enqueued on the same stream; a different stream gets its own buffer.  At most ``LIMIT``
    buffers are kept: the least recently used one is dropped (torch's allocator keeps its
    memory alive until the stream it was used on has passed it)."""

    LIMIT = 16

    def __init__(self):
        self._bufs = {}

    def get(self, purpose: str, device: torch.device, nbytes: int) -> torch.Tensor:
        key = (purpose, device.index, _lib.raw_stream(device))
        buf = self._bufs.pop(key, None)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        self._bufs[key] = buf  # most recently used last
        while len(self._bufs) > self.LIMIT:
            self._bufs.pop(next(iter(self._bufs)))  # dicts keep insertion order: the oldest
        return buf


_scratch = _ScratchPool()


_DENSE = "_brt_dense_counts"
_USE_DENSE = os.environ.get("BRT_DISPATCH_DENSE", "1") != "0"  # 0: always the general route


def _mark_dense(indices: torch.Tensor, counts: torch.Tensor) -> None:
    """Remember, on the tensor itself, that ``indices`` came out of an index kernel: column e
    holds every seat 1 .. counts[e] exactly once.  ``dispatch_with_indices_and_loads`` then
    knows which output rows stay empty without scanning for them and runs as one launch.
    The note does not survive slicing, cloning or any other op; code that edits such a tensor
    IN PLACE must delete the attribute."""
    setattr(indices, _DENSE, counts)


def check_index_status() -> None:
    """Raise (once) if an index scan enqueued earlier gave up a bounded wait: its indices and
    loads are wrong.  Reads a word of host memory that the kernels write, no device
    synchronisation; every index op calls it on entry, so the error surfaces at the next
    index op at the latest."""
    code = _lib.query("brt_index_status")
    if code != 0:
        _lib.query("brt_index_status_reset")
        if code == 1:
            raise _lib.BrtError("a fused throttle + index scan was given a mask with values "
                                "other than 0/1; the indices it returned are zero", 1)
        raise _lib.BrtError("an index scan gave up waiting for the column sums of an earlier "
                            "CTA (BRT_ERR_TIMEOUT); the indices and loads it returned are "
                            "not valid", code)


def throttle_hotmask(hotmask: torch.Tensor, prefix: torch.Tensor, threshold: torch.Tensor):
    """src/backend/torch/router.cc:15-31.  ``prefix`` is updated in place and returned."""
    _check_cuda(hotmask, "hotmask")
    _check_cuda(prefix, "prefix")
    _check_cuda(threshold, "threshold")
    check_index_status()
    if hotmask.size(1) != prefix.size(0) or hotmask.size(1) != threshold.size(0):
        raise RuntimeError("CHECK_EQ fails.")
    hotmask = _int32c(hotmask, "hotmask")
    threshold = _int32c(threshold, "threshold")
    if prefix.dtype != torch.int32 or not prefix.is_contiguous():
        raise RuntimeError("prefix must be a contiguous int32 tensor (it is updated in place)")
    T, E = hotmask.shape
    with _lib.device_guard(hotmask.device):
        out = torch.empty_like(hotmask)
        nbytes = _lib.query("brt_index_scratch_bytes", T, E)
        scratch = _scratch.get("index", hotmask.device, nbytes)
        _lib.call("brt_throttle_hotmask", _ptr(hotmask), _ptr(out), _ptr(prefix),
                  _ptr(threshold), T, E, _ptr(scratch), scratch.numel(),
                  _stream(hotmask.device))
    return out, prefix


def generate_indices_and_loads(
    hot_mask: torch.Tensor,
    supported_capacities: Optional[torch.Tensor] = None,
    capacity_padding: bool = False,
    path_wise_padding: bool = False,
    is_tag_index: bool = False,
):
    """src/backend/torch/router.cc:48-80."""
    _check_cuda(hot_mask, "hot_mask")
    check_index_status()
    hot_mask = _int32c(hot_mask, "hot_mask")
    T, E = hot_mask.shape
    with _lib.device_guard(hot_mask.device):
        if hot_mask.numel() == 0:
            return (torch.zeros((0, E), dtype=torch.int32, device=hot_mask.device),
                    torch.zeros((E,), dtype=torch.int32, device=hot_mask.device))
        caps = None
        ncap = 0
        if supported_capacities is not None:
            _check_cuda(supported_capacities, "supported_capacities.value()")
            caps = _int32c(supported_capacities, "supported_capacities")
            ncap = caps.size(0)
        indices = torch.empty_like(hot_mask)
        both = torch.empty((2, E), dtype=torch.int32, device=hot_mask.device)
        loads, counts = both[0], both[1]
        nbytes = _lib.query("brt_index_scratch_bytes", T, E)
        scratch = _scratch.get("index", hot_mask.device, nbytes)
        _lib.call("brt_generate_indices_and_loads", _ptr(hot_mask), _ptr(indices), _ptr(loads),
                  None if is_tag_index else _ptr(counts), T, E, _ptr(caps), ncap,
                  int(bool(capacity_padding)), int(bool(path_wise_padding)),
                  int(bool(is_tag_index)), _ptr(scratch), scratch.numel(),
                  _stream(hot_mask.device))
        if not is_tag_index:
            _mark_dense(indices, counts)
    return indices, loads


def throttle_and_generate_indices(
    hot_mask: torch.Tensor,
    prefix: torch.Tensor,
    threshold: torch.Tensor,
    supported_capacities: Optional[torch.Tensor] = None,
    capacity_padding: bool = False,
    path_wise_padding: bool = False,
    with_mask: bool = False,
):
    """``throttle_hotmask`` followed by ``generate_indices_and_loads`` (seat indices) of the
    throttled 0/1 mask, as one pass over the mask (no counterpart in the reference's
    extension: python/brt/router/protocol/swin_moe.py:112-140 and
    python/brt/router/fabric/generic.py:83-89 call the two ops one after the other).
    Returns (indices, loads, prefix), plus the throttled mask with ``with_mask``; ``prefix``
    is updated in place.  Masks the single-launch scan cannot take go through the two ops."""
    _check_cuda(hot_mask, "hot_mask")
    _check_cuda(prefix, "prefix")
    _check_cuda(threshold, "threshold")
    check_index_status()
    if hot_mask.size(1) != prefix.size(0) or hot_mask.size(1) != threshold.size(0):
        raise RuntimeError("CHECK_EQ fails.")
    hot_mask = _int32c(hot_mask, "hot_mask")
    threshold = _int32c(threshold, "threshold")
    if prefix.dtype != torch.int32 or not prefix.is_contiguous():
        raise RuntimeError("prefix must be a contiguous int32 tensor (it is updated in place)")
    T, E = hot_mask.shape
    dev = hot_mask.device
    with _lib.device_guard(dev):
        caps, ncap = None, 0
        if supported_capacities is not None:
            _check_cuda(supported_capacities, "supported_capacities.value()")
            caps = _int32c(supported_capacities, "supported_capacities")
            ncap = caps.size(0)
        indices = torch.empty_like(hot_mask)
        both = torch.empty((2, E), dtype=torch.int32, device=dev)
        loads, counts = both[0], both[1]
        throttled = torch.empty_like(hot_mask) if with_mask else None
        nbytes = _lib.query("brt_index_scratch_bytes", T, E)
        scratch = _scratch.get("index", dev, nbytes)
        try:
            _lib.call("brt_throttle_and_generate_indices", _ptr(hot_mask), _ptr(indices),
                      _ptr(loads), _ptr(counts), _ptr(prefix), _ptr(threshold), _ptr(throttled),
                      T, E, _ptr(caps), ncap, int(bool(capacity_padding)),
                      int(bool(path_wise_padding)), _ptr(scratch), scratch.numel(), _stream(dev))
            _mark_dense(indices, counts)
        except _lib.BrtError as exc:
            if exc.status != 4:  # BRT_ERR_UNSUPPORTED: the two-step route takes every shape
                raise
            throttled, prefix = throttle_hotmask(hot_mask, prefix, threshold)
            indices, loads = generate_indices_and_loads(throttled, supported_capacities,
                                                        capacity_padding, path_wise_padding)
    return (indices, loads, prefix, throttled) if with_mask else (indices, loads, prefix)


_GATE = {"topk": 0, "threshold": 1}
_ROUTE_OUT = {"mask": 0, "throttled_mask": 1, "seat_indices": 2, "throttled_seat_indices": 3}


def route_scores_supported(score: torch.Tensor) -> bool:
    """Whether ``route_scores`` can take ``score`` (the single-launch gate wants contiguous
    fp32 CUDA scores over a multiple of 4 and at most 256 paths)."""
    return (score.is_cuda and score.dtype == torch.float32 and score.dim() == 2
            and score.is_contiguous() and score.size(1) % 4 == 0 and 0 < score.size(1) <= 256
            and score.data_ptr() % 16 == 0)


def route_scores(
    score: torch.Tensor,
    decision: str = "topk",
    top_k: int = 1,
    threshold: float = 0.0,
    residual_path: int = -1,
    output: str = "mask",
    supported_capacities: Optional[torch.Tensor] = None,
    capacity_padding: bool = False,
    path_wise_padding: bool = False,
    prefix: Optional[torch.Tensor] = None,
    throttle_capacity: Optional[torch.Tensor] = None,
    with_gates: bool = False,
    with_mask: bool = False,
):
    """Route decision and index scan in one launch, straight from the gate's scores (no
    counterpart in the reference's extension: it fuses a protocol of
    python/brt/router/protocol/ with ``throttle_hotmask`` / ``generate_indices_and_loads``).

    ``output`` = "mask": (hot_mask, cells per path); "throttled_mask": (hot_mask cut at
    ``throttle_capacity`` on top of ``prefix``, prefix) with ``prefix`` updated in place;
    "seat_indices": (indices, loads) as ``generate_indices_and_loads`` of the hot mask;
    "throttled_seat_indices": (indices, loads, prefix) of the throttled hot mask.
    ``with_mask`` (seat-index outputs) appends the 0/1 mask the indices belong to.
    ``with_gates`` appends the picked scores renormalised to sum 1 per cell.  Raises
    ``NotImplementedError`` when the scores do not fit the single-launch kernel; callers then
    route in two steps."""
    _check_cuda(score, "score")
    check_index_status()
    if decision not in _GATE or output not in _ROUTE_OUT:
        raise RuntimeError(f"unknown decision {decision!r} or output {output!r}")
    if not route_scores_supported(score):
        raise NotImplementedError("route_scores needs contiguous fp32 scores over a multiple "
                                  "of 4 and at most 256 paths")
    T, E = score.shape
    dev = score.device
    with _lib.device_guard(dev):
        out = torch.empty((T, E), dtype=torch.int32, device=dev)
        both = torch.empty((2, E), dtype=torch.int32, device=dev)
        loads, counts = both[0], both[1]
        seats = output in ("seat_indices", "throttled_seat_indices")
        gates = torch.empty((T, E), dtype=torch.float32, device=dev) if with_gates else None
        if with_mask and not seats:
            raise RuntimeError("with_mask goes with the seat-index outputs")
        mask_out = torch.empty((T, E), dtype=torch.int32, device=dev) if with_mask else None
        caps, ncap = None, 0
        if supported_capacities is not None:
            _check_cuda(supported_capacities, "supported_capacities")
            caps = _int32c(supported_capacities, "supported_capacities")
            ncap = caps.size(0)
        if capacity_padding and ncap < 1:
            raise RuntimeError("capacity_padding needs at least one supported capacity")
        thr = None
        if output in ("throttled_mask", "throttled_seat_indices"):
            if prefix is None or throttle_capacity is None:
                raise RuntimeError("a throttled output needs prefix and throttle_capacity")
            _check_cuda(prefix, "prefix")
            _check_cuda(throttle_capacity, "throttle_capacity")
            if prefix.dtype != torch.int32 or not prefix.is_contiguous() or prefix.numel() != E:
                raise RuntimeError("prefix must be a contiguous int32 tensor of one entry per "
                                   "path (it is updated in place)")
            thr = _int32c(throttle_capacity, "throttle_capacity")
            if thr.numel() != E:
                raise RuntimeError("CHECK_EQ fails.")
        nbytes = _lib.query("brt_index_scratch_bytes", T, E)
        scratch = _scratch.get("index", dev, nbytes)
        try:
            _lib.call("brt_route_scores", _ptr(score), T, E, _GATE[decision], int(top_k),
                      float(threshold), int(residual_path), _ROUTE_OUT[output], _ptr(out),
                      _ptr(loads), _ptr(counts) if seats else None, _ptr(caps), ncap,
                      int(bool(capacity_padding)),
                      int(bool(path_wise_padding)), _ptr(prefix), _ptr(thr), _ptr(gates),
                      _ptr(mask_out), _ptr(scratch), scratch.numel(), _stream(dev))
        except _lib.BrtError as exc:
            if exc.status == 4:  # BRT_ERR_UNSUPPORTED: too many scores for one launch
                raise NotImplementedError(str(exc)) from None
            raise
        if seats:
            _mark_dense(out, counts)
    if output == "throttled_seat_indices":
        res = (out, loads, prefix)
        if with_gates:
            res += (gates,)
        if with_mask:
            res += (mask_out,)
        return res
    res = (out, prefix if output == "throttled_mask" else loads)
    if with_gates:
        res += (gates,)
    if with_mask:
        res += (mask_out,)
    return res


def convert_index_format(origin_indices: torch.Tensor, loads: torch.Tensor, is_to_tag: bool):
    """src/backend/torch/router.cc:90-110.  As in the reference, ``is_to_tag`` travels into
    the launcher's ``tag_to_seat`` argument, so ``True`` converts tag indices to seat
    indices."""
    _check_cuda(origin_indices, "origin_indices")
    origin = _int32c(origin_indices, "origin_indices")
    T, E = origin.shape
    with _lib.device_guard(origin.device):
        cuda_loads = loads
        if not loads.is_cuda:
            if is_to_tag:
                # the reference only moves CPU loads when is_to_tag is false and then hands a
                # host pointer to the kernel; refuse instead of faulting
                raise RuntimeError("loads must be a CUDA tensor")
            cuda_loads = loads.to(origin.device, non_blocking=True)
        cuda_loads = _int32c(cuda_loads, "loads")
        out = torch.empty_like(origin)
        _lib.call("brt_convert_index_format", _ptr(origin), _ptr(out), _ptr(cuda_loads), T, E,
                  int(bool(is_to_tag)), _stream(origin.device))
    return out


def dispatch_with_indices_and_loads(
    in_data: torch.Tensor,
    route_indices: torch.Tensor,
    loads: torch.Tensor,
    gates: Optional[torch.Tensor] = None,
    tag_generating: bool = False,
    tags: Optional[torch.Tensor] = None,
    max_path_padding: bool = False,
    max_path_load: int = 0,
    is_1d_routing: bool = True,
    is_tag_index: bool = False,
) -> List[torch.Tensor]:
    """src/backend/torch/router.cc:131-273."""
    _check_cuda(in_data, "in_data")
    _check_cuda(route_indices, "route_indices")
    dev = in_data.device
    with _lib.device_guard(dev):
        cell_num = in_data.size(0)
        path_num = route_indices.size(1)
        if cell_num == 0:
            shape = list(in_data.shape)
            if is_1d_routing:
                shape[0] = 0
            else:
                if len(shape) == 2:
                    shape.append(1)
                shape[1] = 0
                shape = shape[1:]
            out = [torch.zeros(shape, dtype=in_data.dtype, device=dev)]
            if tag_generating:
                out.append(torch.zeros((0,), dtype=route_indices.dtype, device=dev))
            return out
        if in_data.dtype not in _DT:
            raise NotImplementedError("data type is not supported")
        cell_size = in_data.numel() // cell_num
        if not is_1d_routing:
            cell_size //= path_num
        if in_data.dtype == torch.float16 and cell_size % 2 != 0:
            raise RuntimeError("cell_size must be even when data type is float16")
        route_indices = _int32c(route_indices, "route_indices")
        cuda_loads = loads if loads.is_cuda else loads.to(dev, non_blocking=True)
        cuda_loads = _int32c(cuda_loads, "loads")
        # output size: the one host<->device sync of this op, as in the reference
        if max_path_padding:
            mpl = int(max_path_load) if max_path_load > 0 else int(loads.max().item())
            total = mpl * path_num
        else:
            mpl = 0
            total = int(loads.sum().item())
        shape = list(in_data.shape)
        if is_1d_routing:
            shape[0] = total
        else:
            if len(shape) == 2:
                shape.append(1)
            shape[1] = total
            shape = shape[1:]
        src = in_data if in_data.is_contiguous() else in_data.contiguous()
        out = torch.empty(shape, dtype=in_data.dtype, device=dev)
        g = None
        if gates is not None:
            if not is_1d_routing:
                raise RuntimeError("CHECK fails.")
            _check_cuda(gates, "gates.value()")
            if gates.dtype != in_data.dtype:
                raise RuntimeError("CHECK_EQ fails.")
            g = gates if gates.is_contiguous() else gates.contiguous()
        old_tags = new_tags = None
        if tag_generating:
            if tags is None:
                old_tags = torch.arange(1, cell_num + 1, dtype=route_indices.dtype, device=dev)
            else:
                _check_cuda(tags, "tags.value()")
                if tags.dtype != route_indices.dtype:
                    raise RuntimeError("CHECK_EQ fails.")
                old_tags = tags if tags.is_contiguous() else tags.contiguous()
            new_tags = torch.empty((total,), dtype=route_indices.dtype, device=dev)
        # indices that came straight out of an index kernel are known to be dense: one launch,
        # no scratch; any other index tensor takes the general two-launch route
        dense = None if is_tag_index else getattr(route_indices, _DENSE, None)
        if dense is not None and (dense.device != dev or dense.numel() != path_num
                                  or path_num > 2048 or not _USE_DENSE):
            dense = None
        scratch, nscratch = None, 0
        if dense is None and not is_tag_index:
            nscratch = _lib.query("brt_dispatch_scratch_bytes", total, path_num)
            scratch = _scratch.get("dispatch", dev, nscratch)
            nscratch = scratch.numel()
        _lib.call("brt_dispatch_with_indices_and_loads", _ptr(src), _ptr(out), _ptr(g),
                  _ptr(route_indices), _ptr(cuda_loads), _ptr(old_tags), _ptr(new_tags),
                  cell_num, cell_size, path_num, mpl, total, int(bool(is_1d_routing)),
                  int(bool(is_tag_index)), _DT[in_data.dtype], _ptr(dense), _ptr(scratch),
                  nscratch, _stream(dev))
    if tag_generating:
        return [out, new_tags]
    return [out]


def split_fused_cells_to_paths(
    in_data: torch.Tensor,
    loads: torch.Tensor,
    max_path_padding: bool = False,
    is_load_split: bool = False,
    is_tag_split: bool = False,
    tags: Optional[torch.Tensor] = None,
):
    """src/backend/torch/router.cc:285-335: per-path views of the fused tensor."""
    path_num = loads.numel()
    if is_tag_split:
        is_load_split = True
        if tags is None:
            raise RuntimeError("CHECK fails.")
    datas, loads_l, tags_l = [], [], []
    if max_path_padding:
        mpl = in_data.size(0) // path_num
        for i in range(path_num):
            datas.append(in_data.narrow(0, i * mpl, mpl))
            if is_load_split:
                loads_l.append(loads.narrow(0, i, 1))
            if is_tag_split:
                tags_l.append(tags.narrow(0, i * mpl, mpl))
    else:
        cpu_loads = loads.cpu().tolist()
        start = 0
        for i in range(path_num):
            n = int(cpu_loads[i])
            datas.append(in_data.narrow(0, start, n))
            if is_load_split:
                loads_l.append(loads.narrow(0, i, 1))
            if is_tag_split:
                tags_l.append(tags.narrow(0, start, n))
            start += n
    if is_tag_split:
        return [datas, loads_l, tags_l]
    if is_load_split:
        return [datas, loads_l]
    return [datas]


def fuse_split_cells_from_paths(
    in_data: List[torch.Tensor],
    is_load_fuse: bool = False,
    is_tag_fuse: bool = False,
    loads: Optional[List[torch.Tensor]] = None,
    tags: Optional[List[torch.Tensor]] = None,
):
    """src/backend/torch/router.cc:348-369."""
    out = torch.cat(in_data, 0)
    if is_load_fuse:
        if loads is None:
            raise RuntimeError("CHECK fails.")
        return [out, torch.cat(loads, 0)]
    if is_tag_fuse:
        if tags is None:
            raise RuntimeError("CHECK fails.")
        all_tags = torch.cat(tags, 0)
        new_tags, inverse = torch.unique(all_tags, sorted=True, return_inverse=True)
        return [out, new_tags, inverse]
    return [out]


def combine_with_indices_and_loads(
    in_data: torch.Tensor,
    route_indices: torch.Tensor,
    loads: Optional[torch.Tensor] = None,
    gates: Optional[torch.Tensor] = None,
    out_data: Optional[torch.Tensor] = None,
    max_path_padding: bool = False,
    ever_padded: bool = True,
    is_tag_index: bool = False,
    tags: Optional[torch.Tensor] = None,
) -> List[torch.Tensor]:
    """src/backend/torch/router.cc:372-473."""
    _check_cuda(in_data, "in_data")
    _check_cuda(route_indices, "route_indices")
    dev = in_data.device
    with _lib.device_guard(dev):
        cell_num = route_indices.size(0)
        if cell_num == 0:
            if not is_tag_index:
                return [out_data if out_data is not None else torch.empty_like(in_data)]
            return [torch.empty_like(in_data), torch.empty_like(tags), torch.zeros_like(tags)]
        if cell_num == 1:
            # single-cell shortcut of the reference binding (router.cc:402-412)
            if not is_tag_index:
                return [out_data + in_data] if out_data is not None else [in_data]
            return [in_data, tags, torch.ones_like(tags)]
        if not is_tag_index:
            if loads is None:
                raise RuntimeError("CHECK fails.")
            if in_data.dtype not in _DT:
                raise NotImplementedError("data type is not supported")
            cuda_loads = _int32c(loads.to(dev, non_blocking=True), "loads")
            route_indices = _int32c(route_indices, "route_indices")
            path_num = route_indices.size(1)
            rows = in_data.size(0)
            cell_size = in_data.numel() // rows if rows else 0
            if rows == 0:
                # nothing was routed anywhere; the shape of a cell is still known
                cell_size = 1
                for s in in_data.shape[1:]:
                    cell_size *= s
            g = None
            gdt = 0
            if gates is not None:
                _check_cuda(gates, "gates.value()")
                if gates.dtype not in (torch.float32, in_data.dtype):
                    raise RuntimeError("gates must be float32 or match the data type")
                g = gates if gates.is_contiguous() else gates.contiguous()
                gdt = _DT[g.dtype]
            mpl = rows // path_num if max_path_padding else 0
            src = in_data if in_data.is_contiguous() else in_data.contiguous()
            if out_data is not None:
                _check_cuda(out_data, "out_data_t")
                if not out_data.is_contiguous() or out_data.dtype != in_data.dtype:
                    raise RuntimeError("out_data must be contiguous and match in_data's dtype")
                out, residual = out_data, 1
            else:
                out = torch.empty((cell_num,) + tuple(in_data.shape[1:]), dtype=in_data.dtype,
                                  device=dev)
                residual = 0
            _lib.call("brt_combine_with_indices_and_loads", _ptr(src), _ptr(out), _ptr(g),
                      _ptr(route_indices), _ptr(cuda_loads), cell_num, cell_size, path_num, mpl,
                      residual, _DT[in_data.dtype], gdt, _stream(dev))
            return [out]
        # tag branch (router.cc:449-472): sum of rows per unique tag
        if tags is None:
            raise RuntimeError("CHECK fails.")
        cell_size = in_data.numel() // in_data.size(0)
        n = tags.size(0)
        tags_value = tags
        if out_data is not None:
            _check_cuda(out_data, "out_data_t")
            if out_data.size(0) != n:
                raise RuntimeError("CHECK_EQ fails.")
            # the reference calls the functional scatter_reduce and drops its result, so the
            # caller's tensor comes back unchanged
            out = out_data
        else:
            flat = _contig_rows(in_data, cell_size)
            index = route_indices.reshape(-1).to(torch.int32)
            if index.numel() != flat.size(0):
                raise RuntimeError("CHECK_EQ fails.")
            out = torch.empty((n, cell_size), dtype=in_data.dtype, device=dev)
            if in_data.dtype not in _DT:
                raise RuntimeError(f"unsupported data type {in_data.dtype}")
            nbytes = _lib.query("brt_sum_rows_scratch_bytes", flat.size(0), n)
            scratch = _scratch.get("row_sum", dev, nbytes)
            _lib.call("brt_sum_rows_by_index", _ptr(flat), _ptr(index), _ptr(out), flat.size(0),
                      n, cell_size, _DT[in_data.dtype], _ptr(scratch), scratch.numel(),
                      _stream(dev))
            out = out.reshape((n,) + tuple(in_data.shape[1:]))
            if ever_padded and int(tags_value[0].item()) == 0:
                out = out.narrow(0, 1, n - 1)
                tags_value = tags_value.narrow(0, 1, n - 1)
        out_loads = torch.tensor([tags_value.numel()], dtype=torch.int32, device=dev)
        return [out, tags_value, out_loads]
