"""Drop-in for the reference's ``brt._C.distributed`` extension
(src/backend/torch/distributed.cc:903-949): same 15 functions, argument names and return
shapes.  The exchange runs over the library's own NCCL communicator through the C ABI in
``include/brt_b200.h``; torch only allocates the outputs.

Deliberate differences from the reference:

* collectives are enqueued on the current stream instead of a private side stream fenced by
  events (the reference waits for them at once, so nothing overlapped there either);
* byte counts are 64-bit (the reference's ``int`` byte counts overflow past 2 GiB);
* sizes reach the host through one copy and one sync per call, not two;
* a second ``init_nccl`` raises ``RuntimeError`` instead of printing a warning.
"""
import ctypes
from typing import List

import numpy as np
import torch

from .. import _lib
from ..runtime import a2a_plan, p2p

_state = {"rank": None, "size": None}


def _check_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")


def _stream(device) -> int:
    return _lib.raw_stream(device)


def _world():
    if _state["size"] is None:
        r, s = ctypes.c_int(0), ctypes.c_int(0)
        _lib.call("brt_nccl_world", ctypes.byref(r), ctypes.byref(s))
        _state["rank"], _state["size"] = r.value, s.value
    return _state["rank"], _state["size"]


def _host_sizes(*tensors: torch.Tensor) -> List[np.ndarray]:
    """int32 size vectors -> host arrays with a single device->host copy and sync."""
    if all(not t.is_cuda for t in tensors):
        return [t.to(torch.int32).contiguous().numpy() for t in tensors]
    dev = next(t.device for t in tensors if t.is_cuda)
    flat = torch.cat([t.to(dev, torch.int32).reshape(-1) for t in tensors]).cpu().numpy()
    out, at = [], 0
    for t in tensors:
        out.append(np.ascontiguousarray(flat[at:at + t.numel()]))
        at += t.numel()
    return out


def _np_ptr(a: np.ndarray):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# ----------------------------------------------------------------------------- bootstrap


def make_nccl_unique_id(world_rank: int) -> torch.Tensor:
    """int8 tensor of 128 bytes on the GPU; only rank 0's content is meaningful.  The caller
    broadcasts it (python/brt/runtime/distributed.py:30-32 in the reference)."""
    t = torch.zeros(128, dtype=torch.int8)
    if world_rank == 0:
        _lib.call("brt_nccl_get_unique_id", t.data_ptr())
    return t.cuda()


def init_nccl(unique_id: torch.Tensor, world_rank: int, world_size: int) -> None:
    cpu = unique_id.to("cpu").contiguous()
    if cpu.numel() != 128:
        raise RuntimeError("unique_id must hold 128 bytes")
    _lib.call("brt_nccl_init", cpu.data_ptr(), int(world_rank), int(world_size))
    _state["rank"], _state["size"] = int(world_rank), int(world_size)


# ----------------------------------------------------------------------------- reorder


def locality_reorder(loads: torch.Tensor, wolrd_size: int):
    """(reordered_loads, reorder_indices); the argument keeps the reference's spelling."""
    return group_locality_reorder(loads, wolrd_size, 1)


def group_locality_reorder(loads: torch.Tensor, wolrd_size: int, group_size: int = 1):
    _check_cuda(loads, "loads")
    if loads.dtype != torch.int32:
        raise RuntimeError("loads must be an int32 tensor")
    W = int(wolrd_size)
    if loads.numel() != W * W * group_size:
        raise RuntimeError(f"loads must hold world_size^2 * group_size = {W * W * group_size} "
                           f"entries, got {loads.numel()}")
    src = _contig(loads)
    with _lib.device_guard(loads.device):
        out = torch.empty_like(src)
        idx = torch.empty(W, dtype=torch.int32, device=loads.device)
        _lib.call("brt_group_locality_reorder", src.data_ptr(), int(group_size), W,
                  idx.data_ptr(), out.data_ptr(), _stream(loads.device))
    return out, idx


def _exchange_one(in_data, dst, src):
    _check_cuda(in_data, "in_data")
    x = _contig(in_data)
    out = torch.empty_like(x)
    _lib.call("brt_exchange", x.data_ptr(), out.data_ptr(), x.numel() * x.element_size(), dst,
              src, _stream(x.device))
    return out


def exchange(in_data: torch.Tensor, reorder_indices: torch.Tensor) -> torch.Tensor:
    rank, _ = _world()
    dst, src = a2a_plan.exchange_partners(reorder_indices.cpu().tolist(), rank)
    return _exchange_one(in_data, dst, src)


def batched_exchange(in_datas: List[torch.Tensor], reorder_indices: torch.Tensor):
    rank, _ = _world()
    dst, src = a2a_plan.exchange_partners(reorder_indices.cpu().tolist(), rank)
    return [_exchange_one(x, dst, src) for x in in_datas]


def reverse_exchange(in_data: torch.Tensor, reorder_indices: torch.Tensor) -> torch.Tensor:
    rank, _ = _world()
    dst, src = a2a_plan.exchange_partners(reorder_indices.cpu().tolist(), rank)
    return _exchange_one(in_data, src, dst)


def batched_reverse_exchange(in_datas: List[torch.Tensor], reorder_indices: torch.Tensor):
    _check_cuda(reorder_indices, "reorder_indices")
    rank, _ = _world()
    dst, src = a2a_plan.exchange_partners(reorder_indices.cpu().tolist(), rank)
    return [_exchange_one(x, src, dst) for x in in_datas]


# ----------------------------------------------------------------------------- padded slots


def _exchange_sizes(send_sizes: torch.Tensor) -> torch.Tensor:
    """Sizes all-to-all: slice i of send_sizes goes to rank i (device tensors)."""
    _, W = _world()
    s = _contig(send_sizes)
    recv = torch.empty_like(s)
    _lib.call("brt_all_to_all", s.data_ptr(), recv.data_ptr(),
              s.numel() * s.element_size() // W, _stream(s.device))
    return recv


def _slot_a2a(in_data, send_np, recv_np, group_size, zero_fill):
    x = _contig(in_data)
    out = torch.zeros_like(x) if zero_fill else torch.empty_like(x)
    total = x.numel() * x.element_size()
    grain = total // x.size(0) if x.size(0) else 0
    slot = total // send_np.size
    _lib.call("brt_group_asymmetry_all_to_all", x.data_ptr(), out.data_ptr(), _np_ptr(send_np),
              _np_ptr(recv_np), grain, slot, group_size, _stream(x.device))
    return out


def _locality_tail(recv_sizes: torch.Tensor, group_size: int):
    """Gather every rank's received sizes on rank 0, match there, scatter the reordered
    loads and broadcast the permutation (src/backend/torch/distributed.cc:246-330)."""
    rank, W = _world()
    dev = recv_sizes.device
    st = _stream(dev)
    recv_sizes = _contig(recv_sizes)
    nbytes = recv_sizes.numel() * 4
    all_sizes = torch.empty(recv_sizes.numel() * W, dtype=torch.int32, device=dev) \
        if rank == 0 else None
    _lib.call("brt_gather", recv_sizes.data_ptr(),
              all_sizes.data_ptr() if rank == 0 else None, nbytes, 0, st)
    reordered = torch.empty_like(recv_sizes)
    if rank == 0:
        all_reordered, reorder_indices = group_locality_reorder(all_sizes, W, group_size)
    else:
        all_reordered = None
        reorder_indices = torch.empty(W, dtype=torch.int32, device=dev)
    _lib.call("brt_scatter", all_reordered.data_ptr() if rank == 0 else None,
              reordered.data_ptr(), nbytes, 0, st)
    _lib.call("brt_broadcast", reorder_indices.data_ptr(), reorder_indices.data_ptr(), W * 4, 0,
              st)
    return reordered, reorder_indices


def _slots_p2p(x: torch.Tensor, send_sizes: torch.Tensor, group_size: int):
    """The padded-slot exchange over peer memory: (out, recv_sizes on the device) or None when
    this exchange cannot take that path (decided from facts every rank shares)."""
    rank, W = _world()
    n = W * group_size
    if not _p2p_usable(x, W, group_size) or x.size(0) == 0 or x.size(0) % n != 0:
        return None
    arena = p2p.arena()
    stride = x.size(0) // n
    x = arena.safe_source(x)
    sizes32 = send_sizes.to(torch.int32).contiguous()
    S, out_rows, fits, ptr, xid = arena.sparse_forward(x, sizes32, group_size, _row_bytes(x),
                                                       stride, p2p.SLOTS)
    # slot (i, j) of my output holds what rank i sent from its slot (me, j)
    recv_np = np.ascontiguousarray(S[:, rank * group_size:(rank + 1) * group_size].reshape(-1))
    recv = torch.from_numpy(recv_np).to(x.device)
    if fits:
        out = _landed(arena, ptr, out_rows, x)
    else:
        send_np = np.ascontiguousarray(S[rank])
        out = _slot_a2a(x, send_np, recv_np, group_size, False)
    setattr(recv, _TAG, (xid, group_size))
    return out, recv


def _asymmetry(in_data, send_sizes, locality_aware, zero_fill=False):
    _check_cuda(in_data, "in_data")
    _check_cuda(send_sizes, "send_sizes")
    _, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(in_data.device):
        moved = _slots_p2p(_contig(in_data), send_sizes, group_size)
        if moved is not None:
            out, recv_sizes = moved
        else:
            recv_sizes = _exchange_sizes(send_sizes)
            send_np, recv_np = _host_sizes(send_sizes, recv_sizes)
            out = _slot_a2a(in_data, send_np, recv_np, group_size, zero_fill)
        if locality_aware:
            reordered, reorder_indices = _locality_tail(recv_sizes, group_size)
            return [out, reordered, reorder_indices]
    return [out, recv_sizes]


def asymmetry_all_to_all(in_data: torch.Tensor, send_sizes: torch.Tensor,
                         locality_aware: bool = False):
    return _asymmetry(in_data, send_sizes, locality_aware)


def group_asymmetry_all_to_all(in_data: torch.Tensor, send_sizes: torch.Tensor,
                               locality_aware: bool = False):
    return _asymmetry(in_data, send_sizes, locality_aware)


def batched_group_asymmetry_all_to_all(in_datas: List[torch.Tensor], send_sizes: torch.Tensor,
                                       locality_aware: bool = False):
    _check_cuda(send_sizes, "send_sizes")
    _, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(send_sizes.device):
        recv_sizes = _exchange_sizes(send_sizes)
        send_np, recv_np = _host_sizes(send_sizes, recv_sizes)
        outs = []
        for x in in_datas:
            _check_cuda(x, "in_data")
            outs.append(_slot_a2a(x, send_np, recv_np, group_size, False))
        if locality_aware:
            reordered, reorder_indices = _locality_tail(recv_sizes, group_size)
            return outs, reordered, reorder_indices
    return outs, recv_sizes, recv_sizes


def size_known_group_asymmetry_all_to_all(in_data: torch.Tensor, send_sizes: torch.Tensor,
                                          recv_sizes: torch.Tensor) -> torch.Tensor:
    """The way back of ``group_asymmetry_all_to_all``: ``send_sizes`` is what that call
    returned as received sizes.  Handed that very tensor, the rows travel over peer memory
    (it names the exchange whose size matrix every rank kept); rows beyond a slot's size come
    back as zeros, as in the reference (src/backend/torch/distributed.cc:523)."""
    _check_cuda(in_data, "in_data")
    _, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        n = W * group_size
        tag = getattr(send_sizes, _TAG, None)
        if tag is not None and tag[1] == group_size and x.size(0) and x.size(0) % n == 0 \
                and _p2p_usable(x, W, group_size):
            arena = p2p.arena()
            x = arena.safe_source(x)
            try:
                ptr, rows = arena.sparse_backward(tag[0], group_size, _row_bytes(x),
                                                  x.size(0) // n, x, p2p.SLOTS_BACK, True)
                return _landed(arena, ptr, rows, x)
            except _lib.BrtError as exc:
                if exc.status != 4:  # BRT_ERR_UNSUPPORTED is the same verdict on every rank
                    raise
        send_np, recv_np = _host_sizes(send_sizes, recv_sizes)
        return _slot_a2a(x, send_np, recv_np, group_size, True)


def batched_size_known_group_asymmetry_all_to_all(in_datas: List[torch.Tensor],
                                                  send_sizes: torch.Tensor,
                                                  recv_sizes: torch.Tensor):
    _, W = _world()
    send_np, recv_np = _host_sizes(send_sizes, recv_sizes)
    outs = []
    for x in in_datas:
        _check_cuda(x, "in_data")
        with _lib.device_guard(x.device):
            outs.append(_slot_a2a(x, send_np, recv_np, send_sizes.numel() // W, False))
    return outs


# ----------------------------------------------------------------------------- packed buckets


def _sparse_a2a(x, send_np, recv_np, stride_rows, out_rows, group_size, forward):
    shape = list(x.shape)
    shape[0] = out_rows
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    grain = (x.numel() * x.element_size()) // x.size(0) if x.size(0) else \
        int(np.prod(shape[1:])) * x.element_size()
    _lib.call("brt_group_sparse_all_to_all", x.data_ptr(), out.data_ptr(), _np_ptr(send_np),
              _np_ptr(recv_np), grain, stride_rows, group_size, int(forward),
              _stream(x.device))
    return out


def _row_bytes(x: torch.Tensor) -> int:
    """Bytes of one row (the same on every rank, even on one that holds no rows)."""
    n = x.element_size()
    for extent in x.shape[1:]:
        n *= int(extent)
    return n


def _p2p_usable(x: torch.Tensor, world: int, group_size: int) -> bool:
    """Whether the peer-memory exchange can move ``x``.  Only facts that are the same on every
    rank decide (arena present, bucket count, row size), so all ranks take the same path."""
    a = p2p.arena()
    if a is None or not p2p.buckets_supported(world, group_size) or x.dim() < 1:
        return False
    row_bytes = _row_bytes(x)
    if row_bytes <= 0 or row_bytes % 16 != 0:
        return False
    if x.data_ptr() % 16 != 0:
        raise RuntimeError("rows of the peer exchange must start on a 16-byte boundary")
    return True


_TAG = "_brt_exchange"


def _landed(arena, ptr: int, rows: int, like: torch.Tensor) -> torch.Tensor:
    out = arena.view(ptr, rows, like)
    return out if p2p.ZERO_COPY else out.clone()


def group_sparse_all_to_all(in_data: torch.Tensor, send_sizes: torch.Tensor,
                            max_path_padding: bool = False, max_path_load: int = 0):
    """(out_data, recv_sizes [G, W] on CPU, send_sizes [W, G] on CPU).

    Over the peer-memory transport ``out_data`` is a view of this rank's landing half (see
    ``brainstorm_b200.runtime.p2p``), and both size tensors carry the identifier of the
    exchange, which is how ``size_known_group_sparse_all_to_all`` finds the size matrix that
    every rank kept for the way back."""
    _check_cuda(in_data, "in_data")
    _check_cuda(send_sizes, "send_sizes")
    rank, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        if _p2p_usable(x, W, group_size) and not (max_path_padding and not max_path_load):
            # The rows leave before the host knows any size: the landing kernel reads the size
            # matrix from the boards on the device.  The host only waits for the matrix (to
            # shape the output and to return the CPU size tensors of the reference's API).
            arena = p2p.arena()
            stride = int(max_path_load) if max_path_padding else 0
            x = arena.safe_source(x)
            sizes32 = send_sizes.to(torch.int32).contiguous()
            S, out_rows, fits, ptr, xid = arena.sparse_forward(x, sizes32, group_size,
                                                               _row_bytes(x), stride)
            S3 = S.reshape(W, W, group_size)
            send_np = np.ascontiguousarray(S3[rank].reshape(-1))
            recv_np = np.ascontiguousarray(S3[:, rank, :].T.reshape(-1))      # [G, W]
            if fits:
                out = _landed(arena, ptr, out_rows, x)
            else:  # some rank's rows exceed its landing half: NCCL on every rank, sizes known
                rows = a2a_plan.total_rows(recv_np, stride)
                out = _sparse_a2a(x, send_np, recv_np, stride, rows, group_size, True)
            recv_t, send_t = torch.from_numpy(recv_np), torch.from_numpy(send_np)
            setattr(recv_t, _TAG, (xid, group_size))
            setattr(send_t, _TAG, (xid, group_size))
            return [out, recv_t, send_t]
        recv_dev = _exchange_sizes(send_sizes.to(torch.int32))
        send_np, recv_np = _host_sizes(send_sizes, recv_dev)
        recv_np = a2a_plan.to_expert_major(recv_np, W)
        if max_path_padding:
            stride = int(max_path_load) if max_path_load else int(recv_np.max())
        else:
            stride = 0
        rows = a2a_plan.total_rows(recv_np, stride)
        out = _sparse_a2a(x, send_np, recv_np, stride, rows, group_size, True)
    return [out, torch.from_numpy(recv_np.copy()), torch.from_numpy(send_np.copy())]


def dispatch_group_sparse_all_to_all(in_data: torch.Tensor, route_indices: torch.Tensor,
                                     loads: torch.Tensor, max_path_padding: bool = False,
                                     max_path_load: int = 0):
    """``dispatch_with_indices_and_loads`` (unweighted, 1-D) followed by
    ``group_sparse_all_to_all``, as ONE kernel over peer memory: the sequence of the reference's
    expert-parallel dispatch fabric (python/brt/router/fabric/distributed.py:35-97) without the
    dispatched buffer in between — every kept copy of a cell is stored straight into the
    destination rank's output.  Returns what ``group_sparse_all_to_all`` returns, or ``None``
    when this call cannot take the fused route (no peer arena, rows that are not 16-byte
    multiples, index tensors that did not come from this library's index ops); the caller then
    runs the two ops.  The verdict depends on the program, not on the data, except for "the
    rows do not fit the landing halves", which every rank sees alike: the op then runs the two
    steps itself, with the sizes it already knows."""
    from . import router as c_router

    _check_cuda(in_data, "in_data")
    _check_cuda(route_indices, "route_indices")
    rank, W = _world()
    E = route_indices.size(1)
    counts = getattr(route_indices, c_router._DENSE, None)
    if counts is None or E % W != 0 or in_data.dim() < 2 or in_data.size(0) == 0 or \
            loads.numel() != E or not loads.is_cuda or route_indices.dtype != torch.int32 or \
            not route_indices.is_contiguous() or (max_path_padding and not max_path_load):
        return None
    group_size = E // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        if not _p2p_usable(x, W, group_size):
            return None
        arena = p2p.arena()
        stride = int(max_path_load) if max_path_padding else 0
        x = arena.safe_source(x)
        loads32 = loads.to(torch.int32).contiguous()
        S, out_rows, fits, ptr, xid = arena.dispatch_forward(
            x, route_indices, loads32, counts, group_size, _row_bytes(x), stride)
        S3 = S.reshape(W, W, group_size)
        send_np = np.ascontiguousarray(S3[rank].reshape(-1))
        recv_np = np.ascontiguousarray(S3[:, rank, :].T.reshape(-1))
        if fits:
            out = _landed(arena, ptr, out_rows, x)
        else:
            (routed,) = c_router.dispatch_with_indices_and_loads(
                x, route_indices, loads, None, False, None, max_path_padding, max_path_load)
            rows = a2a_plan.total_rows(recv_np, stride)
            out = _sparse_a2a(routed, send_np, recv_np, stride, rows, group_size, True)
        recv_t, send_t = torch.from_numpy(recv_np), torch.from_numpy(send_np)
        setattr(recv_t, _TAG, (xid, group_size))
        setattr(send_t, _TAG, (xid, group_size))
        return [out, recv_t, send_t]


def combine_group_sparse_all_to_all(in_data: torch.Tensor, route_indices: torch.Tensor,
                                    gates, send_sizes: torch.Tensor, recv_sizes: torch.Tensor,
                                    max_path_padding: bool = False):
    """``size_known_group_sparse_all_to_all`` followed by ``combine_with_indices_and_loads``
    (seat indices, no residual), as ONE kernel over peer memory: the sequence of the reference's
    expert-parallel combine fabric (python/brt/router/fabric/distributed.py:120-158) without the
    returned buffer in between - the combine of this rank's cells pulls every kept route's row
    from the arena of the rank that hosts the expert.  ``in_data`` are this rank's expert
    outputs in the layout the forward exchange landed (its output, changed in place, or a
    buffer from ``expert_output_buffer``); ``send_sizes`` / ``recv_sizes`` are the second and
    third output of that forward call.  Returns the combined cells [cells, ...], or ``None``
    when the call cannot take the fused route (no peer arena, size tensors that name no
    exchange, expert outputs outside the arena, rows that are not 16-byte multiples); the caller
    then runs the two ops.  The verdict depends on the program, not on the data.  A single cell
    is combined like any other number (the reference's combine hands a lone cell's rows back
    unweighted, router.cc:402-412)."""
    from . import router as c_router

    _check_cuda(in_data, "in_data")
    _check_cuda(route_indices, "route_indices")
    _, W = _world()
    E = route_indices.size(1)
    tag = getattr(send_sizes, _TAG, None)
    if tag is None or tag != getattr(recv_sizes, _TAG, None) or E % W != 0 or \
            tag[1] != E // W or in_data.dtype not in c_router._DT or in_data.dim() < 2 or \
            route_indices.dtype != torch.int32 or not route_indices.is_contiguous() or \
            not in_data.is_contiguous():
        return None
    group_size = E // W
    g, gdt = None, 0
    if gates is not None:
        if not gates.is_cuda or gates.dtype not in (torch.float32, in_data.dtype) or \
                gates.shape != route_indices.shape:
            return None
        g = gates if gates.is_contiguous() else gates.contiguous()
        gdt = c_router._DT[g.dtype]
    with _lib.device_guard(in_data.device):
        if not _p2p_usable(in_data, W, group_size):
            return None
        arena = p2p.arena()
        offset = arena.offset_of(in_data)
        if offset is None or offset % 16 != 0:
            return None
        stride = in_data.size(0) // (W * group_size) if max_path_padding else 0
        out = torch.empty((route_indices.size(0),) + tuple(in_data.shape[1:]),
                          dtype=in_data.dtype, device=in_data.device)
        try:
            arena.combine_backward(tag[0], group_size, _row_bytes(in_data), stride, offset,
                                   route_indices, g, gdt, c_router._DT[in_data.dtype], out)
        except _lib.BrtError as exc:
            if exc.status != 4:  # BRT_ERR_UNSUPPORTED is the same verdict on every rank
                raise
            return None
    return out


def expert_output_buffer(rows: int, like: torch.Tensor) -> torch.Tensor:
    """A buffer of ``rows`` rows like those of ``like`` that the fused combine can pull from:
    experts that do not work in place write their outputs here (same place on every rank;
    valid from the forward exchange until the next forward exchange but one)."""
    arena = p2p.arena()
    if arena is None:
        raise RuntimeError("no peer-memory arena")
    return arena.expert_buffer(rows, like)


class replayable_exchanges:
    """``with replayable_exchanges():`` around ``*_device`` exchanges and their inverses makes
    the sequence fit for CUDA graph capture: put the ``with`` inside ``torch.cuda.graph(...)``
    and replay the graph, or run the block again, as often as wanted, with ordinary exchanges
    in between if need be.  Every rank must do the same (the peers' kernels wait for each
    other).  A replay overwrites the outputs of the previous one."""

    def __enter__(self):
        arena = p2p.arena()
        if arena is None:
            raise RuntimeError("replayable exchanges need the peer-memory arena")
        arena.replay_begin()
        return self

    def __exit__(self, exc_type, exc, tb):
        try:
            p2p.arena().replay_end()
        except Exception:
            if exc_type is None:  # otherwise the error that ended the block is the one to show
                raise
        return False


def _device_result(arena, x, received, ptr, capacity, xid, group_size, sent):
    out = arena.view(ptr, capacity, x)
    setattr(received, _TAG, (xid, group_size))
    setattr(sent, _TAG, (xid, group_size))
    return [out, received, sent]


def group_sparse_all_to_all_device(in_data: torch.Tensor, send_sizes: torch.Tensor,
                                   max_path_padding: bool = False, max_path_load: int = 0):
    """``group_sparse_all_to_all`` without the host synchronisation of the reference's op
    (src/distributed/collective.cc:157-166): the size tensors stay on the device.  Returns
    (out_data, recv_sizes [G, W] int32 on the device, send_sizes on the device).  ``out_data``
    is the whole landing half seen as rows; its first ``recv_sizes.sum()`` rows are the
    output (with padding: every slot).  Peer-memory transport only; rows that do not fit the
    landing half are an error reported by ``p2p.check_status()``."""
    _check_cuda(in_data, "in_data")
    _check_cuda(send_sizes, "send_sizes")
    _, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        if not _p2p_usable(x, W, group_size) or (max_path_padding and not max_path_load):
            raise RuntimeError("this exchange cannot use the peer-memory transport")
        arena = p2p.arena()
        stride = int(max_path_load) if max_path_padding else 0
        x = arena.safe_source(x)
        sizes32 = send_sizes.to(torch.int32).contiguous()
        received, ptr, capacity, xid = arena.sparse_forward_device(
            x, sizes32, group_size, _row_bytes(x), stride)
        return _device_result(arena, x, received, ptr, capacity, xid, group_size, sizes32)


def dispatch_group_sparse_all_to_all_device(in_data: torch.Tensor, route_indices: torch.Tensor,
                                            loads: torch.Tensor, max_path_padding: bool = False,
                                            max_path_load: int = 0):
    """``dispatch_group_sparse_all_to_all`` with device-resident sizes (see
    ``group_sparse_all_to_all_device``).  ``route_indices`` must come from this library's
    index ops (dense seat columns)."""
    from . import router as c_router

    _check_cuda(in_data, "in_data")
    _check_cuda(route_indices, "route_indices")
    _, W = _world()
    E = route_indices.size(1)
    counts = getattr(route_indices, c_router._DENSE, None)
    if counts is None or E % W != 0 or in_data.dim() < 2 or in_data.size(0) == 0 or \
            loads.numel() != E or not loads.is_cuda or route_indices.dtype != torch.int32 or \
            not route_indices.is_contiguous() or (max_path_padding and not max_path_load):
        raise RuntimeError("this dispatch cannot be fused with the peer-memory exchange")
    group_size = E // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        if not _p2p_usable(x, W, group_size):
            raise RuntimeError("this exchange cannot use the peer-memory transport")
        arena = p2p.arena()
        stride = int(max_path_load) if max_path_padding else 0
        x = arena.safe_source(x)
        loads32 = loads.to(torch.int32).contiguous()
        received, ptr, capacity, xid = arena.dispatch_forward_device(
            x, route_indices, loads32, counts, group_size, _row_bytes(x), stride)
        return _device_result(arena, x, received, ptr, capacity, xid, group_size, loads32)


def size_known_group_sparse_all_to_all(in_data: torch.Tensor, send_sizes: torch.Tensor,
                                       recv_sizes: torch.Tensor,
                                       max_path_padding: bool = False) -> torch.Tensor:
    """Inverse of ``group_sparse_all_to_all``: ``send_sizes`` is that call's second output
    ([G, W]), ``recv_sizes`` its third ([W, G]).

    The peer-memory transport is taken when both tensors are the very objects the forward call
    returned (they name the exchange whose size matrix every rank kept); tensors built by the
    caller go over NCCL.  Which of the two happens depends on the program only, never on the
    data, so the ranks cannot disagree."""
    _check_cuda(in_data, "in_data")
    _, W = _world()
    group_size = send_sizes.numel() // W
    with _lib.device_guard(in_data.device):
        x = _contig(in_data)
        n = W * group_size
        stride = x.size(0) // n if max_path_padding else 0
        tag = getattr(send_sizes, _TAG, None)
        if tag is not None and tag == getattr(recv_sizes, _TAG, None) and \
                tag[1] == group_size and _p2p_usable(x, W, group_size):
            arena = p2p.arena()
            x = arena.safe_source(x)
            try:
                ptr, rows = arena.sparse_backward(tag[0], group_size, _row_bytes(x), stride, x)
                if send_sizes.is_cuda:  # device-resident sizes: `rows` is the half's capacity
                    return arena.view(ptr, rows, x)
                return _landed(arena, ptr, rows, x)
            except _lib.BrtError as exc:
                if exc.status != 4:  # BRT_ERR_UNSUPPORTED is the same verdict on every rank
                    raise
        send_np, recv_np = _host_sizes(send_sizes, recv_sizes)
        rows = x.size(0) if max_path_padding else a2a_plan.total_rows(recv_np)
        return _sparse_a2a(x, send_np, recv_np, stride, rows, group_size, False)
