"""Set-up of the NVLink peer-memory exchange (kernels: csrc/exchange_p2p.cu, host side:
csrc/exchange_plan.cu).

One arena per process: a control block (flags, size boards, kept size matrices) followed by
two landing halves that alternate from one exchange to the next.  The arena is exported
through CUDA IPC; handles travel between the ranks of the box through ``torch.distributed``.
An exchange lands every bucket straight at its place in the receiver's output layout, and
the output tensor handed to the caller is a view of the landing half (no copy-out):

* it stays valid until this rank enters the SECOND exchange after the one that produced it
  (peers only write into a half once its owner has entered the exchange that uses it);
* ``BRT_P2P_ZERO_COPY=0`` makes every exchange return a private copy instead.
"""
import ctypes
import os
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib

STATUS_OFFSET = 1024      # status word of the bounded waits inside the control block
ZERO_COPY = os.environ.get("BRT_P2P_ZERO_COPY", "1") != "0"
SPARSE_INVERSE, SPARSE_FORWARD, SLOTS, SLOTS_BACK = 0, 1, 2, 3   # layouts of an exchange
MAX_BUCKETS = 1024        # world * group of one exchange (device planner)
BOARD_INTS = 7936         # world * world * group: the size matrix must fit a board


def buckets_supported(world: int, group_size: int) -> bool:
    return world * group_size <= MAX_BUCKETS and world * world * group_size <= BOARD_INTS


class _DeviceBytes:
    """Zero-copy view of raw device memory for torch (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


def _row_bytes(x: torch.Tensor) -> int:
    n = x.element_size()
    for extent in x.shape[1:]:
        n *= int(extent)
    return n


class PeerArena:
    """This rank's arena, its peers' arenas as mapped here, and the library's exchange
    context on top of them."""

    def __init__(self, rank: int, world: int, half_bytes: int, base: int, peer_base: List[int]):
        self.rank, self.world, self.half_bytes = rank, world, int(half_bytes)
        self.control_bytes = int(_lib.query("brt_p2p_control_bytes"))
        self.total = self.control_bytes + 2 * self.half_bytes
        self.base = base
        self.peer_base = list(peer_base)
        self._view = torch.as_tensor(_DeviceBytes(self.base, self.total), device="cuda")
        # the size matrix comes down on this stream, beside the rows
        self.side = torch.cuda.Stream()
        ctx = ctypes.c_void_p()
        arenas = (ctypes.c_void_p * world)(*self.peer_base)
        _lib.call("brt_p2p_ctx_create", world, rank, self.base, arenas, self.half_bytes,
                  ctypes.byref(ctx))
        self.ctx = ctx

    # ---- views of the landing halves -------------------------------------------------------
    def view(self, ptr: int, rows: int, like: torch.Tensor) -> torch.Tensor:
        """``rows`` rows shaped and typed like the rows of ``like``, at device address ``ptr``
        inside this arena (no copy)."""
        off = ptr - self.base
        nbytes = rows * _row_bytes(like)
        flat = self._view[off:off + nbytes].view(like.dtype)
        return flat.view((rows,) + tuple(like.shape[1:]))

    def _half_of_next_exchange(self):
        nxt = int(_lib.query("brt_p2p_ctx_exchanges", self.ctx)) + 1
        lo = self.base + self.control_bytes + (nxt & 1) * self.half_bytes
        return lo, lo + self.half_bytes

    def safe_source(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` itself unless it lives in the half the next exchange lands in (an output held
        for too long): then a private copy, taken before any peer may write there."""
        lo, hi = self._half_of_next_exchange()
        return x.clone() if lo <= x.data_ptr() < hi else x

    # ---- the two exchanges -----------------------------------------------------------------
    def sparse_forward(self, rows: torch.Tensor, sizes: torch.Tensor, group_size: int,
                       grain: int, stride_rows: int, layout: int = SPARSE_FORWARD):
        """Enqueue a forward exchange (packed buckets, or padded slots with ``layout=SLOTS``)
        on the current stream and wait for its size matrix only.  Returns (matrix
        [world, world * group] int32, my output rows, whether it fits the landing halves,
        device address of my output, exchange id)."""
        main = _lib.raw_stream()
        _lib.call("brt_p2p_sparse_forward_begin", self.ctx, rows.data_ptr(), sizes.data_ptr(),
                  group_size, grain, stride_rows, layout, main, self.side.cuda_stream, 0)
        return self._forward_sizes(group_size)

    def _forward_sizes(self, group_size: int):
        matrix = ctypes.POINTER(ctypes.c_int32)()
        n_rows, fits = ctypes.c_int64(), ctypes.c_int()
        out, xid = ctypes.c_void_p(), ctypes.c_uint64()
        _lib.call("brt_p2p_sparse_forward_sizes", self.ctx, self.side.cuda_stream,
                  ctypes.byref(matrix), ctypes.byref(n_rows), ctypes.byref(fits),
                  ctypes.byref(out), ctypes.byref(xid))
        S = np.ctypeslib.as_array(matrix, shape=(self.world, self.world * group_size)).copy()
        return S, int(n_rows.value), bool(fits.value), int(out.value), int(xid.value)

    def dispatch_forward(self, cells: torch.Tensor, route_indices: torch.Tensor,
                         loads: torch.Tensor, counts: torch.Tensor, group_size: int, grain: int,
                         stride_rows: int):
        """Dispatch fused with the forward packed exchange: every kept copy of a cell goes
        straight to its row in the destination rank's landing half.  Same results as
        ``sparse_forward`` of the dispatched rows."""
        main = _lib.raw_stream()
        _lib.call("brt_p2p_dispatch_forward_begin", self.ctx, cells.data_ptr(),
                  route_indices.data_ptr(), loads.data_ptr(), counts.data_ptr(), cells.size(0),
                  grain, group_size, stride_rows, main, self.side.cuda_stream, 0)
        return self._forward_sizes(group_size)

    # ---- exchanges whose sizes stay on the device (CUDA graph capture) ------------------------
    def replay_begin(self) -> None:
        """Open a section of exchanges that may be captured in a CUDA graph and replayed:
        exchanges issued with ``dispatch_forward_device`` / ``sparse_forward_device`` and
        ``sparse_backward``, closed by ``replay_end``.  Every rank opens, fills, closes and
        replays its sections alike."""
        _lib.call("brt_p2p_ctx_replay_begin", self.ctx)

    def replay_end(self) -> None:
        _lib.call("brt_p2p_ctx_replay_end", self.ctx)

    def _device_sizes(self, group_size: int, device):
        received = torch.empty((group_size * self.world,), dtype=torch.int32, device=device)
        out, cap, xid = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_uint64()
        _lib.call("brt_p2p_forward_device_sizes", self.ctx, received.data_ptr(),
                  _lib.raw_stream(), ctypes.byref(out), ctypes.byref(cap),
                  ctypes.byref(xid))
        return received, int(out.value), int(cap.value), int(xid.value)

    _DEVICE_STAGES = 1 | 4 | 8 | 16  # post, push, wait; rows that do not fit are an error

    def sparse_forward_device(self, rows: torch.Tensor, sizes: torch.Tensor, group_size: int,
                              grain: int, stride_rows: int, layout: int = SPARSE_FORWARD):
        """``sparse_forward`` without a host synchronisation.  Returns (rows this rank receives
        as a device tensor [group, world] flattened, device address of my output, the rows
        the output can hold, exchange id)."""
        main = _lib.raw_stream()
        _lib.call("brt_p2p_sparse_forward_begin", self.ctx, rows.data_ptr(), sizes.data_ptr(),
                  group_size, grain, stride_rows, layout, main, main, self._DEVICE_STAGES)
        return self._device_sizes(group_size, rows.device)

    def dispatch_forward_device(self, cells: torch.Tensor, route_indices: torch.Tensor,
                                loads: torch.Tensor, counts: torch.Tensor, group_size: int,
                                grain: int, stride_rows: int):
        """``dispatch_forward`` without a host synchronisation; returns what
        ``sparse_forward_device`` returns."""
        main = _lib.raw_stream()
        _lib.call("brt_p2p_dispatch_forward_begin", self.ctx, cells.data_ptr(),
                  route_indices.data_ptr(), loads.data_ptr(), counts.data_ptr(), cells.size(0),
                  grain, group_size, stride_rows, main, main, self._DEVICE_STAGES)
        return self._device_sizes(group_size, cells.device)

    # ---- the inverse exchange folded into the combine ---------------------------------------
    def offset_of(self, t: torch.Tensor):
        """Byte offset of ``t`` inside the landing halves of this arena, or None when it lives
        elsewhere."""
        off = t.data_ptr() - self.base
        nbytes = t.numel() * t.element_size()
        if off < self.control_bytes or off + nbytes > self.total:
            return None
        return off

    def expert_buffer(self, rows: int, like: torch.Tensor) -> torch.Tensor:
        """``rows`` rows shaped like the rows of ``like`` in the landing half that the next
        exchange would use: after a forward exchange that is the half its output is NOT in, a
        place for expert outputs that ``combine_backward`` can pull from.  Every rank gets the
        same offset."""
        lo, hi = self._half_of_next_exchange()
        if rows * _row_bytes(like) > hi - lo:
            raise RuntimeError("the expert outputs do not fit a landing half")
        return self.view(lo, rows, like)

    def combine_backward(self, exchange_id: int, group_size: int, grain: int, stride_rows: int,
                         rows_offset: int, route_indices: torch.Tensor, gates, gates_dtype: int,
                         dtype: int, out: torch.Tensor) -> None:
        """Enqueue the combine that pulls the expert outputs (at ``rows_offset`` in every
        rank's arena, laid out as forward exchange ``exchange_id`` landed them) over NVLink."""
        _lib.call("brt_p2p_combine_backward", self.ctx, exchange_id, group_size, grain,
                  stride_rows, rows_offset, route_indices.data_ptr(),
                  None if gates is None else gates.data_ptr(), gates_dtype, dtype,
                  route_indices.size(0), out.data_ptr(), _lib.raw_stream(), 0)

    def sparse_backward(self, exchange_id: int, group_size: int, grain: int, stride_rows: int,
                        rows: torch.Tensor, layout: int = SPARSE_INVERSE,
                        zero_tails: bool = False):
        """Enqueue the inverse of forward exchange ``exchange_id`` on the current stream.
        Returns (device address of my output, its rows).  Raises ``_lib.BrtError`` with status
        BRT_ERR_UNSUPPORTED (on every rank alike) when the exchange cannot take this path."""
        out, n_rows = ctypes.c_void_p(), ctypes.c_int64()
        _lib.call("brt_p2p_sparse_backward", self.ctx, exchange_id, group_size, grain,
                  stride_rows, layout, int(zero_tails), rows.data_ptr(),
                  _lib.raw_stream(), 0, ctypes.byref(out),
                  ctypes.byref(n_rows))
        return int(out.value), int(n_rows.value)

    def trace(self):
        """(wait, move, plan, first CTA out, last CTA out) of the last forward landing kernel
        and the same five of the last inverse one, in microseconds; synchronises the device."""
        t = (ctypes.c_uint64 * 10)()
        _lib.call("brt_p2p_ctx_trace", self.ctx, t)
        return [v / 1e3 for v in t]

    def status(self) -> int:
        return int(_lib.query("brt_p2p_ctx_status", self.ctx))

    def set_wait_limit(self, seconds: float) -> None:
        _lib.call("brt_p2p_ctx_set_wait_limit", self.ctx, int(seconds * 1e9))


_arena: Optional[PeerArena] = None
_disabled_reason: Optional[str] = None


def arena() -> Optional[PeerArena]:
    return _arena


def setup(group, rank: int, world: int) -> Optional[PeerArena]:
    """Create the arena on every rank, or on none.  Every rank takes part in every
    collective of this function whatever happens to it locally, so a rank that cannot
    allocate or map makes all ranks fall back to the NCCL transport instead of hanging."""
    global _arena, _disabled_reason
    if _arena is not None or _disabled_reason is not None:
        return _arena
    if os.environ.get("BRT_P2P", "1") == "0":
        _disabled_reason = "BRT_P2P=0"
        return None
    half = int(os.environ.get("BRT_P2P_ARENA_MB", "2048")) << 20
    base, handle, err = None, None, ""
    try:
        if dist.get_world_size(group) != torch.cuda.device_count() and \
                int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
            raise RuntimeError("ranks span more than one box")
        ptr = ctypes.c_void_p()
        buf = (ctypes.c_ubyte * 64)()
        total = int(_lib.query("brt_p2p_control_bytes")) + 2 * half
        _lib.call("brt_p2p_alloc", total, ctypes.byref(ptr), buf)
        base, handle = ptr.value, bytes(buf)
    except Exception as exc:  # IPC not permitted, out of memory, ...
        err = str(exc)
    handles: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    opened: List[int] = []
    peer_base: List[int] = []
    ok = all(h is not None for h in handles)
    if ok:
        try:
            for r in range(world):
                if r == rank:
                    peer_base.append(base)
                    continue
                p = ctypes.c_void_p()
                _lib.call("brt_p2p_open", (ctypes.c_ubyte * 64).from_buffer_copy(handles[r]),
                          ctypes.byref(p))
                opened.append(p.value)
                peer_base.append(p.value)
        except Exception as exc:
            ok, err = False, str(exc)
    made = None
    if ok:
        try:
            made = PeerArena(rank, world, half, base, peer_base)
        except Exception as exc:
            ok, err = False, str(exc)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 1:
        _arena = made
        return _arena
    for p in opened:
        try:
            _lib.call("brt_p2p_close", p)
        except Exception:
            pass
    if base is not None:
        try:
            _lib.call("brt_p2p_free", base)
        except Exception:
            pass
    _disabled_reason = err or "another rank could not allocate or map the arena"
    return None


def reset(group=None) -> None:
    """Collective: bring the arena of every rank back to its initial state after a bounded
    wait ran out (``check_status`` raised).  Exchanges issued before the reset are lost; CUDA
    graphs that hold exchanges must be captured again."""
    if _arena is None:
        return
    torch.cuda.synchronize()
    dist.barrier(group=group)
    _lib.call("brt_p2p_ctx_reset_status", _arena.ctx)
    dist.barrier(group=group)


def check_status() -> None:
    """Raise if a bounded wait of an earlier exchange ran out.  Reads a word of host memory
    that the kernels write; no device synchronisation."""
    if _arena is not None and _arena.status() != 0:
        raise RuntimeError("peer exchange timed out waiting for another rank (the bound is "
                           "PeerArena.set_wait_limit, 2 s by default)")
