"""Set-up of the NVLink peer-memory exchange (kernels: csrc/exchange_p2p.cu, planning:
csrc/exchange_plan.cu).

One arena per process: a control block (arrival flags, a completion counter, a status word,
size boards) followed by two data halves that alternate from one exchange to the next.  The
arena is exported through CUDA IPC; handles travel between the ranks of the box through
``torch.distributed``.  Everything an exchange enqueues is planned and issued by the
library's exchange context; this module creates it and forwards four calls.
"""
import ctypes
import os
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib

CONTROL_BYTES = 65536     # control block in front of the two data halves (laid out by the
STATUS_OFFSET = 1024      # library: flags, completion counter, status word, size boards)


class _DeviceBytes:
    """Zero-copy view of raw device memory for torch (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class PeerArena:
    def __init__(self, group, rank: int, world: int, half_bytes: int):
        self.rank, self.world, self.half_bytes = rank, world, int(half_bytes)
        self.total = CONTROL_BYTES + 2 * self.half_bytes
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        _lib.call("brt_p2p_alloc", self.total, ctypes.byref(ptr), handle)
        self.base = ptr.value
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_base: List[int] = []
        for r in range(world):
            if r == rank:
                self.peer_base.append(self.base)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
            p = ctypes.c_void_p()
            _lib.call("brt_p2p_open", buf, ctypes.byref(p))
            self.peer_base.append(p.value)
        self._view = torch.as_tensor(_DeviceBytes(self.base, self.total), device="cuda")
        self.status = self._view[STATUS_OFFSET:STATUS_OFFSET + 4].view(torch.int32)
        # copy-outs and the size exchange run on this stream, beside the pushes
        self.side = torch.cuda.Stream()
        self._pending = None
        # host-side planning of the sparse exchanges lives in the library
        ctx = ctypes.c_void_p()
        arenas = (ctypes.c_void_p * world)(*self.peer_base)
        _lib.call("brt_p2p_ctx_create", world, rank, self.base, arenas, self.half_bytes,
                  ctypes.byref(ctx))
        self.ctx = ctx
        self.slot_bytes = int(_lib.query("brt_p2p_ctx_slot_bytes", self.ctx))

    def forward_begin(self, rows: torch.Tensor, sizes: torch.Tensor, group_size: int,
                      grain: int, stride_rows: int) -> None:
        """Enqueue the pushes of a forward sparse exchange on the current stream and its size
        exchange on the side stream (``brt_p2p_forward_begin``)."""
        self._pending = (group_size, sizes)  # keeps the device vector alive
        _lib.call("brt_p2p_forward_begin", self.ctx, rows.data_ptr(), sizes.data_ptr(),
                  group_size, grain, stride_rows, torch.cuda.current_stream().cuda_stream,
                  self.side.cuda_stream)

    def forward_sizes(self):
        """Wait for the size exchange: ([world, world * group] int32 matrix, my output rows,
        whether every rank-to-rank share fits its slot)."""
        group_size, _ = self._pending
        self._pending = None
        matrix = ctypes.POINTER(ctypes.c_int32)()
        rows = ctypes.c_int64()
        fits = ctypes.c_int()
        _lib.call("brt_p2p_forward_sizes", self.ctx, self.side.cuda_stream, ctypes.byref(matrix),
                  ctypes.byref(rows), ctypes.byref(fits))
        n = self.world * group_size
        S = np.ctypeslib.as_array(matrix, shape=(self.world, n)).copy()
        return S, int(rows.value), bool(fits.value)

    def forward_finish(self, rows: torch.Tensor, out: torch.Tensor) -> None:
        _lib.call("brt_p2p_forward_finish", self.ctx, rows.data_ptr(), out.data_ptr(),
                  torch.cuda.current_stream().cuda_stream, self.side.cuda_stream)

    def backward(self, size_matrix: np.ndarray, group_size: int, grain: int, stride_rows: int,
                 rows: torch.Tensor, out: torch.Tensor) -> None:
        """Inverse sparse exchange for the int32 size matrix of the matching forward one."""
        _lib.call("brt_p2p_backward", self.ctx, size_matrix.ctypes.data, group_size, grain,
                  stride_rows, rows.data_ptr(), out.data_ptr(),
                  torch.cuda.current_stream().cuda_stream, self.side.cuda_stream)


_arena: Optional[PeerArena] = None
_disabled_reason: Optional[str] = None
MAX_COPIES = 96


def arena() -> Optional[PeerArena]:
    return _arena


def setup(group, rank: int, world: int) -> Optional[PeerArena]:
    """Create the arena on every rank, or on none: the outcome is agreed by all ranks."""
    global _arena, _disabled_reason
    if _arena is not None or _disabled_reason is not None:
        return _arena
    if os.environ.get("BRT_P2P", "1") == "0":
        _disabled_reason = "BRT_P2P=0"
        return None
    half = int(os.environ.get("BRT_P2P_ARENA_MB", "2048")) << 20
    ok, made, err = 1, None, ""
    try:
        if dist.get_world_size(group) != torch.cuda.device_count() and \
                int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
            raise RuntimeError("ranks span more than one box")
        made = PeerArena(group, rank, world, half)
    except Exception as exc:  # IPC not permitted, out of memory, ...
        ok, err = 0, str(exc)
    flag = torch.tensor([ok], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 1:
        _arena = made
    else:
        _disabled_reason = err or "a peer could not map the arena"
    return _arena


def check_status() -> None:
    """Raise if a bounded wait of an earlier exchange ran out (reads one device word)."""
    if _arena is not None and int(_arena.status.item()) != 0:
        raise RuntimeError("peer exchange timed out waiting for another rank "
                           "(brt_p2p_wait, 2 s limit)")
