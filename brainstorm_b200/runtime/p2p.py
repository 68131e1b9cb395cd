"""Arena bookkeeping for the NVLink peer-memory exchange (see csrc/exchange_p2p.cu).

One arena per process: a control block (arrival flags, a completion counter, a status word)
followed by two data halves that alternate from one exchange to the next.  The arena is
exported through CUDA IPC; handles travel between the ranks of the box through
``torch.distributed``.  Only address arithmetic lives here, the copies are done by the
library's kernels.
"""
import ctypes
import os
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib

CONTROL_BYTES = 65536
FLAGS_OFFSET = 0          # 32 x uint64: data arrival flags
SIZE_FLAGS_OFFSET = 256   # 32 x uint64: size-board arrival flags
COUNTER_OFFSET = 512      # uint32
STATUS_OFFSET = 1024      # int32, directly in front of the board so one copy reads both
BOARD_OFFSET = 1028       # int32 [world][n]: bucket sizes posted by every rank
BOARD_INTS = (CONTROL_BYTES - BOARD_OFFSET) // 4


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
        self.epoch = 0
        self.size_epoch = 0
        self._peer_base_np = np.array(self.peer_base, dtype=np.int64)
        self._size_flag_ptrs = (ctypes.c_void_p * world)(
            *[b + SIZE_FLAGS_OFFSET for b in self.peer_base])
        self._board_ptrs = (ctypes.c_void_p * world)(*[b + BOARD_OFFSET for b in self.peer_base])
        self._flag_ptrs = (ctypes.c_void_p * world)(*[b + FLAGS_OFFSET for b in self.peer_base])
        self._view = torch.as_tensor(_DeviceBytes(self.base, self.total), device="cuda")
        self.status = self._view[STATUS_OFFSET:STATUS_OFFSET + 4].view(torch.int32)

    def half_offset(self, epoch: int) -> int:
        return CONTROL_BYTES + (epoch & 1) * self.half_bytes

    def local_bytes(self, epoch: int, nbytes: int) -> torch.Tensor:
        off = self.half_offset(epoch)
        return self._view[off:off + nbytes]

    def gather_sizes(self, sizes: torch.Tensor, stream: int) -> np.ndarray:
        """All ranks' int32 size vectors as a [world, n] host array (one device->host copy,
        which also carries the status word of earlier bounded waits)."""
        n = sizes.numel()
        if self.world * n > BOARD_INTS:
            raise RuntimeError("size vector too long for the peer size board")
        self.size_epoch += 1
        _lib.call("brt_p2p_post", sizes.data_ptr(), n, self.world, self.rank, self.size_epoch,
                  self._board_ptrs, self._size_flag_ptrs, stream)
        _lib.call("brt_p2p_wait", self.base + SIZE_FLAGS_OFFSET, self.world, self.size_epoch,
                  self.base + STATUS_OFFSET, stream)
        words = self._view[STATUS_OFFSET:BOARD_OFFSET + 4 * self.world * n].view(torch.int32)
        host = words.cpu().numpy()
        if host[0] != 0:
            raise RuntimeError("peer exchange timed out waiting for another rank "
                               "(brt_p2p_wait, 2 s limit)")
        return host[1:].reshape(self.world, n)

    @staticmethod
    def _i64(a) -> np.ndarray:
        return np.ascontiguousarray(a, dtype=np.int64)

    def copy_ranges(self, src_base: int, src_offsets, dst_ptrs, nbytes, stream: int) -> None:
        """Local multi-range copy with the push kernel (no flags involved)."""
        nb = self._i64(nbytes)
        keep = nb > 0
        if not keep.any():
            return
        so, dp, nb = self._i64(src_offsets)[keep], self._i64(dst_ptrs)[keep], nb[keep]
        for at in range(0, nb.size, MAX_COPIES):
            a, b, c = (np.ascontiguousarray(v[at:at + MAX_COPIES]) for v in (so, dp, nb))
            _lib.call("brt_p2p_push", src_base, int(c.size), a.ctypes.data, b.ctypes.data,
                      c.ctypes.data, 0, 0, 0, None, None, stream)

    def exchange(self, src: torch.Tensor, src_offsets, dst_ranks, dst_offsets, nbytes,
                 stream: int, local_out: int = 0) -> int:
        """Push byte ranges of ``src`` to ``dst_offsets`` inside the current half of the
        destination ranks' arenas, signal, and wait for every rank's signal.  Ranges addressed
        to this rank go straight to ``local_out + dst_offset`` when ``local_out`` is given.
        Returns the epoch whose half now holds the data that peers sent to this rank."""
        self.epoch += 1
        e = self.epoch
        half = self.half_offset(e)
        nb = self._i64(nbytes)
        ranks = self._i64(dst_ranks)
        dp = self._peer_base_np[ranks] + half + self._i64(dst_offsets)
        if local_out:
            dp = np.where(ranks == self.rank, local_out + self._i64(dst_offsets), dp)
        keep = nb > 0
        so = np.ascontiguousarray(self._i64(src_offsets)[keep])
        dp = np.ascontiguousarray(dp[keep])
        nb = np.ascontiguousarray(nb[keep])
        if nb.size > MAX_COPIES:
            raise RuntimeError("too many buckets for one peer push")
        _lib.call("brt_p2p_push", src.data_ptr(), int(nb.size), so.ctypes.data, dp.ctypes.data,
                  nb.ctypes.data, self.world, self.rank, e, self._flag_ptrs,
                  self.base + COUNTER_OFFSET, stream)
        _lib.call("brt_p2p_wait", self.base + FLAGS_OFFSET, self.world, e,
                  self.base + STATUS_OFFSET, stream)
        return e


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
