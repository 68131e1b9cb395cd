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
# The overlapped size exchange (sizes_begin / sizes_end) alternates between two boards, so a
# rank that is already one exchange ahead cannot overwrite sizes that are still being read.
BOARD2_OFFSET = 2048
BOARD2_INTS = (CONTROL_BYTES - BOARD2_OFFSET) // 8


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
        self.epoch = 0        # value of the arrival flags: one per push
        self.exchanges = 0    # exchanges begun: its parity selects the data half
        self.size_epoch = 0
        self._peer_base_np = np.array(self.peer_base, dtype=np.int64)
        self._size_flag_ptrs = (ctypes.c_void_p * world)(
            *[b + SIZE_FLAGS_OFFSET for b in self.peer_base])
        self._board_ptrs = (ctypes.c_void_p * world)(*[b + BOARD_OFFSET for b in self.peer_base])
        self._flag_ptrs = (ctypes.c_void_p * world)(*[b + FLAGS_OFFSET for b in self.peer_base])
        self._view = torch.as_tensor(_DeviceBytes(self.base, self.total), device="cuda")
        self.status = self._view[STATUS_OFFSET:STATUS_OFFSET + 4].view(torch.int32)
        # overlapped size exchange: own stream, two boards, a pinned landing buffer
        self.side = torch.cuda.Stream()
        self._board2_ptrs = [
            (ctypes.c_void_p * world)(*[b + BOARD2_OFFSET + 4 * k * BOARD2_INTS
                                        for b in self.peer_base]) for k in range(2)]
        self._pinned = torch.empty(1 + BOARD2_INTS, dtype=torch.int32).pin_memory()
        self._pending = None
        # per-source slots of the device-planned push: slot r of a half belongs to rank r
        self.slot_bytes = (self.half_bytes // world) & ~255
        self._slot_ptrs = [
            (ctypes.c_void_p * world)(*[
                None if r == rank else
                self.peer_base[r] + self.half_offset(k) + rank * self.slot_bytes
                for r in range(world)]) for k in range(2)]

    def half_offset(self, exchange: int) -> int:
        return CONTROL_BYTES + (exchange & 1) * self.half_bytes

    def begin_exchange(self) -> int:
        """Start a new exchange: all its pushes write the same data half.  Returns that
        half's byte offset from the arena base."""
        self.exchanges += 1
        return self.half_offset(self.exchanges)

    def gather_sizes(self, sizes: torch.Tensor, stream: int) -> np.ndarray:
        """All ranks' int32 size vectors as a [world, n] host array (one device->host copy,
        which also carries the status word of earlier bounded waits)."""
        n = sizes.numel()
        if self.world * n > BOARD_INTS:
            raise RuntimeError("size vector too long for the peer size board")
        self.size_epoch += 1
        _lib.call("brt_p2p_post", sizes.data_ptr(), n, self.world, self.rank, self.size_epoch,
                  self._board_ptrs, self._size_flag_ptrs, stream)
        _lib.call("brt_p2p_wait", self.base + SIZE_FLAGS_OFFSET, self.world, -1, self.size_epoch,
                  self.base + STATUS_OFFSET, stream)
        words = self._view[STATUS_OFFSET:BOARD_OFFSET + 4 * self.world * n].view(torch.int32)
        host = words.cpu().numpy()
        if host[0] != 0:
            raise RuntimeError("peer exchange timed out waiting for another rank "
                               "(brt_p2p_wait, 2 s limit)")
        return host[1:].reshape(self.world, n)

    def fork_side(self) -> None:
        """Order the side stream behind the work enqueued on the current stream so far."""
        self.side.wait_stream(torch.cuda.current_stream())

    def sizes_begin(self, sizes: torch.Tensor) -> None:
        """Start the size exchange on the arena's side stream (call ``fork_side`` first, at
        the point of the current stream the sizes depend on); work enqueued on the current
        stream in the meantime overlaps it.  ``sizes_end`` returns the [world, n] host array."""
        n = sizes.numel()
        if self.world * n > BOARD2_INTS:
            raise RuntimeError("size vector too long for the peer size board")
        self.size_epoch += 1
        k = self.size_epoch & 1
        _lib.call("brt_p2p_exchange_sizes", sizes.data_ptr(), n, self.world, self.rank,
                  self.size_epoch, self._board2_ptrs[k], self._size_flag_ptrs,
                  self.base + SIZE_FLAGS_OFFSET, self.base + BOARD2_OFFSET + 4 * k * BOARD2_INTS,
                  self.base + STATUS_OFFSET, self._pinned.data_ptr(), self.side.cuda_stream)
        self._pending = (n, sizes)  # keeps the device vector alive until the copy is done

    def sizes_end(self) -> np.ndarray:
        n, _ = self._pending
        self._pending = None
        self.side.synchronize()
        host = self._pinned[:1 + self.world * n].numpy().copy()
        if host[0] != 0:
            raise RuntimeError("peer exchange timed out waiting for another rank "
                               "(brt_p2p_wait, 2 s limit)")
        return host[1:].reshape(self.world, n)

    def push_buckets(self, src: torch.Tensor, sizes: torch.Tensor, group_size: int,
                     grain: int, stride_rows: int, expert_begin: int, expert_end: int,
                     stream: int) -> int:
        """Device-planned push (sizes stay on the device) of my remote buckets of the local
        experts [expert_begin, expert_end) into my slot of every peer's current half; raises
        my data flag everywhere.  Returns the flag epoch to wait for."""
        self.epoch += 1
        e = self.epoch
        _lib.call("brt_p2p_push_buckets", src.data_ptr(), sizes.data_ptr(), self.world,
                  group_size, self.rank, grain, stride_rows, self._slot_ptrs[self.exchanges & 1],
                  self.slot_bytes, expert_begin, expert_end, e, self._flag_ptrs,
                  self.base + COUNTER_OFFSET, stream)
        return e

    def wait_data(self, epoch: int, stream: int) -> None:
        """Wait (bounded) on ``stream`` until every OTHER rank has raised data flag ``epoch``
        in my arena.  My own pushes are ordered by the caller's stream dependencies, never by
        a kernel that spins on a kernel of the same GPU."""
        _lib.call("brt_p2p_wait", self.base + FLAGS_OFFSET, self.world, self.rank, epoch,
                  self.base + STATUS_OFFSET, stream)

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

    def push(self, src: torch.Tensor, src_offsets, dst_ptrs, nbytes, stream: int) -> int:
        """Host-planned push of byte ranges of ``src`` to absolute addresses (see
        ``peer_address``); raises my data flag everywhere.  Returns the flag epoch."""
        self.epoch += 1
        e = self.epoch
        nb = self._i64(nbytes)
        keep = nb > 0
        so = np.ascontiguousarray(self._i64(src_offsets)[keep])
        dp = np.ascontiguousarray(self._i64(dst_ptrs)[keep])
        nb = np.ascontiguousarray(nb[keep])
        if nb.size > MAX_COPIES:
            raise RuntimeError("too many buckets for one peer push")
        _lib.call("brt_p2p_push", src.data_ptr(), int(nb.size), so.ctypes.data, dp.ctypes.data,
                  nb.ctypes.data, self.world, self.rank, e, self._flag_ptrs,
                  self.base + COUNTER_OFFSET, stream)
        return e

    def peer_address(self, ranks, offsets, local_out: int = 0) -> np.ndarray:
        """Absolute addresses of ``offsets`` inside the current half of ``ranks``' arenas;
        ranges addressed to this rank go to ``local_out + offset`` when that is given."""
        ranks = self._i64(ranks)
        offsets = self._i64(offsets)
        dp = self._peer_base_np[ranks] + self.half_offset(self.exchanges) + offsets
        if local_out:
            dp = np.where(ranks == self.rank, local_out + offsets, dp)
        return dp


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
