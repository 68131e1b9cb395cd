"""Host-side bookkeeping of the variable-size expert-parallel exchange.

Pure functions over Python/NumPy integers: bucket offsets and counts for the packed
("sparse") all-to-all, and the send/receive partners of the reorder exchange.  They carry no
device work, so they are also what the CPU multi-process tests exercise.

Layouts (W ranks, G local experts per rank):
  * rank-major   sizes[i*G + j] : bucket for rank i's local expert j  (what a rank sends)
  * expert-major sizes[j*W + i] : bucket of local expert j from rank i (what a rank holds
                                   after the forward exchange)
"""
from typing import List, Sequence, Tuple

import numpy as np


def to_expert_major(recv_rank_major: Sequence[int], world_size: int) -> np.ndarray:
    """[W, G] -> [G, W] relayout the reference applies to the received sizes
    (src/backend/torch/distributed.cc:784)."""
    a = np.asarray(recv_rank_major, dtype=np.int32)
    return np.ascontiguousarray(a.reshape(world_size, -1).T).reshape(-1)


def total_rows(sizes: Sequence[int], stride_rows: int = 0) -> int:
    a = np.asarray(sizes, dtype=np.int64)
    return int(stride_rows) * a.size if stride_rows else int(a.sum())


def bucket_offsets(sizes: Sequence[int], stride_rows: int = 0) -> np.ndarray:
    """Row offset of every bucket of a packed (or stride-padded) buffer, in walk order."""
    a = np.asarray(sizes, dtype=np.int64)
    if stride_rows:
        return np.arange(a.size, dtype=np.int64) * int(stride_rows)
    return np.concatenate(([0], np.cumsum(a)[:-1])) if a.size else a


def exchange_partners(reorder_indices: Sequence[int], world_rank: int) -> Tuple[int, int]:
    """(dst, src) of ``exchange``: I receive from reorder[me] and send to the rank that adopted
    me (src/backend/torch/distributed.cc:78-87); ``reverse_exchange`` swaps the pair."""
    r = [int(x) for x in reorder_indices]
    src = r[world_rank]
    dst = r.index(world_rank)
    return dst, src


def forward_copies(send_rank_major: Sequence[int], recv_expert_major: Sequence[int],
                   world_size: int, stride_rows: int = 0) -> List[Tuple[int, int, int, int]]:
    """The point-to-point operations of the forward exchange as
    (kind, peer, row_offset, rows) with kind 0 = send, 1 = recv, in issue order
    (src/distributed/collective.cc:156-180)."""
    W = world_size
    G = len(send_rank_major) // W
    ops = []
    s_off = bucket_offsets(send_rank_major, stride_rows)
    for i in range(W):
        for j in range(G):
            k = i * G + j
            ops.append((0, i, int(s_off[k]), int(send_rank_major[k])))
    r_off = bucket_offsets(recv_expert_major, stride_rows)
    for j in range(G):
        for i in range(W):
            k = j * W + i
            ops.append((1, i, int(r_off[k]), int(recv_expert_major[k])))
    return ops


def backward_copies(send_expert_major: Sequence[int], recv_rank_major: Sequence[int],
                    world_size: int, stride_rows: int = 0) -> List[Tuple[int, int, int, int]]:
    """Inverse walk (src/distributed/collective.cc:198-222)."""
    W = world_size
    G = len(send_expert_major) // W
    ops = []
    s_off = bucket_offsets(send_expert_major, stride_rows)
    for j in range(G):
        for i in range(W):
            k = j * W + i
            ops.append((0, i, int(s_off[k]), int(send_expert_major[k])))
    r_off = bucket_offsets(recv_rank_major, stride_rows)
    for i in range(W):
        for j in range(G):
            k = i * G + j
            ops.append((1, i, int(r_off[k]), int(recv_rank_major[k])))
    return ops
