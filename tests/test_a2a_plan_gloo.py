"""World-size-2 (and 4) CPU runs of the expert-parallel exchange bookkeeping.

The product moves bytes with NCCL; what is host logic - bucket offsets, walk order, size
relayout, exchange partners - lives in brainstorm_b200/runtime/a2a_plan.py.  Here each rank
executes the plan's point-to-point list over gloo and the result must equal the reference
semantics restated in oracle/ (src/distributed/collective.cc:142-224) and the round trip of
sample/distributed/sparse_a2a.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from brainstorm_b200.runtime import a2a_plan


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ops(ops, send_buf, recv_buf):
    """gloo has no send-to-self: buckets a rank keeps are matched up locally, in issue order
    (NCCL pairs a rank's sends and receives to itself in the same order)."""
    me = dist.get_rank()
    reqs, self_sends, self_recvs = [], [], []
    for kind, peer, off, rows in ops:
        if rows == 0:
            continue
        if peer == me:
            (self_sends if kind == 0 else self_recvs).append((off, rows))
            continue
        if kind == 0:
            reqs.append(dist.P2POp(dist.isend, send_buf[off:off + rows].contiguous(), peer))
        else:
            reqs.append(dist.P2POp(dist.irecv, recv_buf[off:off + rows], peer))
    assert [r for _, r in self_sends] == [r for _, r in self_recvs]
    for (so, n), (ro, _) in zip(self_sends, self_recvs):
        recv_buf[ro:ro + n] = send_buf[so:so + n]
    if reqs:
        for r in dist.batch_isend_irecv(reqs):
            r.wait()


def _worker(rank, world, port, sizes, stride, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        G = len(sizes[0]) // world
        rng = np.random.default_rng(100 + rank)
        send = np.asarray(sizes[rank], dtype=np.int32)
        rows = a2a_plan.total_rows(send, stride)
        x = torch.from_numpy(rng.standard_normal((rows, 3)).astype(np.float32))
        # sizes all-to-all (slice i of send goes to rank i)
        recv_dev = torch.empty(world * G, dtype=torch.int32)
        dist.all_to_all_single(recv_dev, torch.from_numpy(send.copy()))
        recv = a2a_plan.to_expert_major(recv_dev.numpy(), world)
        out = torch.zeros((a2a_plan.total_rows(recv, stride), 3))
        _run_ops(a2a_plan.forward_copies(send, recv, world, stride), x, out)
        back = torch.zeros_like(x)
        _run_ops(a2a_plan.backward_copies(recv, send, world, stride), out, back)
        out_q.put((rank, x.numpy(), out.numpy(), recv, back.numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _launch(world, sizes, stride=0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, sizes, stride, q))
             for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, x, out, recv, back = q.get(timeout=120)
        got[rank] = (x, out, recv, back)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return got


@pytest.mark.parametrize("sizes,stride", [
    # the literal loads of sample/distributed/sparse_a2a.py (2 ranks, 4 buckets per peer)
    ([[3, 2, 4, 4, 2, 4, 5, 2], [1, 22, 3, 4, 3, 55, 222, 1]], 0),
    ([[3, 0, 4, 1], [0, 7, 2, 5]], 0),
    ([[3, 0, 4, 1], [0, 7, 2, 5]], 8),          # max_path_padding stride
])
def test_sparse_exchange_world2(sizes, stride):
    got = _launch(2, sizes, stride)
    xs = [got[r][0] for r in range(2)]
    fwd = oracle.sim_group_sparse_all_to_all(xs, [np.asarray(s, dtype=np.int32) for s in sizes],
                                             bool(stride), stride)
    for r in range(2):
        x, out, recv, back = got[r]
        assert np.array_equal(recv, fwd[r][1])
        if stride == 0:
            assert np.array_equal(out, fwd[r][0])
        else:  # padding rows are unspecified: compare the filled part of every bucket
            for b, n in enumerate(recv):
                assert np.array_equal(out[b * stride:b * stride + n],
                                      fwd[r][0][b * stride:b * stride + n])
        if stride == 0:
            assert np.array_equal(back, x)          # the sample's round-trip assertion
        else:
            send = np.asarray(sizes[r])
            for b, n in enumerate(send):
                assert np.array_equal(back[b * stride:b * stride + n],
                                      x[b * stride:b * stride + n])


def test_sparse_exchange_world4():
    rng = np.random.default_rng(3)
    sizes = [rng.integers(0, 9, size=8).tolist() for _ in range(4)]  # G = 2
    got = _launch(4, sizes)
    xs = [got[r][0] for r in range(4)]
    fwd = oracle.sim_group_sparse_all_to_all(xs, [np.asarray(s, dtype=np.int32) for s in sizes])
    for r in range(4):
        assert np.array_equal(got[r][1], fwd[r][0])
        assert np.array_equal(got[r][3], got[r][0])


def test_plan_arithmetic():
    assert a2a_plan.to_expert_major([1, 2, 3, 4, 5, 6], 3).tolist() == [1, 3, 5, 2, 4, 6]
    assert a2a_plan.bucket_offsets([3, 0, 4]).tolist() == [0, 3, 3]
    assert a2a_plan.bucket_offsets([3, 0, 4], 5).tolist() == [0, 5, 10]
    assert a2a_plan.total_rows([3, 0, 4]) == 7 and a2a_plan.total_rows([3, 0, 4], 5) == 15
    # exchange: I receive from reorder[me], I send to the rank that adopted me
    assert a2a_plan.exchange_partners([2, 0, 1], 0) == (1, 2)
    assert a2a_plan.exchange_partners([2, 0, 1], 1) == (2, 0)
    assert a2a_plan.exchange_partners([0, 1, 2], 2) == (2, 2)
    # reorder produced by the checker is always a permutation, so partners always exist
    m = np.random.default_rng(0).integers(0, 50, size=(8, 8)).astype(np.int32)
    _, idx = oracle.locality_reorder(m, 8)
    assert sorted(idx.tolist()) == list(range(8))
    for me in range(8):
        dst, src = a2a_plan.exchange_partners(idx.tolist(), me)
        assert idx[dst] == me and src == idx[me]
