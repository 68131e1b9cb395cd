"""The peer-memory sparse exchange with all ranks emulated on ONE GPU.

Each emulated rank has its own arena and its own exchange context; all of them enqueue on one
stream, stage by stage (every rank's post, then every rank's landing kernel, then every
rank's wait), so that each kernel finds the flags it needs already raised by a kernel that
ran before it: nothing ever waits for a kernel enqueued behind it.  The landing kernels, the
device-side planning and the host bookkeeping are exactly those of a real multi-GPU job; the
"peer" pointers simply point into arenas of the same device.  Outputs are compared bit for
bit with the CPU restatement of the reference's walk (src/distributed/collective.cc:142-224).

The last test makes a bounded wait run out on purpose (a rank that never posts) and checks
that the kernels return, that the status says so and that the device keeps working.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from brainstorm_b200 import _lib

pytestmark = pytest.mark.gpu

POST, SIZES, PUSH, WAIT = 1, 2, 4, 8
HALF = 8 << 20


class Ranks:
    """W arenas and contexts on the current device."""

    def __init__(self, world, half=HALF):
        self.world, self.half = world, half
        self.control = int(_lib.query("brt_p2p_control_bytes"))
        self.arenas, self.ctxs = [], []
        for _ in range(world):
            p, h = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
            _lib.call("brt_p2p_alloc", self.control + 2 * half, ctypes.byref(p), h)
            self.arenas.append(p.value)
        table = (ctypes.c_void_p * world)(*self.arenas)
        for r in range(world):
            c = ctypes.c_void_p()
            _lib.call("brt_p2p_ctx_create", world, r, self.arenas[r], table, half,
                      ctypes.byref(c))
            self.ctxs.append(c)

    def close(self):
        torch.cuda.synchronize()
        for c in self.ctxs:
            _lib.query("brt_p2p_ctx_destroy", c)
        for a in self.arenas:
            _lib.call("brt_p2p_free", a)

    def rows_at(self, ptr, rows, cols, dtype=torch.float32):
        nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()

        class Raw:
            __cuda_array_interface__ = {"shape": (max(nbytes, 1),), "typestr": "|u1",
                                        "data": (ptr, False), "version": 2}
        flat = torch.as_tensor(Raw(), device="cuda")[:nbytes]
        return flat.view(dtype).view(rows, cols)

    def forward(self, xs, sizes, group, stride=0, layout=1):
        st = torch.cuda.current_stream().cuda_stream
        grain = xs[0].size(1) * xs[0].element_size()
        for stage in (POST, SIZES, PUSH, WAIT):
            for r in range(self.world):
                _lib.call("brt_p2p_sparse_forward_begin", self.ctxs[r], xs[r].data_ptr(),
                          sizes[r].data_ptr(), group, grain, stride, layout, st, st, stage)
        outs, ids, fit = [], [], []
        for r in range(self.world):
            m = ctypes.POINTER(ctypes.c_int32)()
            n_rows, fits = ctypes.c_int64(), ctypes.c_int()
            out, xid = ctypes.c_void_p(), ctypes.c_uint64()
            _lib.call("brt_p2p_sparse_forward_sizes", self.ctxs[r], st, ctypes.byref(m),
                      ctypes.byref(n_rows), ctypes.byref(fits), ctypes.byref(out),
                      ctypes.byref(xid))
            S = np.ctypeslib.as_array(m, shape=(self.world, self.world * group)).copy()
            outs.append((out.value, n_rows.value, S))
            ids.append(xid.value)
            fit.append(bool(fits.value))
        return outs, ids, fit

    def backward(self, ids, xs, group, stride=0, layout=0, zero_tails=0):
        st = torch.cuda.current_stream().cuda_stream
        grain = xs[0].size(1) * xs[0].element_size()
        res = [None] * self.world
        for stage in (POST, PUSH, WAIT):
            for r in range(self.world):
                out, n_rows = ctypes.c_void_p(), ctypes.c_int64()
                _lib.call("brt_p2p_sparse_backward", self.ctxs[r], ids[r], group, grain, stride,
                          layout, zero_tails, xs[r].data_ptr(), st, stage, ctypes.byref(out),
                          ctypes.byref(n_rows))
                res[r] = (out.value, n_rows.value)
        return res


def make_inputs(world, group, cols, hi, stride, seed):
    rng = np.random.default_rng(seed)
    xs, sizes = [], []
    for _ in range(world):
        s = rng.integers(0, hi, size=world * group).astype(np.int32)
        if rng.random() < 0.3:
            s[rng.integers(0, s.size)] = 0
        rows = stride * world * group if stride else int(s.sum())
        xs.append(rng.standard_normal((rows, cols)).astype(np.float32))
        sizes.append(s)
    return xs, sizes


CASES = [
    # world, group, cols (fp32), largest bucket, stride
    (2, 1, 4, 40, 0), (2, 4, 8, 30, 0), (4, 2, 16, 25, 0), (4, 5, 12, 9, 0),
    (8, 8, 64, 200, 0), (8, 16, 4, 6, 0), (3, 7, 8, 11, 0), (8, 32, 4, 5, 0),
    (2, 2, 4, 17, 16), (4, 3, 8, 11, 10), (8, 4, 4, 8, 7), (2, 128, 4, 3, 0),
]


@pytest.mark.parametrize("world,group,cols,hi,stride", CASES)
def test_forward_and_back(world, group, cols, hi, stride):
    dev = torch.device("cuda", 0)
    xs_np, sizes_np = make_inputs(world, group, cols, hi if not stride else stride + 1, stride,
                                  seed=world * 1000 + group)
    sim = oracle.sim_group_sparse_all_to_all(xs_np, sizes_np, bool(stride), stride)
    ranks = Ranks(world)
    try:
        xs = [torch.from_numpy(x).to(dev) for x in xs_np]
        sizes = [torch.from_numpy(s).to(dev) for s in sizes_np]
        for repeat in range(3):  # both landing halves, and a half that is reused
            outs, ids, fit = ranks.forward(xs, sizes, group, stride)
            assert all(fit)
            landed = []
            for r in range(world):
                ptr, rows, S = outs[r]
                assert rows == sim[r][0].shape[0]
                assert np.array_equal(S, np.stack(sizes_np)), "size matrix differs"
                got = ranks.rows_at(ptr, rows, cols)
                landed.append(got)
                want = sim[r][0]
                g = got.cpu().numpy()
                if stride:
                    for b, n in enumerate(sim[r][1]):
                        assert np.array_equal(g[b * stride:b * stride + n],
                                              want[b * stride:b * stride + n]), (r, b)
                else:
                    assert np.array_equal(g, want), f"rank {r}: forward rows differ"
            back = ranks.backward(ids, landed, group, stride)
            for r in range(world):
                ptr, rows = back[r]
                assert rows == xs_np[r].shape[0]
                g = ranks.rows_at(ptr, rows, cols).cpu().numpy()
                if stride:
                    for b, n in enumerate(sizes_np[r]):
                        assert np.array_equal(g[b * stride:b * stride + n],
                                              xs_np[r][b * stride:b * stride + n]), (r, b)
                else:
                    assert np.array_equal(g, xs_np[r]), f"rank {r}: round trip differs"
        for c in ranks.ctxs:
            assert _lib.query("brt_p2p_ctx_status", c) == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("world,group,cols,slot", [(2, 1, 4, 9), (4, 2, 8, 12), (8, 4, 4, 6),
                                                   (3, 5, 16, 7)])
def test_padded_slot_exchange_and_back(world, group, cols, slot):
    """group_asymmetry_all_to_all and its size-known inverse (src/distributed/collective.cc:
    108-140): slot (i, j) of rank s lands in slot (s, j) of rank i; on the way back the rows
    beyond a slot's size come back as zeros."""
    dev = torch.device("cuda", 0)
    n = world * group
    rng = np.random.default_rng(40 + world + group)
    xs_np = [rng.standard_normal((slot * n, cols)).astype(np.float32) for _ in range(world)]
    sizes_np = [rng.integers(0, slot + 1, size=n).astype(np.int32) for _ in range(world)]
    sim = oracle.sim_group_asymmetry_all_to_all(xs_np, sizes_np)
    ranks = Ranks(world)
    try:
        xs = [torch.from_numpy(x).to(dev) for x in xs_np]
        sizes = [torch.from_numpy(s).to(dev) for s in sizes_np]
        for repeat in range(2):
            outs, ids, fit = ranks.forward(xs, sizes, group, slot, layout=2)
            assert all(fit)
            landed = []
            for r in range(world):
                ptr, rows, _ = outs[r]
                assert rows == slot * n
                got = ranks.rows_at(ptr, rows, cols)
                landed.append(got)
                g = got.cpu().numpy()
                for b, cnt in enumerate(sim[r][1]):
                    assert np.array_equal(g[b * slot:b * slot + cnt],
                                          sim[r][0][b * slot:b * slot + cnt]), (r, b)
            back = ranks.backward(ids, landed, group, slot, layout=3, zero_tails=1)
            for r in range(world):
                g = ranks.rows_at(back[r][0], back[r][1], cols).cpu().numpy()
                for b, cnt in enumerate(sizes_np[r]):
                    assert np.array_equal(g[b * slot:b * slot + cnt],
                                          xs_np[r][b * slot:b * slot + cnt]), (r, b)
                    assert not g[b * slot + cnt:(b + 1) * slot].any(), (r, b)
    finally:
        ranks.close()


    # (method of Ranks, bound below)
def _dispatch_forward(self, xs, idxs, loads, counts, group, stride=0):
    st = torch.cuda.current_stream().cuda_stream
    grain = xs[0].size(1) * xs[0].element_size()
    for stage in (POST, SIZES, PUSH, WAIT):
        for r in range(self.world):
            _lib.call("brt_p2p_dispatch_forward_begin", self.ctxs[r], xs[r].data_ptr(),
                      idxs[r].data_ptr(), loads[r].data_ptr(), counts[r].data_ptr(),
                      xs[r].size(0), grain, group, stride, st, st, stage)
    outs = []
    for r in range(self.world):
        m = ctypes.POINTER(ctypes.c_int32)()
        n_rows, fits = ctypes.c_int64(), ctypes.c_int()
        out, xid = ctypes.c_void_p(), ctypes.c_uint64()
        _lib.call("brt_p2p_sparse_forward_sizes", self.ctxs[r], st, ctypes.byref(m),
                  ctypes.byref(n_rows), ctypes.byref(fits), ctypes.byref(out), ctypes.byref(xid))
        assert fits.value
        outs.append((out.value, n_rows.value))
    return outs


Ranks.dispatch_forward = _dispatch_forward


@pytest.mark.parametrize("world,group,cells,cols,k,mode", [
    (2, 2, 300, 4, 2, "packed"), (4, 2, 257, 8, 2, "packed"), (8, 4, 500, 1024, 2, "packed"),
    (2, 4, 640, 600, 1, "packed"), (4, 1, 300, 16, 1, "padded"), (8, 2, 400, 520, 2, "padded"),
    (2, 3, 200, 4, 2, "capacity"), (4, 4, 900, 12, 3, "capacity"), (8, 8, 1000, 2048, 2, "packed"),
])
def test_dispatch_fused_with_the_forward_exchange(world, group, cells, cols, k, mode):
    """Dispatch that stores its rows straight into the destinations' landing halves equals
    dispatch followed by the exchange (the checker's dispatch, then its walk of the exchange),
    bit for bit: packed buckets, padded buckets, and loads padded above the cell counts (rows
    that must arrive as zeros).  The indices come from the library's index ops, as in the
    fabrics."""
    from brainstorm_b200._C import router as R

    dev = torch.device("cuda", 0)
    E = world * group
    rng = np.random.default_rng(world * 100 + group * 10 + cells)
    xs_np, rows_np, sizes_np = [], [], []
    xs, idxs, loads, counts = [], [], [], []
    per_path = max(1, cells * k // E)
    stride = 0
    for r in range(world):
        mask = oracle.topk_hot_mask(rng.standard_normal((cells, E)).astype(np.float32), k)
        x = rng.standard_normal((cells, cols)).astype(np.float32)
        caps = cpad = None
        if mode == "padded":
            stride = 2 * per_path
            thr = np.full(E, stride, dtype=np.int32)
            m_np, _ = oracle.throttle_hotmask(mask, np.zeros(E, dtype=np.int32), thr)
            i_np, l_np = oracle.generate_indices_and_loads(m_np)
            i_t, l_t, _ = R.throttle_and_generate_indices(
                torch.from_numpy(mask).to(dev), torch.zeros(E, dtype=torch.int32, device=dev),
                torch.from_numpy(thr).to(dev))
        else:
            if mode == "capacity":
                caps, cpad = [per_path // 2 + 1, 2 * per_path, 16 * per_path], True
            i_np, l_np = oracle.generate_indices_and_loads(mask, caps, bool(cpad))
            i_t, l_t = R.generate_indices_and_loads(
                torch.from_numpy(mask).to(dev),
                None if caps is None else torch.tensor(caps, dtype=torch.int32, device=dev),
                bool(cpad))
        assert np.array_equal(i_t.cpu().numpy(), i_np)
        (routed,) = oracle.dispatch_with_indices_and_loads(
            x, i_np, l_np, max_path_padding=bool(stride), max_path_load=stride)
        xs_np.append(x)
        rows_np.append(routed)
        sizes_np.append(l_np)
        xs.append(torch.from_numpy(x).to(dev))
        idxs.append(i_t)
        loads.append(l_t.contiguous())
        counts.append(getattr(i_t, R._DENSE))
    sim = oracle.sim_group_sparse_all_to_all(rows_np, sizes_np, bool(stride), stride)
    ranks = Ranks(world, half=32 << 20)
    try:
        for repeat in range(2):
            # NaN in the landing halves first: rows the kernel must write show if it does not
            for r in range(world):
                ranks.rows_at(ranks.arenas[r] + ranks.control, 2 * ranks.half // 4, 1).fill_(
                    float("nan"))
            outs = ranks.dispatch_forward(xs, idxs, loads, counts, group, stride)
            for r in range(world):
                ptr, rows = outs[r]
                want = sim[r][0]
                assert rows == want.shape[0]
                g = ranks.rows_at(ptr, rows, cols).cpu().numpy()
                if stride:
                    for b, cnt in enumerate(sim[r][1]):
                        assert np.array_equal(g[b * stride:b * stride + cnt],
                                              want[b * stride:b * stride + cnt]), (r, b)
                else:
                    assert np.array_equal(g, want), f"rank {r}: landed rows differ"
    finally:
        ranks.close()


def test_nested_forwards_then_inverses():
    """Two forward exchanges whose inverses come in reverse order (layer 1, layer 2, back 2,
    back 1), with one rank sending the same sizes in both: each inverse must use the matrix
    of its own forward exchange."""
    dev = torch.device("cuda", 0)
    world, group, cols = 4, 2, 8
    a_np, sa_np = make_inputs(world, group, cols, 20, 0, seed=1)
    b_np, sb_np = make_inputs(world, group, cols, 20, 0, seed=2)
    sb_np[1] = sa_np[1].copy()  # rank 1 sends the same sizes in both exchanges
    b_np[1] = np.random.default_rng(3).standard_normal(a_np[1].shape).astype(np.float32)
    ranks = Ranks(world)
    try:
        to = lambda arrs: [torch.from_numpy(a).to(dev) for a in arrs]
        a, sa, b, sb = to(a_np), to(sa_np), to(b_np), to(sb_np)
        outs_a, ids_a, _ = ranks.forward(a, sa, group)
        kept_a = [ranks.rows_at(p, n, cols).clone() for p, n, _ in outs_a]
        outs_b, ids_b, _ = ranks.forward(b, sb, group)
        kept_b = [ranks.rows_at(p, n, cols).clone() for p, n, _ in outs_b]
        back_b = ranks.backward(ids_b, kept_b, group)
        for r in range(world):
            assert np.array_equal(ranks.rows_at(*back_b[r], cols).cpu().numpy(), b_np[r])
        back_a = ranks.backward(ids_a, kept_a, group)
        for r in range(world):
            assert np.array_equal(ranks.rows_at(*back_a[r], cols).cpu().numpy(), a_np[r])
    finally:
        ranks.close()


def test_rows_that_do_not_fit_are_left_alone():
    dev = torch.device("cuda", 0)
    world, group, cols = 2, 1, 1024
    ranks = Ranks(world, half=1 << 16)  # 64 KB halves, 4 KB rows
    try:
        sizes_np = [np.array([10, 30], dtype=np.int32), np.array([5, 2], dtype=np.int32)]
        xs = [torch.zeros((int(s.sum()), cols), device=dev) for s in sizes_np]
        sizes = [torch.from_numpy(s).to(dev) for s in sizes_np]
        outs, ids, fit = ranks.forward(xs, sizes, group)
        assert fit == [False, False]  # rank 1 would receive 32 rows = 128 KB
        with pytest.raises(_lib.BrtError) as err:  # 40 rows go back to rank 0: too many as well
            ranks.backward(ids, xs, group)
        assert err.value.status == 4
    finally:
        ranks.close()


def test_wait_runs_out_and_is_reported():
    """Rank 1 never enters the exchange: rank 0's kernels give up after the (shortened)
    limit, copy nothing, and both the call that reads the sizes and the status query say so."""
    dev = torch.device("cuda", 0)
    ranks = Ranks(2)
    try:
        _lib.call("brt_p2p_ctx_set_wait_limit", ranks.ctxs[0], 20_000_000)  # 20 ms
        x = torch.ones((8, 4), device=dev)
        sizes = torch.tensor([3, 5], dtype=torch.int32, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[0], x.data_ptr(), sizes.data_ptr(),
                  1, 16, 0, 1, st, st, 0)
        m = ctypes.POINTER(ctypes.c_int32)()
        n_rows, fits = ctypes.c_int64(), ctypes.c_int()
        out, xid = ctypes.c_void_p(), ctypes.c_uint64()
        with pytest.raises(_lib.BrtError) as err:
            _lib.call("brt_p2p_sparse_forward_sizes", ranks.ctxs[0], st, ctypes.byref(m),
                      ctypes.byref(n_rows), ctypes.byref(fits), ctypes.byref(out),
                      ctypes.byref(xid))
        assert err.value.status == 7  # BRT_ERR_TIMEOUT
        torch.cuda.synchronize()  # every kernel of the exchange has returned
        assert _lib.query("brt_p2p_ctx_status", ranks.ctxs[0]) == 7
        with pytest.raises(_lib.BrtError):  # refused until the status is cleared
            _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[0], x.data_ptr(),
                      sizes.data_ptr(), 1, 16, 0, 1, st, st, 0)
        # nothing landed in rank 1's arena and the device still answers
        landing = ranks.rows_at(ranks.arenas[1] + ranks.control + ranks.half, 8, 4)  # exchange 1: half 1
        assert float(landing.abs().sum()) == 0.0
        assert float((x * 2).sum()) == 64.0
        for c in ranks.ctxs:  # every rank resets; then the exchanges work again
            _lib.call("brt_p2p_ctx_reset_status", c)
        assert _lib.query("brt_p2p_ctx_status", ranks.ctxs[0]) == 0
        _lib.call("brt_p2p_ctx_set_wait_limit", ranks.ctxs[0], 2_000_000_000)
        xs_np, sizes_np = make_inputs(2, 1, 4, 9, 0, seed=77)
        sim = oracle.sim_group_sparse_all_to_all(xs_np, sizes_np, False, 0)
        outs, ids, fit = ranks.forward([torch.from_numpy(a).to(dev) for a in xs_np],
                                       [torch.from_numpy(s).to(dev) for s in sizes_np], 1)
        assert all(fit)
        for r in range(2):
            assert np.array_equal(ranks.rows_at(outs[r][0], outs[r][1], 4).cpu().numpy(),
                                  sim[r][0])
    finally:
        ranks.close()


STRICT = 16


def _section(ranks, xs, sizes, group, cols, expert=None, stride=0, fused=None):
    """One replay section on every emulated rank: forward exchange with device-resident
    sizes, an optional per-rank transform of the landed rows, the inverse exchange.  Returns
    (received sizes per rank, landed rows per rank (clones), returned rows per rank).
    ``fused`` = (index tensors, dense counts): the forward exchange is the dispatch that lands
    its rows itself, ``xs`` are then the cells."""
    st = torch.cuda.current_stream().cuda_stream
    world = ranks.world
    grain = cols * 4
    for c in ranks.ctxs:
        _lib.call("brt_p2p_ctx_replay_begin", c)
    for stage in (POST, PUSH | STRICT, WAIT):
        for r in range(world):
            if fused is not None:
                _lib.call("brt_p2p_dispatch_forward_begin", ranks.ctxs[r], xs[r].data_ptr(),
                          fused[0][r].data_ptr(), sizes[r].data_ptr(), fused[1][r].data_ptr(),
                          xs[r].size(0), grain, group, stride, st, st, stage)
            else:
                _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[r], xs[r].data_ptr(),
                          sizes[r].data_ptr(), group, grain, stride, 1, st, st, stage)
    received, landed, ids = [], [], []
    for r in range(world):
        got = torch.empty((group * world,), dtype=torch.int32, device="cuda")
        out, cap, xid = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_uint64()
        _lib.call("brt_p2p_forward_device_sizes", ranks.ctxs[r], got.data_ptr(), st,
                  ctypes.byref(out), ctypes.byref(cap), ctypes.byref(xid))
        assert cap.value == (stride * world * group if stride else ranks.half // grain)
        received.append(got)
        landed.append(ranks.rows_at(out.value, cap.value, cols))
        ids.append(xid.value)
    sources = [expert(t) if expert else t for t in landed]
    back = [None] * world
    for stage in (POST, PUSH, WAIT):
        for r in range(world):
            out, n_rows = ctypes.c_void_p(), ctypes.c_int64()
            _lib.call("brt_p2p_sparse_backward", ranks.ctxs[r], ids[r], group, grain, stride, 0,
                      0, sources[r].data_ptr(), st, stage, ctypes.byref(out),
                      ctypes.byref(n_rows))
            back[r] = ranks.rows_at(out.value, n_rows.value, cols)
    for c in ranks.ctxs:
        _lib.call("brt_p2p_ctx_replay_end", c)
    return received, landed, back


@pytest.mark.parametrize("world,group,cols", [(2, 2, 4), (4, 3, 8), (8, 4, 16)])
def test_replay_sections_with_device_resident_sizes(world, group, cols):
    """Sections of forward + inverse exchange whose sizes never reach the host, issued again
    and again with new data (what replaying a captured graph does: the epoch is counted on
    the device), with ordinary exchanges in between.  Everything is compared
    with the checker's walk of the exchange."""
    dev = torch.device("cuda", 0)
    ranks = Ranks(world)
    try:
        # fixed buffers, as under a CUDA graph: new contents are copied into them
        bound = 40 * world * group
        xs = [torch.zeros((bound, cols), device=dev) for _ in range(world)]
        sizes = [torch.zeros((world * group,), dtype=torch.int32, device=dev)
                 for _ in range(world)]
        for it in range(5):
            xs_np, sizes_np = make_inputs(world, group, cols, 40, 0, seed=900 + it)
            sim = oracle.sim_group_sparse_all_to_all(xs_np, sizes_np, False, 0)
            for r in range(world):
                xs[r].zero_()
                xs[r][:xs_np[r].shape[0]].copy_(torch.from_numpy(xs_np[r]))
                sizes[r].copy_(torch.from_numpy(sizes_np[r]))
            if it == 3:
                # an ordinary exchange between two sections: its epoch continues theirs
                tx = [torch.from_numpy(x).to(dev) for x in xs_np]
                outs, ids, fit = ranks.forward(tx, sizes, group)
                assert all(fit)
                held = [ranks.rows_at(p, n, cols).clone() for p, n, _ in outs]
                for r in range(world):
                    assert np.array_equal(held[r].cpu().numpy(), sim[r][0])
                back = ranks.backward(ids, held, group)
                for r in range(world):
                    assert np.array_equal(ranks.rows_at(*back[r], cols).cpu().numpy(), xs_np[r])
                continue
            received, landed, back = _section(ranks, xs, sizes, group, cols)
            torch.cuda.synchronize()
            for r in range(world):
                want_rows, want_sizes = sim[r][0], sim[r][1]
                assert np.array_equal(received[r].cpu().numpy(), want_sizes.reshape(-1)), \
                    f"iteration {it}, rank {r}: received sizes differ"
                n = want_rows.shape[0]
                assert np.array_equal(landed[r][:n].cpu().numpy(), want_rows), \
                    f"iteration {it}, rank {r}: landed rows differ"
                m = xs_np[r].shape[0]
                assert np.array_equal(back[r][:m].cpu().numpy(), xs_np[r]), \
                    f"iteration {it}, rank {r}: round trip differs"
        for c in ranks.ctxs:
            assert _lib.query("brt_p2p_ctx_status", c) == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("world,group,cells,cols,mode", [(2, 2, 300, 8, "packed"),
                                                         (4, 2, 400, 512, "padded"),
                                                         (8, 4, 700, 16, "capacity")])
def test_replay_sections_with_the_fused_dispatch(world, group, cells, cols, mode):
    """The section of a routing step as the distributed fabric issues it with
    ``device_sizes``: dispatch that lands its rows itself, sizes on the device, inverse
    exchange; packed buckets, padded buckets (a slot size) and loads padded above the cell
    counts.  Issued three times with new cells and new picks."""
    from brainstorm_b200._C import router as R

    dev = torch.device("cuda", 0)
    E = world * group
    per_path = max(1, cells * 2 // E)
    stride = 2 * per_path if mode == "padded" else 0
    ranks = Ranks(world, half=32 << 20)
    try:
        for it in range(3):
            rng = np.random.default_rng(7000 + 10 * it + world)
            xs, idxs, loads, counts, xs_np, rows_np, sizes_np = [], [], [], [], [], [], []
            for r in range(world):
                mask = oracle.topk_hot_mask(rng.standard_normal((cells, E)).astype(np.float32), 2)
                x = rng.standard_normal((cells, cols)).astype(np.float32)
                if mode == "padded":
                    thr = np.full(E, stride, dtype=np.int32)
                    m_np, _ = oracle.throttle_hotmask(mask, np.zeros(E, dtype=np.int32), thr)
                    i_np, l_np = oracle.generate_indices_and_loads(m_np)
                    i_t, l_t, _ = R.throttle_and_generate_indices(
                        torch.from_numpy(mask).to(dev),
                        torch.zeros(E, dtype=torch.int32, device=dev),
                        torch.from_numpy(thr).to(dev))
                else:
                    caps = [per_path // 2 + 1, 2 * per_path, 16 * per_path] \
                        if mode == "capacity" else None
                    i_np, l_np = oracle.generate_indices_and_loads(mask, caps, caps is not None)
                    i_t, l_t = R.generate_indices_and_loads(
                        torch.from_numpy(mask).to(dev),
                        None if caps is None else torch.tensor(caps, dtype=torch.int32,
                                                               device=dev),
                        caps is not None)
                (routed,) = oracle.dispatch_with_indices_and_loads(
                    x, i_np, l_np, max_path_padding=bool(stride), max_path_load=stride)
                xs_np.append(x)
                rows_np.append(routed)
                sizes_np.append(l_np)
                xs.append(torch.from_numpy(x).to(dev))
                idxs.append(i_t)
                loads.append(l_t.contiguous())
                counts.append(getattr(i_t, R._DENSE))
            sim = oracle.sim_group_sparse_all_to_all(rows_np, sizes_np, bool(stride), stride)
            received, landed, back = _section(ranks, xs, loads, group, cols, stride=stride,
                                              fused=(idxs, counts))
            torch.cuda.synchronize()
            for r in range(world):
                want, want_sizes = sim[r][0], np.asarray(sim[r][1]).reshape(-1)
                assert np.array_equal(received[r].cpu().numpy(), want_sizes), (it, r)
                g = landed[r].cpu().numpy()
                b = back[r].cpu().numpy()
                if stride:
                    for k, cnt in enumerate(want_sizes):
                        assert np.array_equal(g[k * stride:k * stride + cnt],
                                              want[k * stride:k * stride + cnt]), (it, r, k)
                    for k, cnt in enumerate(sizes_np[r]):
                        assert np.array_equal(b[k * stride:k * stride + cnt],
                                              rows_np[r][k * stride:k * stride + cnt]), (it, r, k)
                else:
                    assert np.array_equal(g[:want.shape[0]], want), (it, r)
                    assert np.array_equal(b[:rows_np[r].shape[0]], rows_np[r]), (it, r)
        for c in ranks.ctxs:
            assert _lib.query("brt_p2p_ctx_status", c) == 0
    finally:
        ranks.close()


def test_replay_section_rules_and_rows_that_do_not_fit():
    dev = torch.device("cuda", 0)
    world, group, cols = 2, 1, 1024
    ranks = Ranks(world, half=1 << 16)  # 64 KB halves, 4 KB rows
    st = torch.cuda.current_stream().cuda_stream
    try:
        sizes_np = [np.array([10, 30], dtype=np.int32), np.array([5, 2], dtype=np.int32)]
        xs = [torch.ones((int(s.sum()), cols), device=dev) for s in sizes_np]
        sizes = [torch.from_numpy(s).to(dev) for s in sizes_np]
        # the host-size stage is refused inside a section
        _lib.call("brt_p2p_ctx_replay_begin", ranks.ctxs[0])
        with pytest.raises(_lib.BrtError):
            _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[0], xs[0].data_ptr(),
                      sizes[0].data_ptr(), group, cols * 4, 0, 1, st, st, 0)
        _lib.call("brt_p2p_ctx_replay_end", ranks.ctxs[0])  # empty section: fine
        # sizes that were never sent to the host cannot be read there
        _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[0], xs[0].data_ptr(),
                  sizes[0].data_ptr(), group, cols * 4, 0, 1, st, st, POST)
        with pytest.raises(_lib.BrtError):
            m = ctypes.POINTER(ctypes.c_int32)()
            n_rows, fits = ctypes.c_int64(), ctypes.c_int()
            out, xid = ctypes.c_void_p(), ctypes.c_uint64()
            _lib.call("brt_p2p_sparse_forward_sizes", ranks.ctxs[0], st, ctypes.byref(m),
                      ctypes.byref(n_rows), ctypes.byref(fits), ctypes.byref(out),
                      ctypes.byref(xid))
        torch.cuda.synchronize()
        for c in ranks.ctxs:  # rank 0 alone posted an exchange: start over
            _lib.call("brt_p2p_ctx_reset_status", c)
        with pytest.raises(_lib.BrtError):
            _lib.call("brt_p2p_ctx_replay_end", ranks.ctxs[0])  # none open
        # rank 1 would receive 32 rows = 128 KB: nothing moves, and the status says why
        for c in ranks.ctxs:
            _lib.call("brt_p2p_ctx_replay_begin", c)
        for stage in (POST, PUSH | STRICT, WAIT):
            for r in range(world):
                _lib.call("brt_p2p_sparse_forward_begin", ranks.ctxs[r], xs[r].data_ptr(),
                          sizes[r].data_ptr(), group, cols * 4, 0, 1, st, st, stage)
        landed = []
        for r in range(world):
            got = torch.empty((group * world,), dtype=torch.int32, device=dev)
            out, cap, xid = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_uint64()
            _lib.call("brt_p2p_forward_device_sizes", ranks.ctxs[r], got.data_ptr(), st,
                      ctypes.byref(out), ctypes.byref(cap), ctypes.byref(xid))
            landed.append(ranks.rows_at(out.value, cap.value, cols))
        for c in ranks.ctxs:
            _lib.call("brt_p2p_ctx_replay_end", c)
        torch.cuda.synchronize()
        assert [_lib.query("brt_p2p_ctx_status", c) for c in ranks.ctxs] == [4, 4]
        assert float(landed[1].abs().sum()) == 0.0
        with pytest.raises(_lib.BrtError) as err:  # refused until the status is cleared
            _lib.call("brt_p2p_ctx_replay_begin", ranks.ctxs[0])
        assert err.value.status == 4
        assert float((xs[0] * 2).sum()) == 2.0 * xs[0].numel()  # the device still answers
    finally:
        ranks.close()


@pytest.mark.parametrize("world,group,cells,cols,k,mode,dtype,gated", [
    (2, 2, 300, 8, 2, "packed", "f32", True), (4, 2, 257, 8, 2, "packed", "f32", False),
    (8, 4, 500, 1024, 2, "packed", "bf16", True), (2, 4, 640, 600, 1, "packed", "f32", True),
    (4, 1, 300, 16, 1, "padded", "f32", True), (8, 2, 400, 520, 2, "padded", "f32", True),
    (2, 3, 200, 4, 2, "capacity", "f32", True), (4, 4, 900, 16, 3, "capacity", "f32", True),
    (4, 2, 333, 64, 4, "packed", "bf16", True),
])
def test_combine_that_pulls_from_the_peers(world, group, cells, cols, k, mode, dtype, gated):
    """Inverse exchange and weighted combine as one kernel: the cells come out as from the
    checker's inverse walk of the exchange followed by its combine, bit for bit (fp32) or
    within one rounding of the checker's bf16 arithmetic.  The experts multiply the landed rows
    in place by a factor of their rank; k = 3 and 4 exercise the routes beyond the two staged
    ones."""
    from brainstorm_b200._C import router as R

    dev = torch.device("cuda", 0)
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    E = world * group
    rng = np.random.default_rng(world * 131 + group * 17 + cells)
    per_path = max(1, cells * k // E)
    stride = 2 * per_path if mode == "padded" else 0
    xs, idxs, loads, counts, gates = [], [], [], [], []
    idx_np, loads_np, gates_np, rows_np = [], [], [], []
    for r in range(world):
        score = rng.standard_normal((cells, E)).astype(np.float32)
        mask = oracle.topk_hot_mask(score, k)
        x = rng.standard_normal((cells, cols)).astype(np.float32)
        if dtype == "bf16":
            x = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x))
        if mode == "padded":
            thr = np.full(E, stride, dtype=np.int32)
            m_np, _ = oracle.throttle_hotmask(mask, np.zeros(E, dtype=np.int32), thr)
            i_np, l_np = oracle.generate_indices_and_loads(m_np)
            i_t, l_t, _ = R.throttle_and_generate_indices(
                torch.from_numpy(mask).to(dev), torch.zeros(E, dtype=torch.int32, device=dev),
                torch.from_numpy(thr).to(dev))
        else:
            caps = [per_path // 2 + 1, 2 * per_path, 16 * per_path] if mode == "capacity" else None
            i_np, l_np = oracle.generate_indices_and_loads(mask, caps, caps is not None)
            i_t, l_t = R.generate_indices_and_loads(
                torch.from_numpy(mask).to(dev),
                None if caps is None else torch.tensor(caps, dtype=torch.int32, device=dev),
                caps is not None)
        g_np = np.abs(score) + 0.25
        (routed,) = oracle.dispatch_with_indices_and_loads(
            x, i_np, l_np, max_path_padding=bool(stride), max_path_load=stride)
        xs.append(torch.from_numpy(x).to(dev).to(tdt))
        idxs.append(i_t)
        loads.append(l_t.contiguous())
        counts.append(getattr(i_t, R._DENSE))
        gates.append(torch.from_numpy(g_np).to(dev))
        idx_np.append(i_np)
        loads_np.append(l_np)
        gates_np.append(g_np)
        rows_np.append(routed)
    fwd = oracle.sim_group_sparse_all_to_all(rows_np, loads_np, bool(stride), stride)
    # the experts: every row on rank r is multiplied by r + 2 (exact in bf16 up to one rounding)
    expert_out = []
    for r in range(world):
        y = fwd[r][0] * np.float32(r + 2)
        if dtype == "bf16":
            y = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(y))
        expert_out.append(y)
    back = oracle.sim_size_known_group_sparse_all_to_all(
        expert_out, [f[1] for f in fwd], loads_np, bool(stride))
    ranks = Ranks(world, half=32 << 20)
    st = torch.cuda.current_stream().cuda_stream
    grain = cols * (4 if dtype == "f32" else 2)
    dt_code = 0 if dtype == "f32" else 2
    try:
        for repeat in range(2):
            outs = ranks.dispatch_forward(xs, idxs, loads, counts, group, stride)
            ids = [int(_lib.query("brt_p2p_ctx_exchanges", c)) for c in ranks.ctxs]
            offsets = []
            for r in range(world):
                ptr, n_rows = outs[r]
                ranks.rows_at(ptr, n_rows, cols, tdt).mul_(r + 2)
                offsets.append(ptr - ranks.arenas[r])
            assert len(set(offsets)) == 1
            results = [torch.full((cells, cols), float("nan"), dtype=tdt, device=dev)
                       for _ in range(world)]
            for stage in (POST, PUSH, WAIT):
                for r in range(world):
                    _lib.call("brt_p2p_combine_backward", ranks.ctxs[r], ids[r], group, grain,
                              stride, offsets[r], idxs[r].data_ptr(),
                              gates[r].data_ptr() if gated else None, 0, dt_code, cells,
                              results[r].data_ptr(), st, stage)
            torch.cuda.synchronize()
            for r in range(world):
                (want,) = oracle.combine_with_indices_and_loads(
                    oracle.to_bits(back[r], dtype), idx_np[r], loads_np[r],
                    gates_np[r] if gated else None, None, bool(stride), dtype=dtype)
                want = oracle.from_bits(want, dtype)
                got = results[r].float().cpu().numpy()
                assert np.array_equal(got, want), \
                    f"rank {r}: {np.abs(got - want).max()} off the checker's combine"
        for c in ranks.ctxs:
            assert _lib.query("brt_p2p_ctx_status", c) == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("world,group,cells,cols,dtype,gate_kind", [
    (3, 1, [5, 0, 1], 8, "f32", "f32"),       # a rank without cells, a rank with one; E = 3: narrow index rows
    (2, 3, [40, 17], 16, "f16", "data"),      # fp16 rows with fp16 gates; E = 6
    (2, 2, [33, 64], 24, "bf16", "data"),     # bf16 gates
    (5, 1, [9, 9, 9, 9, 9], 4, "f32", "none"),
])
def test_combine_that_pulls_edge_cases(world, group, cells, cols, dtype, gate_kind):
    """Uneven and empty cell counts per rank, path counts that are not multiples of 4 (one
    index per lane), gates stored in the data type, no gates.  Packed buckets; the forward
    exchange is the unfused one (rows dispatched by the checker)."""
    dev = torch.device("cuda", 0)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype]
    dt_code = {"f32": 0, "f16": 1, "bf16": 2}[dtype]
    E = world * group
    rng = np.random.default_rng(world * 7 + group)

    def rounded(a):
        return oracle.from_bits(oracle.to_bits(np.ascontiguousarray(a, dtype=np.float32), dtype),
                                dtype)

    idx_np, loads_np, gates_np, rows_np = [], [], [], []
    for r in range(world):
        T = cells[r]
        mask = oracle.topk_hot_mask(rng.standard_normal((T, E)).astype(np.float32), min(2, E)) \
            if T else np.zeros((0, E), dtype=np.int32)
        x = rounded(rng.standard_normal((T, cols)))
        i_np, l_np = oracle.generate_indices_and_loads(mask) if T else \
            (np.zeros((0, E), dtype=np.int32), np.zeros(E, dtype=np.int32))
        (routed,) = oracle.dispatch_with_indices_and_loads(x, i_np, l_np) if T else \
            (np.zeros((0, cols), dtype=np.float32),)
        idx_np.append(i_np)
        loads_np.append(l_np)
        gates_np.append(rounded(rng.random((T, E)) + 0.5))
        rows_np.append(routed)
    fwd = oracle.sim_group_sparse_all_to_all(rows_np, loads_np, False, 0)
    expert_out = [rounded(fwd[r][0] * np.float32(r + 2)) for r in range(world)]
    back = oracle.sim_size_known_group_sparse_all_to_all(
        expert_out, [f[1] for f in fwd], loads_np, False)
    ranks = Ranks(world)
    st = torch.cuda.current_stream().cuda_stream
    grain = cols * (4 if dtype == "f32" else 2)
    try:
        xs = [torch.from_numpy(a).to(dev).to(tdt) for a in rows_np]
        sizes = [torch.from_numpy(l).to(dev) for l in loads_np]
        idxs = [torch.from_numpy(i).to(dev).contiguous() for i in idx_np]
        if gate_kind == "none":
            gates, gdt = [None] * world, 0
        elif gate_kind == "f32":
            gates, gdt = [torch.from_numpy(g).to(dev) for g in gates_np], 0
        else:
            gates, gdt = [torch.from_numpy(g).to(dev).to(tdt) for g in gates_np], dt_code
        outs, ids, fit = ranks.forward(xs, sizes, group)
        assert all(fit)
        offsets = []
        for r in range(world):
            ptr, n_rows, _ = outs[r]
            if n_rows:
                ranks.rows_at(ptr, n_rows, cols, tdt).mul_(r + 2)
            offsets.append(ptr - ranks.arenas[r])
        results = [torch.full((max(cells[r], 1), cols), float("nan"), dtype=tdt, device=dev)
                   for r in range(world)]
        for stage in (POST, PUSH, WAIT):
            for r in range(world):
                _lib.call("brt_p2p_combine_backward", ranks.ctxs[r], ids[r], group, grain, 0,
                          offsets[r], idxs[r].data_ptr() if cells[r] else results[r].data_ptr(),
                          None if gates[r] is None or not cells[r] else gates[r].data_ptr(),
                          gdt, dt_code, cells[r], results[r].data_ptr(), st, stage)
        torch.cuda.synchronize()
        for r in range(world):
            T = cells[r]
            if T == 0:
                continue
            # (a single cell is combined like any other number here; the checker mirrors the
            # reference's shortcut for T == 1, so it is given a second, unrouted cell)
            i_chk, g_chk = idx_np[r], gates_np[r]
            if T == 1:
                i_chk = np.concatenate([i_chk, np.zeros((1, E), dtype=np.int32)])
                g_chk = np.concatenate([g_chk, np.ones((1, E), dtype=np.float32)])
            (want,) = oracle.combine_with_indices_and_loads(
                oracle.to_bits(back[r], dtype), i_chk, loads_np[r],
                None if gate_kind == "none" else
                (g_chk if gate_kind == "f32" else oracle.to_bits(g_chk, dtype)),
                None, False, dtype=dtype, gates_dtype="f32" if gate_kind != "data" else dtype)
            want = oracle.from_bits(want, dtype)[:T]
            got = results[r][:T].float().cpu().numpy()
            assert np.array_equal(got, want), f"rank {r}: {np.abs(got - want).max()}"
        for c in ranks.ctxs:
            assert _lib.query("brt_p2p_ctx_status", c) == 0
    finally:
        ranks.close()
