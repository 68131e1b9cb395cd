"""Per-rank body of the multi-GPU tests; launched by tests/test_distributed_gpu.py through
torch.distributed.run, one process per GPU.  Every rank can rebuild every other rank's
seeded inputs, so each one checks its own outputs against the CPU restatement of the
reference's exchange semantics."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402


def rank_inputs(rank, W, G, d, hi, stride=0):
    rng = np.random.default_rng(1000 + rank)
    sizes = rng.integers(0, hi, size=W * G).astype(np.int32)
    rows = stride * W * G if stride else int(sizes.sum())
    x = rng.standard_normal((rows, d)).astype(np.float32)
    return x, sizes


def main():
    rank = int(os.environ["RANK"])
    W = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import brainstorm_b200.runtime.distributed as brt_dist
    from brainstorm_b200._C import distributed as C_dist

    assert brt_dist.is_nccl_activated()
    from brainstorm_b200.runtime import p2p

    want_p2p = os.environ.get("BRT_P2P", "1") != "0"
    assert (p2p.arena() is not None) == want_p2p, p2p._disabled_reason
    try:
        C_dist.init_nccl(torch.zeros(128, dtype=torch.int8), rank, W)
        raise AssertionError("second init_nccl must be refused")
    except RuntimeError:
        pass

    # ---- packed (sparse) exchange, forward and back, for G local experts
    # (d = 5 floats is not a 16-byte multiple: that case takes the NCCL transport either way)
    # (G = 64: more buckets than a host-planned copy list ever held; d = 1024 with up to 200
    # rows per bucket overflows a 1 MB landing half, which must send every rank to NCCL)
    for G, d, hi in ((1, 8, 40), (2, 16, 30), (4, 5, 12), (4, 8, 12), (3, 4, 20), (5, 12, 7),
                     (64, 4, 5), (2, 1024, 200)):
        all_in = [rank_inputs(r, W, G, d, hi) for r in range(W)]
        fwd = oracle.sim_group_sparse_all_to_all([a[0] for a in all_in], [a[1] for a in all_in])
        x, sizes = all_in[rank]
        out, out_loads, in_loads = brt_dist.group_sparse_a2a(
            torch.from_numpy(x).to(dev), torch.from_numpy(sizes).to(dev))
        assert not out_loads.is_cuda and not in_loads.is_cuda
        assert np.array_equal(out_loads.numpy(), fwd[rank][1])
        assert np.array_equal(in_loads.numpy(), sizes)
        assert np.array_equal(out.cpu().numpy(), fwd[rank][0]), f"rank {rank} forward G={G}"
        back = brt_dist.size_known_group_sparse_a2a(out, out_loads, in_loads)
        assert np.array_equal(back.cpu().numpy(), x), f"rank {rank} round trip G={G}"
    # two forward exchanges before their inverses, the inverses in reverse order, and one
    # rank whose send sizes are the same in both: each inverse must pick its own size matrix
    G, d = 2, 8
    first = [rank_inputs(r, W, G, d, 20) for r in range(W)]
    second = [rank_inputs(r + 50, W, G, d, 20) for r in range(W)]
    second[W - 1] = (np.random.default_rng(77).standard_normal(first[W - 1][0].shape)
                     .astype(np.float32), first[W - 1][1].copy())
    xa, sa = first[rank]
    xb, sb = second[rank]
    out_a, ol_a, il_a = brt_dist.group_sparse_a2a(torch.from_numpy(xa).to(dev),
                                                  torch.from_numpy(sa).to(dev))
    out_a = out_a.clone()  # held across two more exchanges: keep a private copy
    out_b, ol_b, il_b = brt_dist.group_sparse_a2a(torch.from_numpy(xb).to(dev),
                                                  torch.from_numpy(sb).to(dev))
    back_b = brt_dist.size_known_group_sparse_a2a(out_b, ol_b, il_b)
    assert np.array_equal(back_b.cpu().numpy(), xb), f"rank {rank}: nested inverse (second)"
    back_a = brt_dist.size_known_group_sparse_a2a(out_a, ol_a, il_a)
    assert np.array_equal(back_a.cpu().numpy(), xa), f"rank {rank}: nested inverse (first)"
    # size tensors rebuilt by the caller name no exchange: the inverse goes over NCCL
    back_a2 = brt_dist.size_known_group_sparse_a2a(out_a, ol_a.clone(), il_a.clone())
    assert np.array_equal(back_a2.cpu().numpy(), xa), f"rank {rank}: inverse by sizes only"

    # padded buckets
    for G, d, stride in ((2, 4, 16), (3, 8, 10), (1, 4, 7)):
        all_in = [rank_inputs(r, W, G, d, stride + 1, stride) for r in range(W)]
        x, sizes = all_in[rank]
        out, out_loads, in_loads = brt_dist.group_sparse_a2a(
            torch.from_numpy(x).to(dev), torch.from_numpy(sizes).to(dev), True, stride)
        fwd = oracle.sim_group_sparse_all_to_all([a[0] for a in all_in],
                                                 [a[1] for a in all_in], True, stride)
        o = out.cpu().numpy()
        for b, n in enumerate(out_loads.numpy().reshape(-1)):
            assert np.array_equal(o[b * stride:b * stride + n],
                                  fwd[rank][0][b * stride:b * stride + n]), (G, b)
        back = brt_dist.size_known_group_sparse_a2a(out, out_loads, in_loads,
                                                    True).cpu().numpy()
        for b, n in enumerate(sizes):
            assert np.array_equal(back[b * stride:b * stride + n],
                                  x[b * stride:b * stride + n]), (G, b)

    # ---- padded-slot exchange with the locality tail
    for G in (1, 2):
        slot, d = 12, 6
        all_in = []
        for r in range(W):
            rng = np.random.default_rng(2000 + r + 10 * G)
            s = rng.integers(0, slot + 1, size=W * G).astype(np.int32)
            all_in.append((rng.standard_normal((slot * W * G, d)).astype(np.float32), s))
        sim = oracle.sim_group_asymmetry_all_to_all([a[0] for a in all_in],
                                                    [a[1] for a in all_in])
        x, s = all_in[rank]
        xt, st = torch.from_numpy(x).to(dev), torch.from_numpy(s).to(dev)
        out, recv = brt_dist.group_asymmetry_a2a(xt, st, False)
        assert np.array_equal(recv.cpu().numpy(), sim[rank][1])
        o = out.cpu().numpy()
        for k, n in enumerate(sim[rank][1]):
            assert np.array_equal(o[k * slot:k * slot + n], sim[rank][0][k * slot:k * slot + n])
        back = C_dist.size_known_group_asymmetry_all_to_all(out, recv, st)
        b = back.cpu().numpy()
        for k, n in enumerate(s):
            assert np.array_equal(b[k * slot:k * slot + n], x[k * slot:k * slot + n])
            assert not b[k * slot + n:(k + 1) * slot].any()
        out2, reordered, reorder = brt_dist.group_asymmetry_a2a(xt, st, True)
        m = np.stack([sim[r][1] for r in range(W)]).reshape(W, W, G)
        exp_loads, exp_idx = oracle.group_locality_reorder(m, W, G)
        assert np.array_equal(reorder.cpu().numpy(), exp_idx)
        assert np.array_equal(reordered.cpu().numpy(), exp_loads[rank].reshape(-1))
        # exchange along the permutation and back
        mine = torch.full((7, 3), float(rank), device=dev)
        got = brt_dist.exchange(mine, reorder)
        assert torch.all(got == float(exp_idx[rank]))
        assert torch.equal(brt_dist.reverse_exchange(got, reorder), mine)
        outs = brt_dist.batched_exchange([mine, mine * 2], reorder)
        assert torch.all(outs[1] == 2.0 * exp_idx[rank])

    # ---- routers: the distributed fused fabrics equal the local fused fabrics (identity expert)
    from brainstorm_b200 import Annotator
    from brainstorm_b200.router import GatherRouter, ScatterRouter

    g = torch.Generator().manual_seed(rank)
    T, E, d = 512, 4 * W, 64
    x = torch.randn((T, d), generator=g).to(dev)
    score = torch.softmax(torch.randn((T, E), generator=g), dim=1).to(dev)
    local = GatherRouter("fused_combine", {"transform": True})(
        ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                      protocol_kwargs={"top_k": 2})(Annotator([0])(x), score), None, score)
    for pull in (False, True):  # inverse exchange + combine as two kernels, and as one that pulls
        routed = ScatterRouter(protocol_type="topk", fabric_type="distributed_fused_dispatch",
                               protocol_kwargs={"top_k": 2})(Annotator([0])(x), score)
        ep = GatherRouter("distributed_fused_combine",
                          {"transform": True, "pull_combine": pull})(routed, None, score)
        assert torch.equal(ep.data, local.data), \
            f"rank {rank}: expert-parallel route differs (pull_combine={pull})"

    if p2p.arena() is not None and p2p.ZERO_COPY:
        # the same route with the exchange's sizes left on the device (weighted dispatch takes
        # the two-op path, the unweighted one the fused kernel)
        for weighted in (False, True):
            skw = {"device_sizes": True}
            ref = GatherRouter("fused_combine", {"transform": not weighted})(
                ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                              protocol_kwargs={"top_k": 2},
                              fabric_kwargs={"transform": weighted})(Annotator([0])(x), score),
                None, score)
            routed_d = ScatterRouter(protocol_type="topk",
                                     fabric_type="distributed_fused_dispatch",
                                     protocol_kwargs={"top_k": 2},
                                     fabric_kwargs=dict(skw, transform=weighted))(
                Annotator([0])(x), score)
            assert routed_d.load.is_cuda
            ep_d = GatherRouter("distributed_fused_combine", {"transform": not weighted})(
                routed_d, None, score)
            assert torch.equal(ep_d.data, ref.data), \
                f"rank {rank}: device-sized route differs (weighted dispatch: {weighted})"

    # ---- padded-slot fabrics: plain, and with the locality matching (the cells of rank
    # reorder[k] come out on rank k)
    cap = 2 * T // E * 3
    fkw = {"max_path_load": cap}
    local_p = GatherRouter("fused_combine", {"transform": True, "max_path_padding": True})(
        ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                      protocol_kwargs={"top_k": 2},
                      fabric_kwargs={"max_path_padding": True, "max_path_load": cap})(
            Annotator([0])(x), score), None, score)
    slots = GatherRouter("distributed_slot_combine", {"transform": True})(
        ScatterRouter(protocol_type="topk", fabric_type="distributed_slot_dispatch",
                      protocol_kwargs={"top_k": 2}, fabric_kwargs=fkw)(Annotator([0])(x), score),
        None, score)
    assert torch.equal(slots.data, local_p.data), f"rank {rank}: padded-slot route differs"
    matched = GatherRouter("distributed_slot_combine",
                           {"transform": True, "locality_aware": True})(
        ScatterRouter(protocol_type="topk", fabric_type="distributed_slot_dispatch",
                      protocol_kwargs={"top_k": 2},
                      fabric_kwargs=dict(fkw, locality_aware=True))(Annotator([0])(x), score),
        None, score)
    reorder = brt_dist.get_reorder_indices()
    everyone = [torch.empty_like(local_p.data) for _ in range(W)]
    dist.all_gather(everyone, local_p.data.contiguous())
    assert torch.equal(matched.data, everyone[int(reorder[rank])]), \
        f"rank {rank}: locality-matched route differs"

    # ---- a routing step with both exchanges captured in a CUDA graph and replayed on new
    # inputs: the sizes never reach the host, the epochs of the flags advance on the device
    if p2p.arena() is not None and p2p.ZERO_COPY and p2p.arena().half_bytes >= (64 << 20):
        from brainstorm_b200._C import router as R

        T, E, d = 384, 4 * W, 64
        cells = torch.zeros((T, d), device=dev)
        mask = torch.zeros((T, E), dtype=torch.int32, device=dev)

        def step(pull=False):
            idx, loads = R.generate_indices_and_loads(mask)
            with brt_dist.replayable_exchanges():
                landed, received, sent = brt_dist.dispatch_group_sparse_a2a_device(
                    cells, idx, loads)
                if pull:
                    y = brt_dist.combine_group_sparse_a2a(landed, idx, None, received, sent)
                    assert y is not None
                else:
                    back = brt_dist.size_known_group_sparse_a2a(landed, received, sent)
            if not pull:
                (y,) = R.combine_with_indices_and_loads(back, idx, loads, None, None)
            return y, received, landed

        def fill(seed):
            gen = torch.Generator().manual_seed(seed * 100 + rank)
            cells.copy_(torch.randn((T, d), generator=gen))
            picks = torch.topk(torch.randn((T, E), generator=gen), 2, dim=1).indices
            mask.copy_(torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1))

        def check(y, received, landed, what):
            idx, loads = R.generate_indices_and_loads(mask)
            (routed,) = R.dispatch_with_indices_and_loads(cells, idx, loads)
            (want,) = R.combine_with_indices_and_loads(routed, idx, loads, None, None)
            assert torch.equal(y, want), f"rank {rank}: {what}: combined cells differ"
            want_out, want_recv, _ = brt_dist.group_sparse_a2a(routed, loads)
            assert torch.equal(received.cpu(), want_recv.reshape(-1).to(torch.int32)), \
                f"rank {rank}: {what}: received sizes differ"
            n = int(want_recv.sum())
            # (the eager exchange above reused a landing half: compare the clone taken before)
            assert torch.equal(landed[:n], want_out), f"rank {rank}: {what}: landed rows differ"

        fill(1)
        y, received, landed = step()  # issued eagerly: a section run once
        check(y, received, landed[:int(received.sum())].clone(), "eager section")
        fill(2)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y, received, landed = step()
        for seed in (3, 4, 5):
            fill(seed)
            graph.replay()
            torch.cuda.synchronize()
            check(y.clone(), received.clone(), landed[:int(received.sum())].clone(),
                  f"replay {seed}")
        # the same step with the combine that pulls its rows from the peers, captured too
        fill(7)
        step(pull=True)
        torch.cuda.synchronize()
        dist.barrier()
        pull_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(pull_graph):
            y2, received2, landed2 = step(pull=True)
        for seed in (8, 9):
            fill(seed)
            pull_graph.replay()
            torch.cuda.synchronize()
            snap = (y2.clone(), received2.clone(), landed2[:int(received2.sum())].clone())
            graph.replay()  # the two graphs share the arena: they may alternate
            torch.cuda.synchronize()
            assert torch.equal(y, snap[0]), \
                f"rank {rank}: pull replay {seed} differs from the two ops"
            check(*snap, f"pull replay {seed}")
        # ordinary exchanges continue after the replays, and another replay after them
        xs, sizes = rank_inputs(rank, W, 2, 8, 20)
        o, ol, il = brt_dist.group_sparse_a2a(torch.from_numpy(xs).to(dev),
                                              torch.from_numpy(sizes).to(dev))
        assert np.array_equal(brt_dist.size_known_group_sparse_a2a(o, ol, il).cpu().numpy(), xs)
        fill(6)
        graph.replay()
        torch.cuda.synchronize()
        check(y.clone(), received.clone(), landed[:int(received.sum())].clone(), "late replay")

        # ---- a whole expert-parallel FFN layer in one CUDA graph: gate picks -> indices ->
        # dispatch fused with the exchange -> two grouped tensor-core GEMMs that read their
        # loads on the device -> inverse exchange -> weighted combine
        from brainstorm_b200._C import expert as X

        T, G, d, H = 256, 4, 128, 256
        E = G * W
        wgen = torch.Generator().manual_seed(4242)  # the same weights on every rank
        w1_all = (torch.randn((E, H, d), generator=wgen) / d ** 0.5).bfloat16()
        w2_all = (torch.randn((E, d, H), generator=wgen) / H ** 0.5).bfloat16()
        w1 = w1_all[rank * G:(rank + 1) * G].to(dev).contiguous()
        w2 = w2_all[rank * G:(rank + 1) * G].to(dev).contiguous()
        tokens = torch.zeros((T, d), dtype=torch.bfloat16, device=dev)
        picks_mask = torch.zeros((T, E), dtype=torch.int32, device=dev)
        gate_w = torch.zeros((T, E), dtype=torch.float32, device=dev)
        bound = T * 2 * W  # no rank can receive more rows than every rank's picks together

        def ffn_layer():
            idx, loads = R.generate_indices_and_loads(picks_mask)
            with brt_dist.replayable_exchanges():
                landed, received, sent = brt_dist.dispatch_group_sparse_a2a_device(
                    tokens, idx, loads)
                per_expert = received.view(G, W).sum(dim=1).to(torch.int32)
                hidden = X.grouped_expert_linear(landed[:bound], w1, per_expert, relu=True)
                # the experts' outputs go where the combine can pull them from the peers
                y = X.grouped_expert_linear(hidden, w2, per_expert,
                                            out=brt_dist.expert_output_buffer(bound, landed))
                out = brt_dist.combine_group_sparse_a2a(y, idx, gate_w, received, sent)
                assert out is not None
            return out

        def refill(seed):
            gen = torch.Generator().manual_seed(seed * 1000 + rank)
            tokens.copy_(torch.randn((T, d), generator=gen).bfloat16())
            sc = torch.softmax(torch.randn((T, E), generator=gen), dim=1)
            vals, picks = torch.topk(sc, 2, dim=1)
            picks_mask.copy_(torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1))
            gate_w.copy_(torch.zeros((T, E)).scatter_(1, picks, vals))
            return picks, vals

        def reference(picks, vals):
            xt = tokens.cpu().float()
            want = torch.zeros((T, d))
            for t in range(T):
                for e, g_ in zip(picks[t].tolist(), vals[t].tolist()):
                    hid = torch.relu(xt[t] @ w1_all[e].float().T).bfloat16().float()
                    want[t] += g_ * (hid @ w2_all[e].float().T).bfloat16().float()
            return want

        picks, vals = refill(1)
        ffn_layer()  # warm-up, eager
        torch.cuda.synchronize()
        dist.barrier()
        layer_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(layer_graph):
            layer_out = ffn_layer()
        for seed in (2, 3):
            picks, vals = refill(seed)
            layer_graph.replay()
            torch.cuda.synchronize()
            X.check_status()
            want = reference(picks, vals)
            err = float((layer_out.cpu().float() - want).abs().max())
            assert err <= 2e-2 * float(want.abs().max()), \
                f"rank {rank}: FFN layer differs from the fp32 reference by {err}"

    p2p.check_status()
    if p2p.arena() is not None:
        # the collective reset (what a job does after a wait ran out): every rank back to its
        # initial state, then the exchanges work again
        p2p.reset()
        assert int(p2p.arena().status()) == 0
        xs, sizes = rank_inputs(rank, W, 3, 8, 15)
        o, ol, il = brt_dist.group_sparse_a2a(torch.from_numpy(xs).to(dev),
                                              torch.from_numpy(sizes).to(dev))
        assert np.array_equal(brt_dist.size_known_group_sparse_a2a(o, ol, il).cpu().numpy(), xs)
        p2p.check_status()
    dist.barrier()
    if rank == 0:
        print("DIST_OK", W)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
