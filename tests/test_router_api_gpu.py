"""ScatterRouter / GatherRouter behaviour on the GPU, after the reference's own integration
tests (test/python/router_test.py:16-407): threshold scatter -> two identity experts ->
gather, on 2-D/3-D/4-D inputs, with score dispatch and with the capacity-padding variants."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    import brainstorm_b200 as brt
    from brainstorm_b200.router import GatherRouter, ScatterRouter

    return brt.Annotator, ScatterRouter, GatherRouter


def branch_route(api, gate, dispatch_score=False, supported_capacities=None,
                 capacity_padding=False, path_wise_padding=False, fused=False):
    Annotator, ScatterRouter, GatherRouter = api

    class BranchRoute(nn.Module):
        def __init__(self):
            super().__init__()
            self.annotator = Annotator([0])
            self.scatter_router = ScatterRouter(
                dispatch_score=dispatch_score, protocol_type="threshold",
                fabric_type="fused_dispatch" if fused else "dispatch",
                protocol_kwargs={"threshold": 0.5},
                fabric_kwargs={"supported_capacities": supported_capacities,
                               "capacity_padding": capacity_padding,
                               "path_wise_padding": path_wise_padding})
            self.expert1 = nn.Identity()
            self.expert2 = nn.Identity()
            self.gather_router = GatherRouter(
                fabric_type="fused_combine" if fused else "combine",
                fabric_kwargs={"ever_padded": capacity_padding})

        def forward(self, x):
            x = self.annotator(x)
            score = gate(x)
            if dispatch_score:
                score = self.annotator(score)
                dims = x.dim()
                routed, routed_score = self.scatter_router(x, score)
                x0, x1 = self.expert1(routed[0]), self.expert2(routed[1])
                pre = self.gather_router([x0 * routed_score[0].view(-1, *([1] * (dims - 1))),
                                          x1 * routed_score[1].view(-1, *([1] * (dims - 1)))])
                post = self.gather_router([x0, x1])
                s = self.gather_router([routed_score[0], routed_score[1]])
                return pre, post * s.view(-1, *([1] * (dims - 1)))
            routed = self.scatter_router(x, score)
            if fused:
                return self.gather_router(self.expert1(routed))
            x0, x1 = self.expert1(routed[0]), self.expert2(routed[1])
            return x0, x1, self.gather_router([x0, x1])

    return BranchRoute().eval().cuda()


def make_gate(dst, which_half):
    def gate(inputs):
        g = torch.zeros(inputs.shape[0], 2, dtype=torch.float, device=inputs.device)
        n = inputs.shape[0]
        if which_half == "upper":
            g[n // 2:, dst] = 1
        elif which_half == "lower":
            g[: n // 2, dst] = 1
        else:
            g[:, dst] = 1
        return g

    return gate


SAMPLES = [(8, 10), (8, 2, 10), (8, 2, 10, 2)]


def expected_rows(x, which_half):
    n = x.size(0)
    return {None: x, "upper": x[n // 2:], "lower": x[: n // 2]}[which_half]


@pytest.mark.parametrize("shape", SAMPLES)
@pytest.mark.parametrize("dst", [0, 1])
@pytest.mark.parametrize("which_half", [None, "upper", "lower"])
def test_generic_route(api, shape, dst, which_half):
    x = torch.arange(0, int(torch.tensor(shape).prod()), dtype=torch.float32).view(shape).cuda()
    model = branch_route(api, make_gate(dst, which_half))
    want = expected_rows(x, which_half)
    for _ in range(3):
        res = model(x)
        assert torch.equal(res[dst].data, want)
        assert res[1 - dst].numel() == 0
        assert torch.equal(res[2].data, want)


@pytest.mark.parametrize("shape", SAMPLES)
@pytest.mark.parametrize("dst", [0, 1])
@pytest.mark.parametrize("which_half", [None, "upper", "lower"])
def test_weighted_route(api, shape, dst, which_half):
    x = torch.arange(0, int(torch.tensor(shape).prod()), dtype=torch.float32).view(shape).cuda()
    model = branch_route(api, make_gate(dst, which_half), dispatch_score=True)
    pre, post = model(x)
    assert torch.allclose(pre.data, post.data)


@pytest.mark.parametrize("shape", SAMPLES)
@pytest.mark.parametrize("dst", [0, 1])
@pytest.mark.parametrize("which_half", [None, "upper", "lower"])
@pytest.mark.parametrize("cpad,pwise", [(False, False), (True, False), (True, True)])
def test_padded_route(api, shape, dst, which_half, cpad, pwise):
    caps = [10, 12]
    x = torch.arange(0, int(torch.tensor(shape).prod()), dtype=torch.float32).view(shape).cuda()
    model = branch_route(api, make_gate(dst, which_half), supported_capacities=caps,
                         capacity_padding=cpad, path_wise_padding=pwise)
    want = expected_rows(x, which_half)
    load = want.size(0)
    if cpad:
        load = caps[dst] if pwise else next(c for c in caps if load < c)
    for _ in range(3):
        res = model(x)
        assert res[dst].size(0) == load
        assert torch.equal(res[dst].data[: want.size(0)], want)
        if pwise:
            # path-wise padding reports the other path's capacity too: padding rows only
            assert not res[1 - dst].data.any()
        else:
            assert res[1 - dst].numel() == 0
        assert torch.equal(res[2].data, want)


def test_fused_topk_round_trip(api):
    """Fused fabrics: indices and loads ride on the GridTensor from scatter to gather."""
    Annotator, ScatterRouter, GatherRouter = api
    torch.manual_seed(0)
    x = torch.randn(512, 64, device="cuda")
    score = torch.softmax(torch.randn(512, 8, device="cuda"), dim=1)
    scatter = ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                            protocol_kwargs={"top_k": 2})
    gather = GatherRouter(fabric_type="fused_combine", fabric_kwargs={"transform": True})
    routed = scatter(Annotator([0])(x), score)
    assert routed.shape == (1024, 64)
    out = gather(routed, None, score)
    top = torch.topk(score, 2, dim=1)
    want = x * top.values[:, :1] + x * top.values[:, 1:]
    assert torch.allclose(out.data, want, rtol=1e-6, atol=1e-6)
    # distributed fabrics are the identity exchange without a process group
    scatter_d = ScatterRouter(protocol_type="topk", fabric_type="distributed_fused_dispatch",
                              protocol_kwargs={"top_k": 2})
    gather_d = GatherRouter(fabric_type="distributed_fused_combine",
                            fabric_kwargs={"transform": True})
    out_d = gather_d(scatter_d(Annotator([0])(x), score), None, score)
    assert torch.equal(out_d.data, out.data)


def test_slot_fabrics_without_a_process_group(api):
    """Without torch.distributed the padded-slot fabrics are the local fused fabrics."""
    Annotator, ScatterRouter, GatherRouter = api
    torch.manual_seed(2)
    T, E, cap = 600, 8, 200
    x = torch.randn(T, 48, device="cuda")
    score = torch.softmax(torch.randn(T, E, device="cuda"), dim=1)
    local = GatherRouter("fused_combine", {"transform": True, "max_path_padding": True})(
        ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                      protocol_kwargs={"top_k": 2},
                      fabric_kwargs={"max_path_padding": True, "max_path_load": cap})(
            Annotator([0])(x), score), None, score)
    routed = ScatterRouter(protocol_type="topk", fabric_type="distributed_slot_dispatch",
                           protocol_kwargs={"top_k": 2},
                           fabric_kwargs={"max_path_load": cap})(Annotator([0])(x), score)
    assert routed.shape == (E * cap, 48)
    out = GatherRouter("distributed_slot_combine", {"transform": True})(routed, None, score)
    assert torch.equal(out.data, local.data)
    # the placement fabrics are the packed-bucket ones under another name
    packed = GatherRouter("distributed_placement_combine", {"transform": True})(
        ScatterRouter(protocol_type="topk", fabric_type="distributed_placement_dispatch",
                      protocol_kwargs={"top_k": 2})(Annotator([0])(x), score), None, score)
    ref = GatherRouter("fused_combine", {"transform": True})(
        ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                      protocol_kwargs={"top_k": 2})(Annotator([0])(x), score), None, score)
    assert torch.equal(packed.data, ref.data)


def test_swin_moe_scatter(api):
    from brainstorm_b200.router import SwinMoEScatterRouter

    Annotator, _, GatherRouter = api
    torch.manual_seed(1)
    T, E = 1024, 8
    x = torch.randn(T, 32, device="cuda")
    score = torch.softmax(torch.randn(T, E, device="cuda"), dim=1)
    scatter = SwinMoEScatterRouter(
        fabric_type="fused_dispatch",
        protocol_kwargs={"top_k": 2, "capacity_factor": 1.0},
        fabric_kwargs={"max_path_padding": True})
    routed, new_score = scatter(Annotator([0])(x), score)
    cap = 2 * int(1.0 * ((T + E - 1) // E))
    assert routed.shape == (E * cap, 32)
    gather = GatherRouter(fabric_type="fused_combine",
                          fabric_kwargs={"transform": True, "max_path_padding": True})
    out = gather(routed, None, new_score)
    best = score.max(dim=1)
    assert torch.allclose(out.data, x * best.values[:, None], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("cpad", [False, True])
def test_swin_moe_gate_hands_its_indices_to_the_fabric(api, cpad):
    """The router's protocol computes the seat indices and loads along with the throttled mask
    (one launch); the fabric must route exactly as when it scans the mask itself."""
    from brainstorm_b200.router import SwinMoEScatterRouter

    Annotator, _, _ = api
    torch.manual_seed(3)
    T, E = 5000, 16
    x = torch.randn(T, 24, device="cuda")
    score = torch.softmax(torch.randn(T, E, device="cuda") * 3, dim=1)

    def make():
        return SwinMoEScatterRouter(
            fabric_type="fused_dispatch",
            protocol_kwargs={"top_k": 1, "capacity_factor": 0.5},
            fabric_kwargs={"max_path_padding": True, "capacity_padding": cpad})
    fused, plain = make(), make()
    assert fused.protocol.index_rules == (cpad, False)
    plain.protocol.index_rules = None  # the fabric scans the mask itself
    a, _ = fused(Annotator([0])(x), score)
    b, _ = plain(Annotator([0])(x), score)
    assert torch.equal(a.data, b.data)
    assert torch.equal(a.tag_stack[-1], b.tag_stack[-1])
    assert torch.equal(a.load_stack[-1], b.load_stack[-1])


@pytest.mark.parametrize("protocol,pkw", [("topk", {"top_k": 2}), ("threshold", {"threshold": 0.08}),
                                          ("threshold", {"threshold": 0.3, "residual_path": 1})])
@pytest.mark.parametrize("rules", [{}, {"supported_capacities": [300, 900, 4000]},
                                   {"supported_capacities": [300, 900, 4000],
                                    "capacity_padding": True}])
def test_scatter_gate_hands_its_indices_to_the_fabric(api, protocol, pkw, rules, monkeypatch):
    """ScatterRouter with a top-k or threshold protocol: the gate kernel that makes the hot
    mask also scans it under the fabric's capacity rules, and the fabric runs no index scan
    of its own; the routed rows equal those of a router whose fabric scans the mask."""
    from brainstorm_b200._C import router as c_router

    Annotator, ScatterRouter, GatherRouter = api
    torch.manual_seed(5)
    T, E = 3000, 8
    x = torch.randn(T, 32, device="cuda")
    score = torch.softmax(torch.randn(T, E, device="cuda") * 2, dim=1)

    def make():
        return ScatterRouter(protocol_type=protocol, fabric_type="fused_dispatch",
                             protocol_kwargs=pkw, fabric_kwargs=dict(rules)).cuda()
    fused, plain = make(), make()
    assert fused.protocol.index_rules_of is not None
    plain.protocol.index_rules_of = None
    scans = []
    real = c_router.generate_indices_and_loads
    monkeypatch.setattr(c_router, "generate_indices_and_loads",
                        lambda *a, **k: (scans.append(1), real(*a, **k))[1])
    a = fused(Annotator([0])(x), score)
    assert not scans, "the fabric scanned a mask whose indices the gate had already made"
    b = plain(Annotator([0])(x), score)
    assert len(scans) == 1
    assert torch.equal(a.data, b.data)
    assert torch.equal(a.load_stack[-1], b.load_stack[-1])
    assert torch.equal(a.tag_stack[-1], b.tag_stack[-1])
    out_a = GatherRouter(fabric_type="fused_combine", fabric_kwargs={"transform": True})(
        a, None, score)
    out_b = GatherRouter(fabric_type="fused_combine", fabric_kwargs={"transform": True})(
        b, None, score)
    assert torch.equal(out_a.data, out_b.data)
    # a copy of the router reads the rules of ITS fabric
    import copy
    twin = copy.deepcopy(fused)
    assert twin.protocol.index_rules_of.fabric is twin.fabric


def test_install_as_brt(api):
    import brainstorm_b200

    brainstorm_b200.install_as_brt()
    import brt._C.router as c_router
    from brt.router import ScatterRouter as S

    assert S is api[1]
    assert c_router.generate_indices_and_loads is \
        brainstorm_b200._C.router.generate_indices_and_loads
