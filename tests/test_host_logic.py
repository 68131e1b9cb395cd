"""CPU-side checks: the C ABI library loads and exports what the header declares, and the
host-side mirror of the reference's Python surface (GridTensor, Annotator, Registry,
protocols, argument checks) behaves like the reference.  No kernel is launched."""
import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def header_symbols():
    text = (ROOT / "include" / "brt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(brt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from brainstorm_b200 import _lib, build

    build.build()
    lib = _lib.load()
    names = header_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    unbound = [n for n in names if n not in _lib.SIGNATURES]
    assert not unbound, f"declared in the header but not bound in _lib.py: {unbound}"
    extra = [n for n in _lib.SIGNATURES if n not in names]
    assert not extra, f"bound in _lib.py but not declared in the header: {extra}"


def test_queries_that_need_no_gpu():
    from brainstorm_b200 import _lib

    assert _lib.query("brt_abi_version") >= 1
    assert _lib.query("brt_last_error") in (b"", None) or isinstance(
        _lib.query("brt_last_error"), bytes)
    small = _lib.query("brt_index_scratch_bytes", 4096, 8)
    big = _lib.query("brt_index_scratch_bytes", 262144, 128)
    assert 256 <= small < big
    assert big >= 2 * (262144 // 32) * 128 * 4
    assert _lib.query("brt_dispatch_scratch_bytes", 65536, 32) >= 65536
    assert _lib.query("brt_static_index_scratch_bytes") == 2 << 20
    assert _lib.query("brt_nccl_is_initialized") == 0


def test_status_codes_without_gpu():
    """Argument checks run before any CUDA call."""
    from brainstorm_b200 import _lib

    with pytest.raises(_lib.BrtError, match="bad shape"):
        _lib.call("brt_generate_indices_and_loads", None, None, None, None, 4, 0, None, 0, 0, 0,
                  0, None, 0, None)
    with pytest.raises(_lib.BrtError, match="capacity_padding needs"):
        _lib.call("brt_generate_indices_and_loads", 16, 16, 16, None, 4, 4, None, 0, 1, 0, 0,
                  None, 0, None)
    # the gate entry point applies the same capacity rules before it touches anything
    with pytest.raises(_lib.BrtError, match="capacity_padding needs"):
        _lib.call("brt_route_scores", 16, 64, 8, 0, 1, 0.0, -1, 2, 16, 16, None, None, 0, 1, 0,
                  None, None, None, None, None, 0, None)
    with pytest.raises(_lib.BrtError, match="path_wise_padding needs"):
        _lib.call("brt_route_scores", 16, 64, 8, 0, 1, 0.0, -1, 2, 16, 16, None, 16, 3, 1, 1,
                  None, None, None, None, None, 0, None)
    with pytest.raises(_lib.BrtError, match="has not been called"):
        _lib.call("brt_all_to_all", None, None, 0, None)
    with pytest.raises(_lib.BrtError, match="world_size"):
        _lib.call("brt_locality_reorder", 16, 64, 16, 16, None)
    with pytest.raises(_lib.BrtError, match="holds 2097152 bytes"):
        _lib.call("brt_generate_indices_and_loads_static", 16, 16, 16, 1 << 20, 128, None, 0, 0,
                  0, 0, None)


def test_ops_refuse_cpu_tensors():
    from brainstorm_b200._C import router as R

    m = torch.zeros((4, 2), dtype=torch.int32)
    for call in (lambda: R.generate_indices_and_loads(m),
                 lambda: R.throttle_hotmask(m, torch.zeros(2, dtype=torch.int32),
                                            torch.zeros(2, dtype=torch.int32)),
                 lambda: R.dispatch_with_indices_and_loads(torch.zeros(4, 3), m, m[0]),
                 lambda: R.combine_with_indices_and_loads(torch.zeros(4, 3), m, m[0])):
        with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
            call()


def test_grid_tensor_stacks():
    from brainstorm_b200.runtime.grid_tensor import (GridTensor, deinit_grid_tensor,
                                                     init_grid_tensor, to_torch_tensor)

    x = init_grid_tensor(torch.arange(6.).view(3, 2), [None], [None])
    assert isinstance(x, GridTensor) and x.stack_size == 1 and x.tag is None
    tag, load = torch.tensor([1, 2, 3]), torch.tensor([3])
    x.pack(tag, load, note="n")
    assert x.stack_size == 2 and x.tag is tag and x.get_extra_attr("note") == "n"
    y = x * 2 + 1                      # stacks follow results of torch functions
    assert isinstance(y, GridTensor) and y.tag is tag and y.load is load
    assert y.extra_attr_dict == {"note": "n"}
    plain, tags, loads, extra = to_torch_tensor(y, retrieve_attr=True)
    assert type(plain) is torch.Tensor and tags[-1] is tag
    # stacks travel by reference (SHALLOW_TRANSPORT, as in the reference): y shares x's lists
    assert y.tag_stack is x.tag_stack
    z, t, l, extra = x.unpack("note")
    assert t is tag and l is load and extra == {"note": "n"} and x.stack_size == 1
    assert y.stack_size == 1
    plain2, tags2, _, _ = deinit_grid_tensor(y)
    assert type(plain2) is torch.Tensor and y.tag_stack == [] and tags2 == [None]
    empty = init_grid_tensor(torch.zeros(2))
    assert empty.annotation_empty() and empty.cell_initilized


def test_annotator():
    from brainstorm_b200 import Annotator, GridTensor

    t = torch.arange(24.).view(2, 3, 4)
    cells = Annotator([0])(t)
    assert isinstance(cells, GridTensor) and cells.shape == (2, 3, 4)
    assert cells.tag_stack == [None] and cells.load_stack == [None]
    cells = Annotator([0, 1])(t)
    assert cells.shape == (6, 4)
    cells = Annotator([1], gridding=False)(t)
    assert type(cells) is torch.Tensor and cells.shape == (3, 2, 4)
    assert torch.equal(cells[1], t[:, 1])


def test_registry_and_factories():
    from brainstorm_b200.router import (GatherRouter, RouterBase, ScatterRouter, is_router,
                                        make_router, register_router)
    from brainstorm_b200.router.fabric import make_fabric
    from brainstorm_b200.router.protocol import make_protocol
    from brainstorm_b200.router.utils import make_kwargs

    s = make_router("scatter", {"protocol_type": "threshold", "fabric_type": "dispatch",
                                "protocol_kwargs": {"threshold": 0.3}})
    assert isinstance(s, ScatterRouter) and s.protocol.threshold == 0.3
    assert s.fabric.is_tag_index and s.fabric_kwargs["flow_num"] == 1
    assert is_router(s) and is_router(GatherRouter) and not is_router(torch.nn.Linear(1, 1))
    with pytest.raises(ValueError):
        make_router("no_such_router", {})
    with pytest.raises(ValueError):
        make_kwargs({1: 2})
    with pytest.raises(ValueError):
        register_router("x")(torch.nn.Linear)
    assert make_protocol("topk", {"top_k": 2}).top_k == 2
    f = make_fabric("fused_dispatch", {"flow_num": 1, "supported_capacities": [4, 8],
                                       "capacity_padding": True})
    assert not f.is_tag_index and f.supported_capacities.tolist() == [4, 8]
    d = ScatterRouter(dispatch_score=True)
    assert d.fabric.flow_num == 2 and d.fabric.route_logics == ["1d", "2d"]

    @register_router("my_router")
    class MyRouter(RouterBase):
        pass

    assert MyRouter._router_type == "my_router" and MyRouter.brt_abs_type == "my_router"


def test_protocols_match_reference_outputs(golden_dir):
    from brainstorm_b200.router.protocol import make_protocol

    z = np.load(golden_dir / "ref_python_vectors.npz")
    score = torch.from_numpy(z["proto/score"])
    for k in (1, 2, 3):
        got = make_protocol("topk", {"top_k": k})(score)
        assert got.dtype == torch.int32 and np.array_equal(got.numpy(), z[f"proto/topk{k}"])
    sig = torch.from_numpy(z["proto/sigmoid"])
    got = make_protocol("threshold", {"threshold": 0.5})(sig)
    assert np.array_equal(got.numpy(), z["proto/threshold_0.5"])
    got = make_protocol("threshold", {"threshold": 0.8, "residual_path": 3})(sig)
    assert np.array_equal(got.numpy(), z["proto/threshold_0.8_residual3"])
    one_hot = torch.eye(4)[torch.tensor([1, 3, 0])]
    assert make_protocol("switch_top1", {})(one_hot).tolist() == one_hot.int().tolist()
    two = make_protocol("residual_threshold", {"threshold": 1.0, "residual_path": 0})(
        torch.tensor([[0.2, 0.3], [0.9, 0.9]]))
    assert two.tolist() == [[1, 0], [0, 1]]


def test_stats_capture_is_off_by_default():
    from brainstorm_b200.router.fabric import make_fabric

    f = make_fabric("dispatch", {"flow_num": 1})
    assert f.capturing is False and f.load_history is None
    f.capture_flow_stats([torch.zeros(1)], None, None)  # no-op
    assert f.history_len == 0


def test_distributed_wrappers_are_identity_without_process_group():
    import brainstorm_b200.runtime.distributed as brt_dist

    x, loads = torch.randn(5, 3), torch.tensor([2, 3], dtype=torch.int32)
    assert brt_dist.is_nccl_activated() is False
    out, out_loads, in_loads = brt_dist.group_sparse_a2a(x, loads)
    assert out is x and out_loads is loads and in_loads is loads
    assert brt_dist.size_known_group_sparse_a2a(x, loads, loads) is x
    assert brt_dist.exchange(x, loads) is x and brt_dist.reverse_exchange(x, loads) is x
    assert brt_dist.group_asymmetry_a2a(x, loads) == (x, loads)


def test_workload_generator_is_deterministic():
    import bench

    a = bench.make_workload("cfg1")
    b = bench.make_workload("cfg1")
    assert torch.equal(a["x"], b["x"]) and torch.equal(a["mask"], b["mask"])
    assert a["cap"] == 640 and a["mask"].sum().item() == 4096
    c2 = bench.WORKLOADS["cfg2"]
    assert bench.capacity_of(c2) == 2048 and bench.capacity_of(bench.WORKLOADS["cfg3"]) == 4096


def test_scatter_router_tells_its_protocol_the_fabric_rules():
    """The hand-over of seat indices from the gate kernel to the fabric is set up on the host:
    the router gives its protocol a view of the fabric's capacity rules (which follows a deep
    copy to the copy's own fabric), and without CUDA scores the protocol routes with torch ops
    and attaches nothing."""
    import copy

    import torch

    from brainstorm_b200.router import ScatterRouter

    router = ScatterRouter(protocol_type="topk", fabric_type="fused_dispatch",
                           protocol_kwargs={"top_k": 2},
                           fabric_kwargs={"supported_capacities": [4, 8],
                                          "capacity_padding": True})
    rules = router.protocol.index_rules_of
    caps, cpad, pwise = rules()
    assert caps is router.fabric.supported_capacities and cpad is True and pwise is False
    twin = copy.deepcopy(router)
    assert twin.protocol.index_rules_of.fabric is twin.fabric
    assert "index_rules_of" not in dict(router.protocol.named_modules())
    assert not any("index_rules_of" in k for k in router.state_dict())
    mask = router.protocol(torch.rand(6, 4))
    assert mask.dtype == torch.int32 and int(mask.sum()) == 12
    assert not hasattr(mask, "_brt_routes")


def test_replayable_exchanges_need_the_arena():
    import pytest

    from brainstorm_b200._C import distributed as C_dist

    with pytest.raises(RuntimeError):
        with C_dist.replayable_exchanges():
            pass
