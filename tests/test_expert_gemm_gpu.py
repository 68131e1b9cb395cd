"""The grouped expert GEMM (tcgen05 tensor cores) on dispatched layouts, against an fp32 torch
reference of the same op: relative error below 1e-2 of the largest reference value (bf16
inputs, fp32 accumulation, one rounding to bf16)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOLERANCE = 1e-2


@pytest.fixture(scope="module")
def X():
    from brainstorm_b200._C import expert

    return expert


def reference(rows, weights, loads, cap, relu):
    out = {}
    base = 0
    for e, n in enumerate(loads):
        start = e * cap if cap else base
        n = min(n, cap) if cap else n
        y = rows[start:start + n].float() @ weights[e].float().T
        out[e] = (start, n, y.relu() if relu else y)
        base += loads[e]
    return out


CASES = [
    # experts, in, out, loads, padded slot (0 = packed), relu
    (1, 64, 128, [128], 0, False),
    (1, 64, 128, [37], 0, False),
    (2, 128, 128, [100, 200], 0, False),
    (4, 256, 256, [0, 300, 5, 129], 0, True),
    (4, 256, 256, [0, 300, 5, 129], 320, False),
    (4, 256, 256, [400, 0, 0, 7], 320, False),   # a load above the slot is cut at the slot
    (8, 1024, 1024, [50, 0, 700, 128, 127, 129, 1, 999], 0, True),
    (32, 1024, 1024, None, 0, False),             # cfg2 shape, skewed loads
    (32, 1024, 1024, None, 2048, False),          # cfg2 shape, capacity-padded
    (128, 768, 768, None, 0, False),              # cfg3 shape, Zipf-like loads
    (128, 768, 3072, None, 0, True),
]


@pytest.mark.parametrize("E,K,N,loads,cap,relu", CASES)
def test_grouped_expert_linear(X, E, K, N, loads, cap, relu):
    rng = np.random.default_rng(E * 7 + K + N + cap)
    if loads is None:
        ranks = rng.permutation(E) + 1.0
        share = ranks ** -1.1
        loads = [int(v) for v in (share / share.sum() * 40000).astype(np.int64)]
        loads[int(rng.integers(0, E))] = 0
        if cap:
            loads = [min(v, cap) for v in loads]
    L = cap * E if cap else sum(loads)
    torch.manual_seed(E + K)
    rows = (torch.randn(L, K, device="cuda") * 0.5).bfloat16()
    weights = (torch.randn(E, N, K, device="cuda") / K ** 0.5).bfloat16()
    loads_t = torch.tensor(loads, dtype=torch.int32, device="cuda")
    out = X.grouped_expert_linear(rows, weights, loads_t, bool(cap), cap, relu)
    X.check_status()
    assert out.shape == (L, N) and out.dtype == torch.bfloat16
    for e, (start, n, want) in reference(rows, weights, loads, cap, relu).items():
        if n == 0:
            continue
        got = out[start:start + n].float()
        scale = max(float(want.abs().max()), 1e-6)
        assert float((got - want).abs().max()) / scale < TOLERANCE, f"expert {e}"


def test_rows_beyond_a_load_are_left_alone(X):
    E, K, N, cap = 4, 128, 128, 200
    loads = [10, 200, 0, 77]
    rows = torch.randn(E * cap, K, device="cuda").bfloat16()
    weights = torch.randn(E, N, K, device="cuda").bfloat16()
    # make the allocator hand the op a block full of NaNs: what it does not write stays NaN
    junk = torch.full((E * cap, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ptr = junk.data_ptr()
    del junk
    out = X.grouped_expert_linear(rows, weights, torch.tensor(loads, dtype=torch.int32,
                                                              device="cuda"), True, cap)
    X.check_status()
    for e, n in enumerate(loads):
        assert torch.isfinite(out[e * cap:e * cap + n].float()).all()
        if out.data_ptr() == ptr:
            assert torch.isnan(out[e * cap + n:(e + 1) * cap].float()).all()


def test_unsupported_shapes_and_arguments(X):
    rows = torch.zeros(8, 100, device="cuda", dtype=torch.bfloat16)
    weights = torch.zeros(2, 128, 100, device="cuda", dtype=torch.bfloat16)
    loads = torch.tensor([4, 4], dtype=torch.int32, device="cuda")
    with pytest.raises(NotImplementedError):
        X.grouped_expert_linear(rows, weights, loads)             # in_features % 64 != 0
    with pytest.raises(NotImplementedError):
        X.grouped_expert_linear(rows.float(), weights.float(), loads)
    with pytest.raises(RuntimeError):
        X.grouped_expert_linear(rows.cpu(), weights, loads)
    empty = X.grouped_expert_linear(torch.zeros(0, 64, device="cuda", dtype=torch.bfloat16),
                                    torch.zeros(2, 128, 64, device="cuda", dtype=torch.bfloat16),
                                    torch.zeros(2, dtype=torch.int32, device="cuda"))
    assert empty.shape == (0, 128)
