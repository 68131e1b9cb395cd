"""Parity of the single-launch gate (brt_route_scores through the C ABI) with the CPU checker
and with the golden outputs of the reference's protocol classes.  Integer outputs are compared
bit for bit; the renormalised gates within 1e-6 relative (fp32)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def R():
    from brainstorm_b200._C import router

    return router


def scores(T, E, seed, softmax=True):
    rng = np.random.default_rng(seed)
    s = rng.standard_normal((T, E)).astype(np.float32)
    return oracle.softmax(s) if softmax else s


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


CASES = [(1, 4, 1), (33, 8, 2), (1037, 8, 1), (4096, 8, 1), (5000, 32, 2), (3000, 128, 1),
         (2500, 64, 4), (700, 256, 8), (100000, 16, 2), (300000, 128, 2), (150000, 32, 2)]


@pytest.mark.parametrize("T,E,k", CASES)
def test_topk_mask_and_loads(R, T, E, k):
    s = scores(T, E, T + E + k)
    exp_m, exp_l = oracle.route_scores(s, "topk", k, output="mask")
    got_m, got_l = R.route_scores(cuda(s), "topk", k, output="mask")
    assert np.array_equal(got_l.cpu().numpy(), exp_l)
    assert np.array_equal(got_m.cpu().numpy(), exp_m)


@pytest.mark.parametrize("T,E,k", CASES)
def test_topk_seat_indices(R, T, E, k):
    s = scores(T, E, 3 * T + E + k, softmax=False)
    caps = np.array(sorted({1, 16, 256, max(1, T * k // E), max(1, 2 * T * k // E)}),
                    dtype=np.int32)
    for c, cpad in ((None, False), (caps, False), (caps, True)):
        exp_i, exp_l = oracle.route_scores(s, "topk", k, output="seat_indices",
                                           supported_capacities=None if c is None else list(c),
                                           capacity_padding=cpad)
        got_i, got_l = R.route_scores(cuda(s), "topk", k, output="seat_indices",
                                      supported_capacities=None if c is None else cuda(c),
                                      capacity_padding=cpad)
        assert np.array_equal(got_l.cpu().numpy(), exp_l), cpad
        assert np.array_equal(got_i.cpu().numpy(), exp_i), cpad


@pytest.mark.parametrize("T,E,k", [(33, 8, 1), (5000, 32, 1), (32768, 32, 2), (262144, 128, 1)])
def test_topk_throttled_mask(R, T, E, k):
    """The Swin-MoE gate (python/brt/router/protocol/swin_moe.py:69-80): first pick, cut at the
    runtime capacity."""
    s = scores(T, E, 7 * T + E)
    rng = np.random.default_rng(T)
    prefix = rng.integers(0, 5, size=E).astype(np.int32)
    cap = np.full(E, k * ((T + E - 1) // E), dtype=np.int32)
    exp_p = prefix.copy()
    exp_m, _ = oracle.route_scores(s, "topk", k, output="throttled_mask", prefix=exp_p,
                                   throttle_capacity=cap)
    p = cuda(prefix)
    got_m, got_p = R.route_scores(cuda(s), "topk", k, output="throttled_mask", prefix=p,
                                  throttle_capacity=cuda(cap))
    assert got_p is p
    assert np.array_equal(got_p.cpu().numpy(), exp_p)
    assert np.array_equal(got_m.cpu().numpy(), exp_m)


@pytest.mark.parametrize("T,E,k", [(33, 8, 1), (5000, 32, 1), (32768, 32, 2), (262144, 128, 1),
                                   (65536, 64, 2)])
def test_topk_throttled_seat_indices(R, T, E, k):
    """Scores straight to the seat indices and loads of the throttled mask: gate, throttle
    and index scan in one launch."""
    s = scores(T, E, 5 * T + E)
    rng = np.random.default_rng(T + 1)
    prefix = rng.integers(0, 5, size=E).astype(np.int32)
    cap = np.full(E, k * ((T + E - 1) // E), dtype=np.int32)
    exp_p = prefix.copy()
    exp_m, _ = oracle.route_scores(s, "topk", k, output="throttled_mask", prefix=exp_p,
                                   throttle_capacity=cap)
    for caps, cpad in ((None, False), ([64, 1024, 16384], True)):
        exp_i, exp_l = oracle.generate_indices_and_loads(exp_m, caps, cpad)
        p = cuda(prefix)
        got_i, got_l, got_p = R.route_scores(
            cuda(s), "topk", k, output="throttled_seat_indices", prefix=p,
            throttle_capacity=cuda(cap),
            supported_capacities=None if caps is None else cuda(np.array(caps, dtype=np.int32)),
            capacity_padding=cpad)
        assert got_p is p
        assert np.array_equal(got_p.cpu().numpy(), exp_p)
        assert np.array_equal(got_l.cpu().numpy(), exp_l)
        assert np.array_equal(got_i.cpu().numpy(), exp_i)


@pytest.mark.parametrize("T,E,thr,res", [(64, 8, 0.5, -1), (5000, 8, 0.5, -1), (5000, 8, 0.8, 3),
                                         (70000, 64, 0.9, 40), (3000, 128, 0.2, 0)])
def test_threshold(R, T, E, thr, res):
    rng = np.random.default_rng(T + E)
    s = (1.0 / (1.0 + np.exp(-rng.standard_normal((T, E))))).astype(np.float32)
    for output in ("mask", "seat_indices"):
        exp = oracle.route_scores(s, "threshold", threshold=thr, residual_path=res, output=output)
        got = R.route_scores(cuda(s), "threshold", threshold=thr, residual_path=res,
                             output=output)
        assert np.array_equal(got[1].cpu().numpy(), exp[1]), output
        assert np.array_equal(got[0].cpu().numpy(), exp[0]), output


@pytest.mark.parametrize("T,E,k", [(33, 8, 2), (5000, 32, 2), (2500, 64, 4), (32768, 32, 2)])
def test_renormalised_gates(R, T, E, k):
    s = scores(T, E, 11 * T + E)
    exp = oracle.renormalised_topk_score(s, k)
    got_m, _, got_g = R.route_scores(cuda(s), "topk", k, output="mask", with_gates=True)
    g = got_g.cpu().numpy()
    assert np.array_equal(g != 0, got_m.cpu().numpy() != 0)
    np.testing.assert_allclose(g, exp, rtol=1e-6, atol=0)
    # the same formula in torch (python/brt/router/protocol/swin_moe.py:193-204)
    ts = torch.from_numpy(s)
    vals, picks = torch.topk(ts, k, dim=1)
    ref = torch.zeros_like(ts).scatter_(1, picks, vals / vals.sum(1, keepdim=True).clamp(
        min=torch.finfo(ts.dtype).eps))
    np.testing.assert_allclose(g, ref.numpy(), rtol=1e-6, atol=0)


def test_switch_top1_capacity_mask():
    """The Switch gate's capacity mask (argmax -> one-hot -> cumsum -> <= capacity, per group)
    from the gate kernel, against the torch formula of the reference's model code."""
    from brainstorm_b200.router.protocol.switch import switch_top1_capacity_mask

    torch.manual_seed(5)
    for shape, cap in (((3, 700, 8), 60), ((4096, 32), 100), ((2, 513, 6), 40)):
        probs = torch.softmax(torch.randn(shape, device="cuda") * 2, dim=-1)
        one_hot = torch.nn.functional.one_hot(torch.argmax(probs, dim=-1), num_classes=shape[-1])
        want = one_hot * (torch.cumsum(one_hot, dim=-2) <= cap)
        got = switch_top1_capacity_mask(probs, cap)
        assert got.dtype == torch.int32 and got.shape == probs.shape
        assert torch.equal(got, want.to(torch.int32))


def test_ties_go_to_the_lower_path(R):
    s = np.zeros((40, 8), dtype=np.float32)
    s[:, 5] = 1.0
    got_m, got_l = R.route_scores(cuda(s), "topk", 3, output="mask")
    exp = np.zeros((40, 8), dtype=np.int32)
    exp[:, [5, 0, 1]] = 1
    assert np.array_equal(got_m.cpu().numpy(), exp)
    assert got_l.tolist() == [40, 40, 0, 0, 0, 40, 0, 0]


def test_golden_protocol_vectors(R, golden_dir):
    """Outputs of the reference's own protocol classes (tests/golden/make_golden.py)."""
    z = np.load(golden_dir / "ref_python_vectors.npz")
    score = z["proto/score"]
    if score.shape[1] % 4:
        pytest.skip("golden scores are not a multiple of 4 paths wide")
    for k in (1, 2, 3):
        got_m, _ = R.route_scores(cuda(score), "topk", k, output="mask")
        assert np.array_equal(got_m.cpu().numpy(), z[f"proto/topk{k}"]), k
    sig = z["proto/sigmoid"]
    got_m, _ = R.route_scores(cuda(sig), "threshold", threshold=0.5, output="mask")
    assert np.array_equal(got_m.cpu().numpy(), z["proto/threshold_0.5"])
    got_m, _ = R.route_scores(cuda(sig), "threshold", threshold=0.8, residual_path=3, output="mask")
    assert np.array_equal(got_m.cpu().numpy(), z["proto/threshold_0.8_residual3"])


def test_unsupported_shapes_and_errors(R):
    with pytest.raises(NotImplementedError):
        R.route_scores(torch.rand((16, 6), device="cuda"), "topk", 1)       # 6 paths
    with pytest.raises(NotImplementedError):
        R.route_scores(torch.rand((16, 260), device="cuda"), "topk", 1)     # > 256 paths
    with pytest.raises(RuntimeError):
        R.route_scores(torch.rand((16, 8)), "topk", 1)                      # CPU tensor
    with pytest.raises(RuntimeError):
        R.route_scores(torch.rand((16, 8), device="cuda"), "topk", 9)       # top_k > paths
    with pytest.raises(RuntimeError):
        R.route_scores(torch.rand((16, 8), device="cuda"), "topk", 1, output="throttled_mask")
    m, l = R.route_scores(torch.rand((0, 8), device="cuda"), "topk", 1)
    assert m.shape == (0, 8) and l.tolist() == [0] * 8
