"""Parity of the CUDA router ops (through the C ABI) with the CPU checker.

Integer outputs (indices, loads, masks, tags) and unweighted dispatch are compared bit for
bit; weighted dispatch and combine are compared bit for bit too (the kernels keep the
checker's operation order), which is tighter than the 1e-6 (fp32) / 1e-2 (bf16) relative
tolerance the path is specified with.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


@pytest.fixture(scope="module")
def R():
    from brainstorm_b200._C import router

    return router


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype in ("f16", "bf16"):
        t = t.view(torch.int16).view(DTYPES[dtype])
    return t.cuda()


def host(t):
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def rand_mask(rng, T, E, k):
    return oracle.topk_hot_mask(rng.standard_normal((T, E)).astype(np.float32), k)


@pytest.fixture(params=["auto", "split"])
def index_path(request, monkeypatch):
    """Runs a test once with the library's own choice of index kernels (one chained launch
    whenever it fits) and once with the three-launch variant forced."""
    if request.param == "split":
        monkeypatch.setenv("BRT_INDEX_PATH", "split")
    else:
        monkeypatch.delenv("BRT_INDEX_PATH", raising=False)
    return request.param


INDEX_CASES = [
    # T, E, k
    (16, 4, 2), (1, 1, 1), (31, 2, 1), (33, 3, 2), (1037, 5, 2), (4096, 8, 1), (512, 16, 4),
    (4096, 16, 4), (777, 12, 3), (2048, 32, 2), (1500, 64, 2), (3000, 128, 1), (260, 260, 3),
    (70, 1028, 5), (100000, 8, 1), (300000, 128, 2), (150000, 32, 2), (9000, 512, 2),
]


@pytest.mark.parametrize("T,E,k", INDEX_CASES)
@pytest.mark.parametrize("tag", [False, True])
def test_generate_indices(R, T, E, k, tag, index_path):
    rng = np.random.default_rng(T * 131 + E)
    mask = rand_mask(rng, T, E, k)
    exp_i, exp_l = oracle.generate_indices_and_loads(mask, is_tag_index=tag)
    got_i, got_l = R.generate_indices_and_loads(dev(mask), is_tag_index=tag)
    assert np.array_equal(host(got_l), exp_l)
    assert np.array_equal(host(got_i), exp_i)


@pytest.mark.parametrize("caps,cpad,pwise", [
    ([1, 2, 4, 8, 16, 32, 64, 128, 256, 512], False, False),
    ([1, 2, 4, 8, 16, 32, 64, 128], False, False),
    ([1, 2, 4, 8, 16, 32, 64, 128, 256, 512], True, False),
    ([16, 32, 100], True, False),
    ([2, 4, 8, 16, 32, 64, 128, 256], True, True),
    ([2, 4, 8, 16, 32, 64, 128, 256], False, True),
])
def test_generate_indices_capacities(R, caps, cpad, pwise, index_path):
    rng = np.random.default_rng(len(caps) * 7 + cpad)
    mask = rand_mask(rng, 600, 8, 3)
    mask[:, 5] = 0  # an empty path
    for tag in (False, True):
        exp_i, exp_l = oracle.generate_indices_and_loads(mask, caps, cpad, pwise, tag)
        got_i, got_l = R.generate_indices_and_loads(
            dev(mask), dev(np.array(caps, dtype=np.int32)), cpad, pwise, tag)
        assert np.array_equal(host(got_l), exp_l)
        assert np.array_equal(host(got_i), exp_i)


def test_generate_indices_golden(R, golden_dir):
    z = np.load(golden_dir / "ref_python_vectors.npz")
    names = sorted({k.split("/")[1] for k in z.files if k.startswith("idx/")})
    for name in names:
        caps = z[f"idx/{name}/caps"]
        cpad, pwise = (bool(x) for x in z[f"idx/{name}/flags"])
        for kind in ("seat", "tag"):
            got_i, got_l = R.generate_indices_and_loads(
                dev(z[f"idx/{name}/mask"]), dev(caps) if caps.size else None, cpad, pwise,
                kind == "tag")
            assert np.array_equal(host(got_i), z[f"idx/{name}/{kind}_indices"]), (name, kind)
            assert np.array_equal(host(got_l), z[f"idx/{name}/{kind}_loads"]), (name, kind)


def test_generate_indices_errors_and_empty(R):
    i, l = R.generate_indices_and_loads(torch.zeros((0, 4), dtype=torch.int32, device="cuda"))
    assert i.shape == (0, 4) and l.tolist() == [0, 0, 0, 0]
    with pytest.raises(RuntimeError):
        R.generate_indices_and_loads(torch.zeros((4, 4), dtype=torch.int32))  # CPU tensor
    with pytest.raises(RuntimeError):
        R.generate_indices_and_loads(torch.ones((4, 4), dtype=torch.int32, device="cuda"),
                                     None, True)


def test_generate_indices_general_integers(R, index_path):
    """Masks holding values other than 0/1 follow index = running sum * value
    (src/router/location.cu:176-178)."""
    rng = np.random.default_rng(5)
    mask = rng.integers(0, 4, size=(900, 8)).astype(np.int32)
    exp_i, exp_l = oracle.generate_indices_and_loads(mask)
    got_i, got_l = R.generate_indices_and_loads(dev(mask))
    assert np.array_equal(host(got_i), exp_i) and np.array_equal(host(got_l), exp_l)
    # the binary path must come back on the next call through the same scratch
    mask = rand_mask(rng, 900, 8, 2)
    exp_i, exp_l = oracle.generate_indices_and_loads(mask)
    got_i, got_l = R.generate_indices_and_loads(dev(mask))
    assert np.array_equal(host(got_i), exp_i) and np.array_equal(host(got_l), exp_l)
    # many tiles per CTA, a few non-binary values in only some of them
    mask = rand_mask(rng, 60000, 16, 2)
    mask[rng.integers(0, 60000, size=40), rng.integers(0, 16, size=40)] = 3
    mask[41000, 3] = -2
    exp_i, exp_l = oracle.generate_indices_and_loads(mask)
    got_i, got_l = R.generate_indices_and_loads(dev(mask))
    assert np.array_equal(host(got_l), exp_l)
    assert np.array_equal(host(got_i), exp_i)


def test_generate_indices_unaligned_view(R):
    """A mask whose storage offset breaks 16-byte alignment takes the narrow-vector path."""
    rng = np.random.default_rng(9)
    mask = rand_mask(rng, 500, 8, 2)
    flat = torch.zeros(500 * 8 + 1, dtype=torch.int32, device="cuda")
    view = flat[1:].view(500, 8)
    view.copy_(dev(mask))
    exp_i, exp_l = oracle.generate_indices_and_loads(mask)
    got_i, got_l = R.generate_indices_and_loads(view)
    assert np.array_equal(host(got_i), exp_i) and np.array_equal(host(got_l), exp_l)


def test_throttle_golden(R, golden_dir):
    import json

    v = json.load(open(golden_dir / "notebook_vectors.json"))["throttle"]
    prefix = dev(np.array(v["prefix_in"], dtype=np.int32))
    out, p2 = R.throttle_hotmask(dev(np.array(v["hot_mask"], dtype=np.int32)), prefix,
                                 dev(np.array(v["threshold"], dtype=np.int32)))
    assert p2 is prefix
    assert host(out).tolist() == v["throttled_mask"]
    assert host(prefix).tolist() == v["prefix_out"]


@pytest.mark.parametrize("T,E,k", [(16, 4, 2), (1037, 5, 2), (5000, 32, 2), (3000, 128, 1),
                                   (40000, 8, 2), (200000, 64, 2)])
def test_throttle(R, T, E, k, index_path):
    rng = np.random.default_rng(T + E)
    mask = rand_mask(rng, T, E, k)
    prefix = rng.integers(0, 20, size=E).astype(np.int32)
    thr = rng.integers(0, max(2, 2 * T * k // E), size=E).astype(np.int32)
    exp_p = prefix.copy()
    exp_m, _ = oracle.throttle_hotmask(mask, exp_p, thr)
    p = dev(prefix)
    got_m, got_p = R.throttle_hotmask(dev(mask), p, dev(thr))
    assert np.array_equal(host(got_m), exp_m)
    assert np.array_equal(host(got_p), exp_p)


FUSED_CASES = [(16, 4, 2), (1037, 8, 2), (5000, 32, 2), (3000, 128, 1), (40000, 8, 2),
               (200000, 64, 2), (32768, 32, 2), (262144, 128, 1), (777, 12, 3), (50, 6, 2)]


@pytest.mark.parametrize("T,E,k", FUSED_CASES)
@pytest.mark.parametrize("caps_mode", ["none", "list", "padding", "path_wise"])
def test_throttle_and_generate_indices(R, T, E, k, caps_mode):
    """One pass = throttle_hotmask then generate_indices_and_loads of the throttled mask
    (E = 6 is not a multiple of 4: the wrapper takes the two ops there)."""
    rng = np.random.default_rng(3 * T + E)
    mask = rand_mask(rng, T, E, k)
    prefix = rng.integers(0, 20, size=E).astype(np.int32)
    thr = rng.integers(0, max(2, 2 * T * k // E), size=E).astype(np.int32)
    if caps_mode == "none":
        caps, cpad, pwise = None, False, False
    elif caps_mode == "list":
        caps, cpad, pwise = [8, 64, 512, 4096], False, False
    elif caps_mode == "padding":
        caps, cpad, pwise = [8, 64, 512, 4096], True, False
    else:
        caps, cpad, pwise = list(rng.integers(1, 5000, size=E)), True, True
    exp_p = prefix.copy()
    exp_m, _ = oracle.throttle_hotmask(mask, exp_p, thr)
    exp_i, exp_l = oracle.generate_indices_and_loads(exp_m, caps, cpad, pwise)
    p = dev(prefix)
    got_i, got_l, got_p = R.throttle_and_generate_indices(
        dev(mask), p, dev(thr), None if caps is None else dev(np.array(caps, dtype=np.int32)),
        cpad, pwise)
    assert got_p is p
    assert np.array_equal(host(got_p), exp_p)
    assert np.array_equal(host(got_l), exp_l)
    assert np.array_equal(host(got_i), exp_i)


def test_throttle_and_generate_indices_golden(R, golden_dir):
    import json

    v = json.load(open(golden_dir / "notebook_vectors.json"))["throttle"]
    prefix = dev(np.array(v["prefix_in"], dtype=np.int32))
    idx, loads, p2 = R.throttle_and_generate_indices(
        dev(np.array(v["hot_mask"], dtype=np.int32)), prefix,
        dev(np.array(v["threshold"], dtype=np.int32)))
    want_i, want_l = oracle.generate_indices_and_loads(
        np.array(v["throttled_mask"], dtype=np.int32))
    assert host(prefix).tolist() == v["prefix_out"]
    assert np.array_equal(host(idx), want_i) and np.array_equal(host(loads), want_l)


def test_fused_scan_refuses_other_mask_values(R):
    """The fused pass is defined for 0/1 masks; another value is reported, not guessed at."""
    from brainstorm_b200 import _lib

    mask = torch.zeros((4096, 8), dtype=torch.int32, device="cuda")
    mask[17, 3] = 5
    E = 8
    R.throttle_and_generate_indices(mask, torch.zeros(E, dtype=torch.int32, device="cuda"),
                                    torch.full((E,), 9, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert _lib.query("brt_index_status") == 1  # BRT_ERR_INVALID_ARGUMENT
    _lib.query("brt_index_status_reset")


def test_convert_index_format(R):
    rng = np.random.default_rng(11)
    mask = rand_mask(rng, 3000, 6, 2)
    seat, loads = oracle.generate_indices_and_loads(mask)
    tag, _ = oracle.generate_indices_and_loads(mask, is_tag_index=True)
    # flag forwarded inverted, as in the reference: False = seat -> tag
    got_tag = R.convert_index_format(dev(seat), dev(loads), False)
    assert np.array_equal(host(got_tag), tag)
    got_seat = R.convert_index_format(dev(tag), dev(loads), True)
    assert np.array_equal(host(got_seat), seat)
    assert np.array_equal(host(got_seat), oracle.convert_index_format(tag, loads, True))


def make_data(rng, shape, dtype):
    return oracle.to_bits(rng.standard_normal(shape).astype(np.float32), dtype)


DISPATCH_CASES = [
    # T, E, k, cell shape
    (16, 4, 2, (8,)), (300, 8, 1, (768,)), (257, 5, 2, (3,)), (200, 8, 2, (4, 3, 2, 3)),
    (128, 16, 2, (1024,)), (64, 4, 2, (2050,)), (37, 3, 1, (1,)), (50, 130, 3, (64,)),
]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("T,E,k,cell", DISPATCH_CASES)
@pytest.mark.parametrize("variant", ["plain", "padded", "capacity", "weighted", "tags"])
def test_dispatch_and_combine(R, dtype, T, E, k, cell, variant):
    if dtype == "f16" and int(np.prod(cell)) % 2:
        pytest.skip("the reference requires an even cell size for fp16")
    rng = np.random.default_rng(T * 7 + E + len(variant))
    mask = rand_mask(rng, T, E, k)
    caps, cpad = None, False
    kw = {}
    if variant == "capacity":
        caps, cpad = [max(1, T * k // E // 2)], True  # forces drops and padding
    idx, loads = oracle.generate_indices_and_loads(mask, caps, cpad)
    if variant == "padded":
        kw = dict(max_path_padding=True, max_path_load=int(loads.max()) + 3)
    x = make_data(rng, (T,) + cell, dtype)
    gates = make_data(rng, (T, E), dtype) if variant == "weighted" else None
    tagging = variant == "tags"
    exp = oracle.dispatch_with_indices_and_loads(x, idx, loads, gates, tagging, None,
                                                 dtype=dtype, **kw)
    got = R.dispatch_with_indices_and_loads(
        dev(x, dtype), dev(idx), dev(loads), None if gates is None else dev(gates, dtype),
        tagging, None, **kw)
    assert len(got) == len(exp)
    assert got[0].shape == exp[0].shape
    assert np.array_equal(host(got[0]), exp[0])
    if tagging:
        assert np.array_equal(host(got[1]), exp[1])
    # combine what was dispatched, with fp32 gates, with and without a residual
    g32 = rng.standard_normal((T, E)).astype(np.float32)
    ckw = dict(max_path_padding=kw.get("max_path_padding", False))
    for use_gates in (False, True):
        (exp_c,) = oracle.combine_with_indices_and_loads(
            exp[0], idx, loads, g32 if use_gates else None, dtype=dtype, **ckw)
        (got_c,) = R.combine_with_indices_and_loads(
            got[0], dev(idx), dev(loads), dev(g32) if use_gates else None, **ckw)
        assert np.array_equal(host(got_c), exp_c)
    res = make_data(rng, (T,) + cell, dtype)
    exp_res = res.copy()
    oracle.combine_with_indices_and_loads(exp[0], idx, loads, g32, out_data=exp_res, dtype=dtype,
                                          **ckw)
    res_d = dev(res, dtype)
    (got_res,) = R.combine_with_indices_and_loads(got[0], dev(idx), dev(loads), dev(g32), res_d,
                                                  **ckw)
    assert got_res is res_d
    assert np.array_equal(host(res_d), exp_res)


def poison_allocator(nbytes):
    """Fill a block with a NaN pattern and hand it back to torch's allocator, so that an output
    the next call leaves partly unwritten shows up as garbage, not as stale zeros."""
    junk = torch.full((max(nbytes, 1024) // 4 + 64,), float("nan"), device="cuda")
    del junk


DENSE_VARIANTS = ["plain", "padded", "padded_capacity", "capped", "throttled", "weighted",
                  "tags", "2d"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("T,E,k,cell", DISPATCH_CASES + [(3000, 32, 2, (1024,)),
                                                         (2000, 8, 1, (2600,))])
@pytest.mark.parametrize("variant", DENSE_VARIANTS)
def test_dispatch_of_library_made_indices(R, dtype, T, E, k, cell, variant):
    """Indices that come straight out of the index kernels carry the per-path cell counts, and
    the dispatch runs as one launch that zeroes the empty rows from those counts alone.  The
    result must equal the checker's whatever the relation between counts, loads and slot size:
    loads above the counts (capacity padding), below them (capped), slots above the loads."""
    from brainstorm_b200._C.router import _DENSE

    rng = np.random.default_rng(T * 5 + E + len(variant))
    mask = rand_mask(rng, T, E, k)
    caps, cpad, kw = None, False, {}
    per_path = max(1, T * k // E)
    if variant == "padded_capacity":
        caps, cpad = [per_path // 2, 2 * per_path, 8 * per_path], True
    elif variant == "capped":
        caps, cpad = [max(1, per_path // 2)], False  # loads capped below the counts: drops
    mask_d = dev(mask)
    if variant == "throttled":
        thr = rng.integers(0, 2 * per_path, size=E).astype(np.int32)
        m_np, _ = oracle.throttle_hotmask(mask, np.zeros(E, dtype=np.int32), thr)
        idx_np, loads_np = oracle.generate_indices_and_loads(m_np)
        idx, loads, _ = R.throttle_and_generate_indices(
            mask_d, torch.zeros(E, dtype=torch.int32, device="cuda"), dev(thr))
    else:
        idx_np, loads_np = oracle.generate_indices_and_loads(mask, caps, cpad)
        idx, loads = R.generate_indices_and_loads(
            mask_d, None if caps is None else dev(np.array(caps, dtype=np.int32)), cpad)
    assert getattr(idx, _DENSE, None) is not None
    if variant in ("padded", "padded_capacity", "throttled"):
        kw = dict(max_path_padding=True, max_path_load=int(loads_np.max()) + 5)
    is_1d = variant != "2d"
    x = make_data(rng, (T,) + cell if is_1d else (T, E) + cell[:1], dtype)
    gates = make_data(rng, (T, E), dtype) if variant == "weighted" else None
    tagging = variant == "tags"
    exp = oracle.dispatch_with_indices_and_loads(x, idx_np, loads_np, gates, tagging, None,
                                                 is_1d_routing=is_1d, dtype=dtype, **kw)
    poison_allocator(exp[0].size * exp[0].itemsize)
    got = R.dispatch_with_indices_and_loads(
        dev(x, dtype), idx, loads, None if gates is None else dev(gates, dtype), tagging, None,
        kw.get("max_path_padding", False), kw.get("max_path_load", 0), is_1d)
    assert got[0].shape == exp[0].shape
    assert np.array_equal(host(got[0]), exp[0])
    if tagging:
        assert np.array_equal(host(got[1]), exp[1])
    # an index tensor that lost the note (a clone) takes the general route: same rows
    again = R.dispatch_with_indices_and_loads(
        dev(x, dtype), idx.clone(), loads, None if gates is None else dev(gates, dtype), tagging,
        None, kw.get("max_path_padding", False), kw.get("max_path_load", 0), is_1d)
    assert np.array_equal(host(again[0]), exp[0])


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_combine_gates_in_data_dtype(R, dtype):
    rng = np.random.default_rng(2)
    T, E = 500, 8
    idx, loads = oracle.generate_indices_and_loads(rand_mask(rng, T, E, 2))
    x = make_data(rng, (int(loads.sum()), 96), dtype)
    g = make_data(rng, (T, E), dtype)
    (exp,) = oracle.combine_with_indices_and_loads(x, idx, loads, g, dtype=dtype,
                                                   gates_dtype=dtype)
    (got,) = R.combine_with_indices_and_loads(dev(x, dtype), dev(idx), dev(loads), dev(g, dtype))
    assert np.array_equal(host(got), exp)


def test_dispatch_2d_scores(R):
    rng = np.random.default_rng(4)
    T, E = 700, 8
    idx, loads = oracle.generate_indices_and_loads(rand_mask(rng, T, E, 2))
    score = rng.standard_normal((T, E)).astype(np.float32)
    (exp,) = oracle.dispatch_with_indices_and_loads(score, idx, loads, is_1d_routing=False)
    (got,) = R.dispatch_with_indices_and_loads(dev(score), dev(idx), dev(loads),
                                               is_1d_routing=False)
    assert got.shape == exp.shape == (int(loads.sum()), 1)
    assert np.array_equal(host(got), exp)
    x3 = rng.standard_normal((T, E, 6)).astype(np.float32)
    exp = oracle.dispatch_with_indices_and_loads(x3, idx, loads, tag_generating=True,
                                                 is_1d_routing=False)
    got = R.dispatch_with_indices_and_loads(dev(x3), dev(idx), dev(loads), None, True, None,
                                            False, 0, False)
    assert np.array_equal(host(got[0]), exp[0]) and np.array_equal(host(got[1]), exp[1])


@pytest.mark.parametrize("weighted", [False, True])
def test_dispatch_with_tag_indices(R, weighted):
    rng = np.random.default_rng(6)
    T, E = 900, 6
    mask = rand_mask(rng, T, E, 2)
    tag, loads = oracle.generate_indices_and_loads(mask, [64, 128, 256, 512], True, False, True)
    x = rng.standard_normal((T, 40)).astype(np.float32)
    g = rng.standard_normal((T, E)).astype(np.float32) if weighted else None
    for kw in ({}, dict(max_path_padding=True, max_path_load=600)):
        exp = oracle.dispatch_with_indices_and_loads(x, tag, loads, g, True, None,
                                                     is_tag_index=True, **kw)
        got = R.dispatch_with_indices_and_loads(
            dev(x), dev(tag), dev(loads), None if g is None else dev(g), True, None,
            kw.get("max_path_padding", False), kw.get("max_path_load", 0), True, True)
        assert np.array_equal(host(got[0]), exp[0]) and np.array_equal(host(got[1]), exp[1])


def test_dispatch_2d_with_tag_indices(R):
    """Tag-index routing of a [cell, path, ...] input: row i of path e pulls cell tag-1 from
    that path's own slice (src/router/route.cu:161-206)."""
    rng = np.random.default_rng(8)
    T, E = 640, 8
    mask = rand_mask(rng, T, E, 3)
    tag, loads = oracle.generate_indices_and_loads(mask, None, False, False, True)
    for cell in (1, 6):
        x = rng.standard_normal((T, E, cell)).astype(np.float32)
        for kw in ({}, dict(max_path_padding=True, max_path_load=400)):
            exp = oracle.dispatch_with_indices_and_loads(x, tag, loads, None, True, None,
                                                         is_1d_routing=False, is_tag_index=True,
                                                         **kw)
            got = R.dispatch_with_indices_and_loads(
                dev(x), dev(tag), dev(loads), None, True, None,
                kw.get("max_path_padding", False), kw.get("max_path_load", 0), False, True)
            assert got[0].shape == exp[0].shape
            assert np.array_equal(host(got[0]), exp[0]), (cell, kw)
            assert np.array_equal(host(got[1]), exp[1]), (cell, kw)


def test_index_scan_reports_a_wait_that_ran_out(R):
    """The single-launch scan lets a CTA wait for the column sums of earlier CTAs.  With the
    test hooks the first run of tiles has no owner and a wait gives up after 50 polls: the
    kernel must return (no hang), and the status word, then the next index op, must say so."""
    from brainstorm_b200 import _lib

    rng = np.random.default_rng(11)
    mask = dev(rand_mask(rng, 150000, 32, 2))
    good = R.generate_indices_and_loads(mask)
    torch.cuda.synchronize()
    assert _lib.query("brt_index_status") == 0
    _lib.query("brt_index_set_test_hooks", 50, 1)
    try:
        R.generate_indices_and_loads(mask)
        torch.cuda.synchronize()  # returns: every wait is bounded
        assert _lib.query("brt_index_status") == 7  # BRT_ERR_TIMEOUT
    finally:
        _lib.query("brt_index_set_test_hooks", 0, 0)
    with pytest.raises(_lib.BrtError) as err:
        R.generate_indices_and_loads(mask)
    assert err.value.status == 7
    again = R.generate_indices_and_loads(mask)  # reported once; the library keeps working
    assert torch.equal(again[0], good[0]) and torch.equal(again[1], good[1])


def test_dispatch_empty_and_single(R):
    x = torch.zeros((0, 5), device="cuda")
    idx = torch.zeros((0, 3), dtype=torch.int32, device="cuda")
    loads = torch.zeros((3,), dtype=torch.int32, device="cuda")
    (o,) = R.dispatch_with_indices_and_loads(x, idx, loads)
    assert o.shape == (0, 5)
    o, t = R.dispatch_with_indices_and_loads(x, idx, loads, None, True)
    assert o.shape == (0, 5) and t.shape == (0,)
    (o,) = R.combine_with_indices_and_loads(x, idx, loads)
    assert o.shape == (0, 5)
    # single-cell shortcut: data returned as is / added to the residual
    one = torch.randn((1, 5), device="cuda")
    idx1 = torch.ones((1, 3), dtype=torch.int32, device="cuda")
    (o,) = R.combine_with_indices_and_loads(one, idx1, loads)
    assert o is one
    res = torch.ones((1, 5), device="cuda")
    (o,) = R.combine_with_indices_and_loads(one, idx1, loads, None, res)
    assert torch.equal(o, res + one)


def test_path_wise_padding_with_no_cells_routed(R):
    """Every output row is padding: the whole output must come back zero."""
    mask = np.zeros((10, 4), dtype=np.int32)
    caps = np.array([3, 0, 2, 5], dtype=np.int32)
    idx, loads = oracle.generate_indices_and_loads(mask, caps, True, True)
    x = np.ones((10, 7), dtype=np.float32)
    (exp,) = oracle.dispatch_with_indices_and_loads(x, idx, loads)
    (got,) = R.dispatch_with_indices_and_loads(dev(x), dev(idx), dev(loads))
    assert got.shape == (10, 7) and np.array_equal(host(got), exp) and not host(got).any()


def test_notebook_round_trip(R):
    """sample/cpp/dispatch.ipynb: both combine paths return 2*x for a top-2 mask."""
    rng = np.random.default_rng(1)
    T, E = 2048, 4
    mask = dev(rand_mask(rng, T, E, 2))
    caps = torch.tensor([64, 128, 256, 512, 1024, 2048], dtype=torch.int32, device="cuda")
    idx, loads = R.generate_indices_and_loads(mask, caps, capacity_padding=True)
    x = torch.randn((T, 4, 3, 2, 3), device="cuda")
    out, tags = R.dispatch_with_indices_and_loads(x, idx, loads, tag_generating=True)
    datas, sloads, stags = R.split_fused_cells_to_paths(out, loads, is_load_split=True,
                                                        is_tag_split=True, tags=tags)
    fused, new_tags, inverse = R.fuse_split_cells_from_paths(datas, is_tag_fuse=True, tags=stags)
    final, ftags, n = R.combine_with_indices_and_loads(fused, inverse, loads, tags=new_tags,
                                                       is_tag_index=True)
    assert n.item() == T and torch.equal(final, 2 * x)
    fused2, floads = R.fuse_split_cells_from_paths(datas, is_load_fuse=True, loads=sloads)
    (final2,) = R.combine_with_indices_and_loads(fused2, idx, floads)
    assert torch.equal(final2, 2 * x)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows_in,rows_out,cell", [(1, 1, 8), (37, 9, 3), (300, 40, 24),
                                                   (5000, 1200, 64), (256, 64, 4100),
                                                   (20000, 20000, 16)])
def test_tag_combine_sums_rows_in_source_order(R, dtype, rows_in, rows_out, cell):
    """Tag-index combine (src/backend/torch/router.cc:449-459): rows that share an inverse
    index are added up; this library adds them in ascending source order, in fp32, which the
    plain loop below restates."""
    rng = np.random.default_rng(rows_in + rows_out + cell)
    x32 = rng.standard_normal((rows_in, cell)).astype(np.float32)
    index = rng.integers(0, rows_out, size=rows_in).astype(np.int64)
    if rows_out > 2:
        index[index == 1] = 0                      # destination 1 gets nothing
    tags = np.arange(1, rows_out + 1, dtype=np.int32)
    x = torch.from_numpy(x32).to(DTYPES[dtype]).cuda()
    exp = np.zeros((rows_out, cell), dtype=np.float32)
    xs = x.float().cpu().numpy()
    for r in range(rows_in):
        exp[index[r]] = exp[index[r]] + xs[r]
    exp_t = torch.from_numpy(exp).to(DTYPES[dtype])
    out, otags, n = R.combine_with_indices_and_loads(
        x, torch.from_numpy(index).cuda(), None, tags=torch.from_numpy(tags).cuda(),
        is_tag_index=True, ever_padded=False)
    assert n.item() == rows_out and torch.equal(otags.cpu(), torch.from_numpy(tags))
    assert out.shape == (rows_out, cell)
    assert torch.equal(out.cpu().view(torch.int16 if dtype != "f32" else torch.int32),
                       exp_t.view(torch.int16 if dtype != "f32" else torch.int32))
