"""Pins the CPU checker (oracle/) to the reference's own recorded behaviour.

Sources of truth, all produced by tests/golden/make_golden.py from the reference tree:
  * saved cell outputs of sample/router/generate_indices.ipynb (seat indices, throttle);
  * the reference's torch oracle test/python/fabric_test.py:35-92 run on seeded masks;
  * the reference's protocol classes run on CPU tensors;
plus the identities its samples assert (sample/cpp/dispatch.ipynb round trip == 2*x,
sample/distributed/sparse_a2a.py round trip == identity).
"""
import json

import numpy as np
import pytest

import oracle


@pytest.fixture(scope="module")
def nb(golden_dir):
    return json.load(open(golden_dir / "notebook_vectors.json"))


@pytest.fixture(scope="module")
def refpy(golden_dir):
    return np.load(golden_dir / "ref_python_vectors.npz")


def test_notebook_seat_indices(nb):
    v = nb["indices"]
    mask = np.array(v["hot_mask"], dtype=np.int32)
    idx, loads = oracle.generate_indices_and_loads(mask)
    assert np.array_equal(idx, np.array(v["seat_indices"], dtype=np.int32))
    assert loads.tolist() == v["shuffled_loads"] == [10, 3, 11, 11]


def test_notebook_tag_indices_are_legacy_plus_one(nb):
    """The notebook was saved with an older API whose tag ("src") indices were 0-based; the
    current kernels write cell+1 (src/router/location.cu:182).  Within each path's load the
    saved values + 1 must equal today's tag indices."""
    v = nb["indices"]
    mask = np.array(v["hot_mask"], dtype=np.int32)
    tag, loads = oracle.generate_indices_and_loads(mask, is_tag_index=True)
    legacy = np.array(v["legacy_src_indices_zero_based"], dtype=np.int32)
    for e in range(mask.shape[1]):
        n = loads[e]
        assert np.array_equal(tag[:n, e], legacy[:n, e] + 1)
        assert not tag[n:, e].any()


def test_notebook_convert_shuffled(nb):
    v = nb["indices"]
    shuffled = np.array(v["shuffled_seat_indices"], dtype=np.int32)
    loads = np.array(v["shuffled_loads"], dtype=np.int32)
    legacy = np.array(v["legacy_converted_zero_based"], dtype=np.int32)
    # seat -> tag is the launcher's tag_to_seat == False branch, i.e. is_to_tag=False at the
    # binding (the flag is forwarded inverted, src/backend/torch/router.cc:106-108)
    tag = oracle.convert_index_format(shuffled, loads, is_to_tag=False)
    for e in range(shuffled.shape[1]):
        n = loads[e]
        assert np.array_equal(tag[:n, e], legacy[:n, e] + 1)
    back = oracle.convert_index_format(tag, loads, is_to_tag=True)
    assert np.array_equal(back, shuffled)


def test_notebook_throttle(nb):
    v = nb["throttle"]
    mask = np.array(v["hot_mask"], dtype=np.int32)
    assert mask.sum(0).tolist() == v["column_sums"]
    prefix = np.array(v["prefix_in"], dtype=np.int32)
    out, prefix_out = oracle.throttle_hotmask(mask, prefix, np.array(v["threshold"]))
    assert np.array_equal(out, np.array(v["throttled_mask"], dtype=np.int32))
    assert out.sum(0).tolist() == v["kept_counts"] == [5, 1, 3, 5]
    assert prefix_out.tolist() == v["prefix_out"] == [6, 3, 7, 8]
    assert prefix is prefix_out  # mutated in place like the reference


def _idx_cases(refpy):
    return sorted({k.split("/")[1] for k in refpy.files if k.startswith("idx/")})


def test_reference_torch_oracle_cases(refpy):
    names = _idx_cases(refpy)
    assert len(names) >= 8
    for name in names:
        mask = refpy[f"idx/{name}/mask"]
        caps = refpy[f"idx/{name}/caps"]
        cpad, pwise = (bool(x) for x in refpy[f"idx/{name}/flags"])
        caps_arg = caps if caps.size else None
        for kind in ("seat", "tag"):
            idx, loads = oracle.generate_indices_and_loads(
                mask, caps_arg, cpad, pwise, is_tag_index=(kind == "tag"))
            assert np.array_equal(idx, refpy[f"idx/{name}/{kind}_indices"]), (name, kind)
            assert np.array_equal(loads, refpy[f"idx/{name}/{kind}_loads"]), (name, kind)
            idx2, loads2 = oracle.generate_indices_and_loads_numpy(
                mask, caps_arg, cpad, pwise, is_tag_index=(kind == "tag"))
            assert np.array_equal(idx, idx2) and np.array_equal(loads, loads2)


def test_reference_protocols(refpy):
    score = refpy["proto/score"]
    for k in (1, 2, 3):
        assert np.array_equal(oracle.topk_hot_mask(score, k), refpy[f"proto/topk{k}"])
    sig = refpy["proto/sigmoid"]
    assert np.array_equal(oracle.threshold_hot_mask(sig, 0.5), refpy["proto/threshold_0.5"])
    assert np.array_equal(oracle.threshold_hot_mask(sig, 0.8, 3),
                          refpy["proto/threshold_0.8_residual3"])


def test_loads_corner_cases():
    """Kernel rules the reference's torch oracle does not reach
    (src/router/location.cu:227-254)."""
    mask = np.zeros((8, 3), dtype=np.int32)
    mask[:, 0] = 1          # load 8
    mask[:3, 2] = 1         # load 3, path 1 empty
    caps = [2, 4]
    # empty path stays 0 under capacity_padding, overflow maps to the last capacity
    _, l = oracle.generate_indices_and_loads(mask, caps, capacity_padding=True)
    assert l.tolist() == [4, 0, 4]
    # path-wise padding reports the path's capacity even for an empty path
    _, l = oracle.generate_indices_and_loads(mask, [5, 6, 7], True, True)
    assert l.tolist() == [5, 6, 7]
    # no padding + capacities: real load if it fits, else last capacity
    _, l = oracle.generate_indices_and_loads(mask, caps)
    assert l.tolist() == [4, 0, 3]
    # path_wise_padding without capacity_padding is ignored by the launcher
    _, l = oracle.generate_indices_and_loads(mask, [5, 6, 7], False, True)
    assert l.tolist() == [7, 0, 3]
    with pytest.raises(RuntimeError):
        oracle.generate_indices_and_loads(mask, None, capacity_padding=True)
    i, l = oracle.generate_indices_and_loads(np.zeros((0, 4), dtype=np.int32))
    assert i.shape == (0, 4) and l.tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_dispatch_notebook_round_trip(dtype):
    """sample/cpp/dispatch.ipynb: top-2 mask, capacity_padding, tag-generating dispatch ->
    split -> fuse(tags) -> tag combine == 2*x, and fuse(loads) -> seat combine == 2*x."""
    rng = np.random.default_rng(7)
    T, E = 2048, 4
    score = rng.standard_normal((T, E)).astype(np.float32)
    mask = oracle.topk_hot_mask(score, 2)
    caps = [64, 128, 256, 512, 1024, 2048]
    idx, loads = oracle.generate_indices_and_loads(mask, caps, capacity_padding=True)
    assert all(int(l) in caps for l in loads)
    x32 = rng.standard_normal((T, 4, 3, 2, 3)).astype(np.float32)
    x = oracle.to_bits(x32, dtype)
    x32 = oracle.from_bits(x, dtype)
    out, tags = oracle.dispatch_with_indices_and_loads(x, idx, loads, tag_generating=True,
                                                       dtype=dtype)
    assert out.shape[0] == loads.sum()
    datas, sloads, stags = oracle.split_fused_cells_to_paths(
        out, loads, is_load_split=True, is_tag_split=True, tags=tags)
    fused, new_tags, inverse = oracle.fuse_split_cells_from_paths(datas, is_tag_fuse=True,
                                                                  tags=stags)
    assert new_tags.tolist() == list(range(0, T + 1))
    final, ftags, n = oracle.combine_with_indices_and_loads(
        fused, inverse, None, tags=new_tags, is_tag_index=True, dtype=dtype)
    assert n.tolist() == [T] and ftags.tolist() == list(range(1, T + 1))
    assert np.array_equal(oracle.from_bits(final, dtype), 2 * x32)
    fused2, floads = oracle.fuse_split_cells_from_paths(datas, is_load_fuse=True, loads=sloads)
    (final2,) = oracle.combine_with_indices_and_loads(fused2, idx, floads, dtype=dtype)
    assert np.array_equal(oracle.from_bits(final2, dtype), 2 * x32)


def test_dispatch_rows_and_drop():
    """Row addressing and the drop rule (src/router/route.cu:26-43)."""
    mask = np.array([[1, 0], [1, 1], [1, 1], [0, 1], [1, 0]], dtype=np.int32)
    idx, loads = oracle.generate_indices_and_loads(mask, [2], capacity_padding=True)
    assert loads.tolist() == [2, 2]  # path 0 has 4 cells: seats 3, 4 are dropped
    x = np.arange(10, dtype=np.float32).reshape(5, 2) + 1
    (out,) = oracle.dispatch_with_indices_and_loads(x, idx, loads)
    assert out.tolist() == [[1, 2], [3, 4], [3, 4], [5, 6]]
    (out,) = oracle.dispatch_with_indices_and_loads(x, idx, loads, max_path_padding=True,
                                                    max_path_load=3)
    assert out.tolist() == [[1, 2], [3, 4], [0, 0], [3, 4], [5, 6], [0, 0]]
    g = np.full((5, 2), 0.5, dtype=np.float32)
    (back,) = oracle.combine_with_indices_and_loads(out, idx, loads, gates=g,
                                                    max_path_padding=True)
    assert back.tolist() == [[0.5, 1], [3, 4], [2.5, 3], [0, 0], [0, 0]]
    res = np.full((5, 2), 9, dtype=np.float32)
    (back,) = oracle.combine_with_indices_and_loads(out, idx, loads, out_data=res,
                                                    max_path_padding=True)
    assert back is res and res.tolist() == [[1, 2], [6, 8], [5, 6], [9, 9], [9, 9]]


def test_dispatch_2d_routes_scores():
    """2-D routing picks element e of cell t for path e (src/router/route.cu:116-158), as used
    to route the score matrix itself (python/brt/router/scatter.py:86-89)."""
    mask = np.array([[1, 1], [0, 1], [1, 0]], dtype=np.int32)
    idx, loads = oracle.generate_indices_and_loads(mask)
    score = np.array([[0.1, 0.2], [0.3, 0.4], [0.5, 0.6]], dtype=np.float32)
    (out,) = oracle.dispatch_with_indices_and_loads(score, idx, loads, is_1d_routing=False)
    assert out.shape == (4, 1)
    assert np.allclose(out[:, 0], [0.1, 0.5, 0.2, 0.4])


def test_tag_dispatch_matches_seat_dispatch():
    rng = np.random.default_rng(3)
    mask = oracle.topk_hot_mask(rng.standard_normal((700, 6)).astype(np.float32), 2)
    seat, loads = oracle.generate_indices_and_loads(mask)
    tag, loads_t = oracle.generate_indices_and_loads(mask, is_tag_index=True)
    assert np.array_equal(loads, loads_t)
    x = rng.standard_normal((700, 5)).astype(np.float32)
    g = rng.standard_normal((700, 6)).astype(np.float32)
    a = oracle.dispatch_with_indices_and_loads(x, seat, loads, gates=g, tag_generating=True)
    b = oracle.dispatch_with_indices_and_loads(x, tag, loads, gates=g, tag_generating=True,
                                               is_tag_index=True)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_locality_reorder_rules():
    """src/distributed/local_reorder.cu:15-63: greedy arg-max, smallest flat index on ties,
    output column c = input column reorder[c]."""
    m = np.array([[5, 1, 9], [9, 2, 3], [4, 8, 9]], dtype=np.int32)
    out, idx = oracle.locality_reorder(m, 3)
    # pick 1: max 9 first at (0,2) -> reorder[0]=2; pick 2: remaining rows 1,2 x cols 0,1:
    # max 9 at (1,0) -> reorder[1]=0; pick 3: (2,1) -> reorder[2]=1
    assert idx.tolist() == [2, 0, 1]
    assert np.array_equal(out, m[:, [2, 0, 1]])
    eye = np.eye(4, dtype=np.int32) * 7
    out, idx = oracle.locality_reorder(eye, 4)
    assert idx.tolist() == [0, 1, 2, 3] and np.array_equal(out, eye)
    # all equal: ties resolve to the smallest flat index each round -> identity
    out, idx = oracle.locality_reorder(np.ones((4, 4), dtype=np.int32), 4)
    assert idx.tolist() == [0, 1, 2, 3]
    g = np.array([[[0, 1], [6, 7]], [[8, 9], [2, 3]]], dtype=np.int32)
    out, idx = oracle.group_locality_reorder(g, 2, 2)
    assert idx.tolist() == [1, 0] and np.array_equal(out, g[:, [1, 0], :])


def test_sparse_a2a_sample_round_trip():
    """sample/distributed/sparse_a2a.py: 2 ranks, 2 local experts, literal loads; forward then
    size-known backward restores every rank's input."""
    rng = np.random.default_rng(0)
    loads = [np.array([3, 2, 4, 4, 2, 4, 5, 2][:4], dtype=np.int32),
             np.array([1, 22, 3, 4], dtype=np.int32)]
    # the sample passes 8 sizes per rank on 2 ranks (G = 4); keep its literal vectors too
    for sizes in (loads, [np.array([3, 2, 4, 4, 2, 4, 5, 2], dtype=np.int32),
                          np.array([1, 22, 3, 4, 3, 55, 222, 1], dtype=np.int32)]):
        xs = [rng.standard_normal((int(s.sum()), 3)).astype(np.float32) for s in sizes]
        fwd = oracle.sim_group_sparse_all_to_all(xs, sizes)
        W = 2
        G = sizes[0].size // W
        for me, (out, recv, send) in enumerate(fwd):
            assert np.array_equal(send, sizes[me])
            expect = np.stack([sizes[i].reshape(W, G)[me] for i in range(W)]).T.reshape(-1)
            assert np.array_equal(recv, expect)
            assert out.shape[0] == recv.sum()
        back = oracle.sim_size_known_group_sparse_all_to_all(
            [f[0] for f in fwd], [f[1] for f in fwd], [f[2] for f in fwd])
        for me in range(W):
            assert np.array_equal(back[me], xs[me])
        # padded variant
        mpl = int(max(s.max() for s in sizes))
        xs_p = []
        for s in sizes:
            buf = np.zeros((mpl * s.size, 3), dtype=np.float32)
            for b, n in enumerate(s):
                buf[b * mpl:b * mpl + n] = rng.standard_normal((int(n), 3))
            xs_p.append(buf)
        fwd = oracle.sim_group_sparse_all_to_all(xs_p, sizes, True, mpl)
        back = oracle.sim_size_known_group_sparse_all_to_all(
            [f[0] for f in fwd], [f[1] for f in fwd], [f[2] for f in fwd], True)
        for me in range(W):
            assert np.array_equal(back[me], xs_p[me])


def test_route_scores_checker_matches_reference_protocols(golden_dir):
    """oracle.route_scores composes a protocol with the index functions; its masks must be the
    ones the reference's protocol classes produced (tests/golden/make_golden.py)."""
    z = np.load(golden_dir / "ref_python_vectors.npz")
    score, sig = z["proto/score"], z["proto/sigmoid"]
    for k in (1, 2, 3):
        mask, counts = oracle.route_scores(score, "topk", k, output="mask")
        assert np.array_equal(mask, z[f"proto/topk{k}"])
        assert np.array_equal(counts, z[f"proto/topk{k}"].sum(axis=0))
        idx, loads = oracle.route_scores(score, "topk", k, output="seat_indices")
        exp_i, exp_l = oracle.generate_indices_and_loads(z[f"proto/topk{k}"])
        assert np.array_equal(idx, exp_i) and np.array_equal(loads, exp_l)
    mask, _ = oracle.route_scores(sig, "threshold", threshold=0.5, output="mask")
    assert np.array_equal(mask, z["proto/threshold_0.5"])
    mask, _ = oracle.route_scores(sig, "threshold", threshold=0.8, residual_path=3, output="mask")
    assert np.array_equal(mask, z["proto/threshold_0.8_residual3"])
    gates = oracle.renormalised_topk_score(score, 2)
    assert np.array_equal(gates != 0, z["proto/topk2"] != 0)
    picked = np.sort(score, axis=1)[:, -2:]
    np.testing.assert_allclose(gates.sum(axis=1), picked.sum(1) / np.maximum(
        picked.sum(1), np.finfo(np.float32).eps), rtol=1e-6)
