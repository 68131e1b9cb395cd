"""Bit-for-bit comparison with the reference project's own CUDA extension.

``python oracle/build.py --ref`` compiles the reference's unmodified router sources into
``oracle/_ref/``; when that build is present these tests run both implementations on the
same seeded inputs on the GPU.  (The checker in ``oracle/`` is itself pinned by the same
comparison.)  bf16, which the reference lacks, is covered by viewing the bits as fp16 for
unweighted moves.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


@pytest.fixture(scope="module")
def ref():
    if not any(REF_DIR.glob("brt_ref_router*.so")):
        pytest.skip("reference extension not built (python oracle/build.py --ref)")
    sys.path.insert(0, str(REF_DIR))
    import brt_ref_router

    return brt_ref_router


@pytest.fixture(scope="module")
def R():
    from brainstorm_b200._C import router

    return router


def topk_mask(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    score = torch.randn((T, E), generator=g)
    idx = torch.topk(score, k, dim=1).indices
    return torch.zeros((T, E), dtype=torch.int32).scatter_(1, idx, 1).cuda()


@pytest.mark.parametrize("T,E,k", [(4096, 8, 1), (4096, 16, 4), (5000, 32, 2), (3000, 128, 1),
                                   (1037, 5, 2), (100, 64, 2)])
def test_indices_all_modes(ref, R, T, E, k):
    mask = topk_mask(T, E, k, T + E)
    caps = torch.tensor(sorted({1, 4, 16, 64, 256, max(1, T * k // E)}), dtype=torch.int32,
                        device="cuda")
    pw = torch.arange(1, E + 1, dtype=torch.int32, device="cuda") * 3
    for tag in (False, True):
        for c, cpad, pwise in ((None, False, False), (caps, False, False), (caps, True, False),
                               (pw, True, True)):
            a = ref.generate_indices_and_loads(mask, c, cpad, pwise, tag)
            b = R.generate_indices_and_loads(mask, c, cpad, pwise, tag)
            torch.cuda.synchronize()
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), (tag, cpad, pwise)


def test_checker_matches_reference_build(ref):
    mask = topk_mask(3000, 8, 2, 5)
    caps = torch.tensor([100, 500, 700], dtype=torch.int32, device="cuda")
    for tag in (False, True):
        a = ref.generate_indices_and_loads(mask, caps, True, False, tag)
        e = oracle.generate_indices_and_loads(mask.cpu().numpy(), [100, 500, 700], True, False,
                                              tag)
        assert np.array_equal(a[0].cpu().numpy(), e[0])
        assert np.array_equal(a[1].cpu().numpy(), e[1])
    idx, loads = ref.generate_indices_and_loads(mask, caps, True, False, False)
    x = torch.randn((3000, 24), device="cuda")
    g = torch.rand((3000, 8), device="cuda")
    (d,) = ref.dispatch_with_indices_and_loads(x, idx, loads, g)
    (e,) = oracle.dispatch_with_indices_and_loads(x.cpu().numpy(), idx.cpu().numpy(),
                                                  loads.cpu().numpy(), g.cpu().numpy())
    assert np.array_equal(d.cpu().numpy(), e)
    (c,) = ref.combine_with_indices_and_loads(d, idx, loads, g)
    (ec,) = oracle.combine_with_indices_and_loads(e, idx.cpu().numpy(), loads.cpu().numpy(),
                                                  g.cpu().numpy())
    assert np.array_equal(c.cpu().numpy(), ec)


def test_throttle(ref, R):
    mask = topk_mask(5000, 16, 2, 3)
    thr = torch.randint(0, 900, (16,), dtype=torch.int32).cuda()
    p0 = torch.randint(0, 50, (16,), dtype=torch.int32).cuda()
    pa, pb = p0.clone(), p0.clone()
    a = ref.throttle_hotmask(mask, pa, thr)
    b = R.throttle_hotmask(mask, pb, thr)
    assert torch.equal(a[0], b[0]) and torch.equal(pa, pb)


def test_convert(ref, R):
    mask = topk_mask(3000, 8, 2, 8)
    seat, loads = ref.generate_indices_and_loads(mask, None, False, False, False)
    for flag, src in ((False, seat), (True, ref.convert_index_format(seat, loads, False))):
        assert torch.equal(ref.convert_index_format(src, loads, flag),
                           R.convert_index_format(src, loads, flag))


@pytest.mark.parametrize("T,E,k,cell", [(4096, 8, 1, (768,)), (2048, 4, 2, (4, 3, 2, 3)),
                                        (1000, 32, 2, (1024,)), (333, 6, 3, (10,))])
def test_dispatch_combine_fp32(ref, R, T, E, k, cell):
    mask = topk_mask(T, E, k, T)
    cap = torch.tensor([max(1, T * k // E - 3)], dtype=torch.int32, device="cuda")
    x = torch.randn((T,) + cell, device="cuda")
    g = torch.rand((T, E), device="cuda")
    for caps, cpad in ((None, False), (cap, True)):
        idx, loads = ref.generate_indices_and_loads(mask, caps, cpad, False, False)
        for gates in (None, g):
            for tagging in (False, True):
                for pad in (False, True):
                    mpl = int(loads.max().item()) + 2 if pad else 0
                    a = ref.dispatch_with_indices_and_loads(x, idx, loads, gates, tagging, None,
                                                            pad, mpl)
                    b = R.dispatch_with_indices_and_loads(x, idx, loads, gates, tagging, None,
                                                          pad, mpl)
                    assert all(torch.equal(p, q) for p, q in zip(a, b))
                    (ca,) = ref.combine_with_indices_and_loads(a[0], idx, loads, gates, None, pad)
                    (cb,) = R.combine_with_indices_and_loads(b[0], idx, loads, gates, None, pad)
                    assert torch.equal(ca, cb)
                    ra, rb = x.clone(), x.clone()
                    ref.combine_with_indices_and_loads(a[0], idx, loads, gates, ra, pad)
                    R.combine_with_indices_and_loads(b[0], idx, loads, gates, rb, pad)
                    assert torch.equal(ra, rb)


def test_dispatch_bf16_as_fp16_bits(ref, R):
    """Unweighted dispatch is a bit copy: run the reference on the bf16 buffer viewed as fp16."""
    T, E = 2000, 8
    mask = topk_mask(T, E, 2, 12)
    idx, loads = ref.generate_indices_and_loads(mask, None, False, False, False)
    x = torch.randn((T, 256), device="cuda").to(torch.bfloat16)
    (a,) = ref.dispatch_with_indices_and_loads(x.view(torch.float16), idx, loads)
    (b,) = R.dispatch_with_indices_and_loads(x, idx, loads)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_dispatch_fp16_weighted(ref, R):
    T, E = 2000, 8
    mask = topk_mask(T, E, 2, 13)
    idx, loads = ref.generate_indices_and_loads(mask, None, False, False, False)
    x = torch.randn((T, 256), device="cuda").half()
    g = torch.rand((T, E), device="cuda").half()
    (a,) = ref.dispatch_with_indices_and_loads(x, idx, loads, g)
    (b,) = R.dispatch_with_indices_and_loads(x, idx, loads, g)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_dispatch_2d_scores(ref, R):
    T, E = 3000, 8
    mask = topk_mask(T, E, 2, 14)
    idx, loads = ref.generate_indices_and_loads(mask, None, False, False, False)
    score = torch.rand((T, E), device="cuda")
    (a,) = ref.dispatch_with_indices_and_loads(score, idx, loads, None, False, None, False, 0,
                                               False)
    (b,) = R.dispatch_with_indices_and_loads(score, idx, loads, None, False, None, False, 0,
                                             False)
    assert a.shape == b.shape and torch.equal(a, b)
