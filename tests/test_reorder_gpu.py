"""Locality-reorder kernel against the checker and, when built, the reference's own kernel
(src/distributed/local_reorder.cu)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


@pytest.fixture(scope="module")
def D():
    from brainstorm_b200._C import distributed

    return distributed


@pytest.mark.parametrize("W", [1, 2, 3, 4, 8, 16, 32])
@pytest.mark.parametrize("kind", ["random", "ties", "diag"])
def test_locality_reorder(D, W, kind):
    rng = np.random.default_rng(W * 7 + len(kind))
    if kind == "random":
        m = rng.integers(0, 5000, size=(W, W))
    elif kind == "ties":
        m = rng.integers(0, 3, size=(W, W))
    else:
        m = np.eye(W) * 9 + 1
    m = m.astype(np.int32)
    exp_loads, exp_idx = oracle.locality_reorder(m, W)
    got_loads, got_idx = D.locality_reorder(torch.from_numpy(m).cuda(), W)
    assert np.array_equal(got_idx.cpu().numpy(), exp_idx)
    assert np.array_equal(got_loads.cpu().numpy(), exp_loads)
    assert sorted(exp_idx.tolist()) == list(range(W))


@pytest.mark.parametrize("W,G", [(2, 2), (4, 4), (8, 8), (8, 3), (4, 37), (16, 2)])
def test_group_locality_reorder(D, W, G):
    rng = np.random.default_rng(W * 31 + G)
    m = rng.integers(0, 1024, size=(W, W, G)).astype(np.int32)
    exp_loads, exp_idx = oracle.group_locality_reorder(m, W, G)
    got_loads, got_idx = D.group_locality_reorder(torch.from_numpy(m).cuda().view(-1), W, G)
    assert np.array_equal(got_idx.cpu().numpy(), exp_idx)
    assert np.array_equal(got_loads.cpu().numpy().reshape(W, W, G), exp_loads)


def test_against_reference_kernel(D):
    if not any(REF_DIR.glob("brt_ref_distributed*.so")):
        pytest.skip("reference extension not built (python oracle/build.py --ref)")
    sys.path.insert(0, str(REF_DIR))
    import brt_ref_distributed as ref

    rng = np.random.default_rng(5)
    for W in (2, 4, 8):
        for trial in range(3):
            hi = 4 if trial == 2 else 2000  # the last trial is tie-heavy
            m = torch.from_numpy(rng.integers(0, hi, size=(W, W)).astype(np.int32)).cuda()
            a = ref.locality_reorder(m.view(-1), W)
            b = D.locality_reorder(m.view(-1), W)
            torch.cuda.synchronize()
            assert torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
        for G in (2, 4):
            # The reference sums the G loads of a pair in place and then compacts the sums
            # inside the same shared array without a barrier (local_reorder.cu:83-102);
            # that is only race-free while all W*W*G threads sit in one warp.
            if W * W * G > 32:
                continue
            m = torch.from_numpy(rng.integers(0, 1024, size=(W * W * G,)).astype(np.int32)).cuda()
            a = ref.group_locality_reorder(m, W, G)
            b = D.group_locality_reorder(m, W, G)
            torch.cuda.synchronize()
            assert torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
