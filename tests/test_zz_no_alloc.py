"""The allocation-free entry point of the C ABI.

``brt_generate_indices_and_loads_static`` is for callers that cannot get device memory of
their own (a runtime whose memory planner owns the heap, a plugin host that passes only
inputs and outputs): its scratch is a fixed array in the library image.  This test drives it through the C ABI only - torch is used to hold the
inputs and outputs, never by the call under test - and checks it bit for bit against the
regular entry point on two calls in a row, the second on a different mask so that whatever
the first call left in the shared array must not matter.

Collected last on purpose (file name), so that a run that stops at the first failure has
already run every other test; it also passes on its own in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _mask(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    picks = torch.topk(torch.randn((T, E), generator=g), k, dim=1).indices
    return torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1).cuda()


def _regular(lib, mask, caps, cpad, tag):
    T, E = mask.shape
    idx = torch.full_like(mask, -7)
    loads = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    n = lib.query("brt_index_scratch_bytes", T, E)
    scratch = torch.empty(n, dtype=torch.uint8, device="cuda")
    lib.call("brt_generate_indices_and_loads", mask.data_ptr(), idx.data_ptr(), loads.data_ptr(),
             None, T, E, None if caps is None else caps.data_ptr(), 0 if caps is None else caps.numel(),
             int(cpad), 0, int(tag), scratch.data_ptr(), n,
             torch.cuda.current_stream().cuda_stream)
    return idx, loads


def _static(lib, mask, caps, cpad, tag):
    T, E = mask.shape
    idx = torch.full_like(mask, -7)
    loads = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    lib.call("brt_generate_indices_and_loads_static", mask.data_ptr(), idx.data_ptr(),
             loads.data_ptr(), T, E, None if caps is None else caps.data_ptr(),
             0 if caps is None else caps.numel(), int(cpad), 0, int(tag),
             torch.cuda.current_stream().cuda_stream)
    return idx, loads


def test_static_scratch_entry_point_matches_regular_one():
    from brainstorm_b200 import _lib

    assert _lib.query("brt_static_index_scratch_bytes") == 2 << 20
    caps = torch.tensor([64, 256, 1024, 4096], dtype=torch.int32, device="cuda")
    calls = [
        # first call: top-2 over 32 paths, padded loads, seat indices
        (_mask(32768, 32, 2, 1), caps, True, False),
        # second call, right after: another shape, path count and index format
        (_mask(5000, 8, 1, 2), None, False, True),
        # and one through the strip kernels (path count not a multiple of 4)
        (_mask(3001, 6, 2, 3), None, False, False),
    ]
    for mask, c, cpad, tag in calls:
        got_i, got_l = _static(_lib, mask, c, cpad, tag)
        want_i, want_l = _regular(_lib, mask, c, cpad, tag)
        torch.cuda.synchronize()
        assert torch.equal(got_l, want_l)
        assert torch.equal(got_i, want_i)
        # and against the CPU restatement of the reference's kernel
        ref_i, ref_l = oracle.generate_indices_and_loads(
            mask.cpu().numpy(), None if c is None else c.cpu().numpy().tolist(), cpad, False,
            tag)
        assert np.array_equal(got_i.cpu().numpy(), ref_i)
        assert np.array_equal(got_l.cpu().numpy(), ref_l)
    # back to back on one stream without a sync in between
    a = _static(_lib, calls[0][0], caps, True, False)
    b = _static(_lib, calls[1][0], None, False, True)
    torch.cuda.synchronize()
    assert torch.equal(a[0], _regular(_lib, calls[0][0], caps, True, False)[0])
    assert torch.equal(b[0], _regular(_lib, calls[1][0], None, False, True)[0])


def test_static_scratch_entry_point_refuses_large_masks():
    from brainstorm_b200 import _lib

    T, E = 262144, 128  # needs ~8 MiB of scratch
    mask = torch.zeros((8, E), dtype=torch.int32, device="cuda")  # never read: refused first
    idx = torch.zeros_like(mask)
    loads = torch.zeros((E,), dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.BrtError) as err:
        _lib.call("brt_generate_indices_and_loads_static", mask.data_ptr(), idx.data_ptr(),
                  loads.data_ptr(), T, E, None, 0, 0, 0, 0,
                  torch.cuda.current_stream().cuda_stream)
    assert "holds 2097152 bytes" in str(err.value)
