"""The reference project's own CUDA kernels, timed beside this library on the same GPU.

Uses the reference extension that ``python oracle/build.py --ref`` compiles from the
reference's unmodified sources into ``oracle/_ref/`` (skipped when absent).  Every op is run
on the same seeded inputs by both implementations at the benchmark shapes, the outputs are
compared bit for bit (the reference has fp32 and fp16 only, so the bf16 workloads run with
fp32 values here) and the median CUDA-event time of each is printed; run with ``-s`` to see
the table, set ``BRT_TIMING_OUT`` to a file name to also get it as JSON.  L2 is flushed
between repetitions.
"""
import json
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"

SHAPES = {
    # name: T, d, E, k, capacity (0 = packed output)
    "cfg1 fp32 T=4096 d=768 E=8 top-1 cap=640": (4096, 768, 8, 1, 640),
    "cfg2 shape, fp32 values T=32768 d=1024 E=32 top-2 cap=2048": (32768, 1024, 32, 2, 2048),
    "cfg3 shape, fp32 values T=262144 d=768 E=128 top-1 cap=4096": (262144, 768, 128, 1, 4096),
    "cfg4 shape, fp32 values T=65536 d=2048 E=64 top-2 packed": (65536, 2048, 64, 2, 0),
}


@pytest.fixture(scope="module")
def ref():
    if not any(REF_DIR.glob("brt_ref_router*.so")):
        pytest.skip("reference extension not built (python oracle/build.py --ref)")
    sys.path.insert(0, str(REF_DIR))
    import brt_ref_router

    return brt_ref_router


def median_us(fn, flush, reps=7):
    for _ in range(2):
        out = fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    return sorted(times)[len(times) // 2], out


@pytest.mark.parametrize("name", list(SHAPES))
def test_reference_kernels_beside_ours(ref, name):
    from brainstorm_b200._C import router as ours

    T, d, E, k, cap = SHAPES[name]
    g = torch.Generator().manual_seed(T + E)
    bias = torch.randn(E, generator=g) * 0.5
    score = torch.softmax(torch.randn((T, E), generator=g) + bias, dim=1)
    picks = torch.topk(score, k, dim=1).indices
    mask = torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1).cuda()
    gates = score.cuda()
    x = torch.randn((T, d), generator=g).cuda()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    padded = cap > 0
    caps = torch.full((E,), cap, dtype=torch.int32, device="cuda") if padded else None
    rows = {}

    def both(op, f_ref, f_ours, same):
        t_ref, o_ref = median_us(f_ref, flush)
        t_ours, o_ours = median_us(f_ours, flush)
        assert same(o_ref, o_ours), f"{op}: outputs differ"
        rows[op] = {"reference_us": round(t_ref, 1), "ours_us": round(t_ours, 1),
                    "speedup": round(t_ref / t_ours, 2)}
        return o_ours

    eq_all = lambda a, b: all(torch.equal(p, q) for p, q in zip(a, b))
    m = mask
    if padded:
        zeros = torch.zeros(E, dtype=torch.int32, device="cuda")
        m = both("throttle_hotmask",
                 lambda: ref.throttle_hotmask(mask, zeros.clone(), caps),
                 lambda: ours.throttle_hotmask(mask, zeros.clone(), caps), eq_all)[0]
    idx, loads = both("generate_indices_and_loads",
                      lambda: ref.generate_indices_and_loads(m, caps),
                      lambda: ours.generate_indices_and_loads(m, caps), eq_all)
    (routed,) = both("dispatch_with_indices_and_loads",
                     lambda: ref.dispatch_with_indices_and_loads(x, idx, loads, None, False, None,
                                                                 padded, cap),
                     lambda: ours.dispatch_with_indices_and_loads(x, idx, loads, None, False,
                                                                  None, padded, cap), eq_all)
    both("combine_with_indices_and_loads",
         lambda: ref.combine_with_indices_and_loads(routed, idx, loads, gates, None, padded),
         lambda: ours.combine_with_indices_and_loads(routed, idx, loads, gates, None, padded),
         eq_all)
    total_ref = sum(r["reference_us"] for r in rows.values())
    total_ours = sum(r["ours_us"] for r in rows.values())
    rows["step"] = {"reference_us": round(total_ref, 1), "ours_us": round(total_ours, 1),
                    "speedup": round(total_ref / total_ours, 2)}
    print(f"\n{name}")
    for op, r in rows.items():
        print(f"  {op:34s} reference {r['reference_us']:10.1f} us   ours {r['ours_us']:9.1f} us"
              f"   x{r['speedup']:.2f}")
    out = os.environ.get("BRT_TIMING_OUT")
    if out:
        known = json.load(open(out)) if os.path.exists(out) else {}
        known[name] = rows
        json.dump(known, open(out, "w"), indent=1)
