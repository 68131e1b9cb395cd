"""Timing of the combine that pulls its rows (combine_land_kernel) with two ranks emulated on
ONE GPU, beside the plain combine on the same rows: shows the kernel itself, without NVLink.
cfg2-sized routing (32768 cells per rank, 1024 bf16 elements, 32 experts, top-2, slots of 2048
rows).  Not a test (pytest does not collect it): run it by hand, or under ncu as
profiles/ncu_full_emulated_ranks_combine_land.txt says.

    python tests/emulated_combine_land_timing.py
"""
import ctypes
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parent))

import test_exchange_emulated_gpu as emulated  # noqa: E402
from brainstorm_b200 import _lib  # noqa: E402
from brainstorm_b200._C import router as R  # noqa: E402

POST, PUSH, WAIT = 1, 4, 8
WORLD, GROUP, CELLS, COLS, TOP_K, SLOT = 2, 16, 32768, 1024, 2, 2048


def main():
    dev = torch.device("cuda", 0)
    E = WORLD * GROUP
    gen = torch.Generator().manual_seed(0)
    xs, idxs, loads, counts, gates = [], [], [], [], []
    for _ in range(WORLD):
        picks = torch.topk(torch.randn((CELLS, E), generator=gen), TOP_K, dim=1).indices
        mask = torch.zeros((CELLS, E), dtype=torch.int32).scatter_(1, picks, 1).to(dev)
        limit = torch.full((E,), SLOT, dtype=torch.int32, device=dev)
        indices, load, _ = R.throttle_and_generate_indices(
            mask, torch.zeros(E, dtype=torch.int32, device=dev), limit, limit)
        xs.append(torch.randn((CELLS, COLS), generator=gen).to(dev).bfloat16())
        idxs.append(indices)
        loads.append(load.contiguous())
        counts.append(getattr(indices, R._DENSE))
        gates.append(torch.rand((CELLS, E), generator=gen).to(dev))
    ranks = emulated.Ranks(WORLD, half=256 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    grain = COLS * 2
    try:
        for rep in range(4):
            outs = ranks.dispatch_forward(xs, idxs, loads, counts, GROUP, SLOT)
            ids = [int(_lib.query("brt_p2p_ctx_exchanges", c)) for c in ranks.ctxs]
            offsets = [outs[r][0] - ranks.arenas[r] for r in range(WORLD)]
            results = [torch.empty((CELLS, COLS), dtype=torch.bfloat16, device=dev)
                       for _ in range(WORLD)]
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(WORLD + 1)]
            for stage in (POST, PUSH, WAIT):
                for r in range(WORLD):
                    if stage == PUSH:
                        marks[r].record()
                    _lib.call("brt_p2p_combine_backward", ranks.ctxs[r], ids[r], GROUP, grain,
                              SLOT, offsets[r], idxs[r].data_ptr(), gates[r].data_ptr(), 0, 2,
                              CELLS, results[r].data_ptr(), stream, stage)
                if stage == PUSH:
                    marks[WORLD].record()
            torch.cuda.synchronize()
            trace = (ctypes.c_uint64 * 10)()
            _lib.call("brt_p2p_ctx_trace", ranks.ctxs[WORLD - 1], trace)
            # the plain combine of the same routing, on a local buffer
            (routed,) = R.dispatch_with_indices_and_loads(xs[0], idxs[0], loads[0], None, False,
                                                          None, True, SLOT)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            R.combine_with_indices_and_loads(routed, idxs[0], loads[0], gates[0], None, True)
            b.record()
            torch.cuda.synchronize()
            pulls = ", ".join(f"{marks[r].elapsed_time(marks[r + 1]) * 1e3:.1f}"
                              for r in range(WORLD))
            print(f"rep {rep}: combine_land per emulated rank {pulls} us; "
                  f"plain combine {a.elapsed_time(b) * 1e3:.1f} us")
            print("   last rank's kernel by its own clock: wait %.1f, flags after %.1f, plan "
                  "%.1f, first CTA out %.1f, last CTA out %.1f us"
                  % tuple(v / 1e3 for v in trace[5:10]))
    finally:
        ranks.close()


if __name__ == "__main__":
    main()
