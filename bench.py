"""Benchmark of the routing hot path (mask -> throttle -> seat indices/loads -> dispatch ->
combine, plus the expert-parallel exchange when run on more than one GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

Prints ONE JSON line (rank 0).  Inputs are seeded synthetic tensors with the shapes and value
distributions of the named workload; nothing is read from disk.  With ``--impl reference``
the CPU restatement of the reference's router (``oracle/``) is timed on the host cores
instead, on the same workload.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "routed tokens/sec (dispatch+combine)"
UNIT = "tokens/s"

WORKLOADS = {
    # name: T, d, E, top_k, dtype, bias_std, capacity rule
    "cfg1": dict(T=4096, d=768, E=8, k=1, dtype="f32", seed=0, bias="none", cap="ceil1.25",
                 desc="Switch top-1, T=4096 d=768 E=8 fp32, capacity ceil(1.25*T/E), drop"),
    "cfg2": dict(T=32768, d=1024, E=32, k=2, dtype="bf16", seed=2, bias="normal0.5",
                 cap="swin1.0",
                 desc="top-2 MoE route bf16, T=32768 d=1024 E=32, biased logits, renormalised "
                      "gates, capacity factor 1.0 with drop"),
    "cfg3": dict(T=262144, d=768, E=128, k=1, dtype="bf16", seed=3, bias="zipf", cap="ceil2.0",
                 desc="Switch-Base-128-like top-1 bf16, T=262144 d=768 E=128, Zipf-biased "
                      "logits, capacity factor 2.0 with drop"),
    "cfg3nd": dict(T=262144, d=768, E=128, k=1, dtype="bf16", seed=3, bias="zipf", cap="none",
                   desc="Switch-Base-128-like top-1 bf16, T=262144 d=768 E=128, Zipf-biased "
                        "logits, no-drop variant (packed output sized by the generated loads)"),
    "cfg5": dict(T=64, d=256 * 56 * 56, E=8, k=0, dtype="f32", seed=5, bias="none", cap="none",
                 protocol="threshold", threshold=0.5,
                 desc="dynamic-routing threshold router fp32: 64 samples of [256,56,56], 8 "
                      "branches, sigmoid gates, threshold 0.5, empty routes allowed, samples "
                      "gathered back by sum (seat-index kernels)"),
    "cfg4": dict(T=65536, d=2048, E=64, k=2, dtype="bf16", seed=4, bias="normal1.0", cap="none",
                 desc="expert-parallel top-2 bf16 per GPU T=65536 d=2048 E=64, no capacity"),
}

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


# --------------------------------------------------------------------------------- workloads
def capacity_of(w) -> int:
    T, E, k = w["T"], w["E"], w["k"]
    rule = w["cap"]
    if rule == "ceil1.25":
        return math.ceil(1.25 * T / E)
    if rule == "ceil2.0":
        return math.ceil(2.0 * T / E)
    if rule == "swin1.0":
        return k * int(1.0 * math.ceil(T / E))
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum per launch of each timed kernel, from the ncu
# captures summarised under profiles/ (ncu_full_cfg2_routing_step_kernels.txt,
# ncu_counters_cfg3_dispatch_combine.txt, ncu_counters_cfg4_dispatch_combine.txt).  Each
# kernel alone and cold; dirty lines that the 126 MB L2 still holds when a kernel ends are not
# in these counters, so the write-heavy ops can read below their algorithmic bytes.
NCU_DRAM_KERNEL_TRAFFIC = {
    "cfg2": {"throttle_index_chain_kernel": 4.24e6, "dispatch_kernel": 132.97e6,
             "combine_kernel": 117.16e6},
    "cfg3": {"dispatch_kernel": 935.44e6, "combine_kernel": 673.39e6},
    "cfg4": {"dispatch_kernel": 763.28e6, "combine_kernel": 800.58e6},
}


def make_workload(name: str, rank: int = 0, local_bias: float = 0.0, world: int = 1):
    """Host (CPU) tensors of one workload: activations, fp32 logits, softmax scores, top-k hot
    mask, combine gates.  Generated on CPU in fp32 so that the CPU checker and the GPU see the
    same bits."""
    w = WORKLOADS[name]
    T, d, E, k = w["T"], w["d"], w["E"], w["k"]
    g = torch.Generator(device="cpu").manual_seed(w["seed"] * 1000 + rank)
    gb = torch.Generator(device="cpu").manual_seed(w["seed"] * 1000 + 999)  # shared by all ranks
    x = torch.randn((T, d), generator=g, dtype=torch.float32).to(TORCH_DT[w["dtype"]])
    logits = torch.randn((T, E), generator=g, dtype=torch.float32)
    if w["bias"].startswith("normal"):
        logits = logits + float(w["bias"][6:]) * torch.randn((E,), generator=gb)
    elif w["bias"] == "zipf":
        ranks = torch.randperm(E, generator=gb).to(torch.float32) + 1.0
        z = ranks.pow(-1.1)
        logits = logits + 4.0 * z / z.max()
    if local_bias and world > 1:
        G = E // world
        logits[:, rank * G:(rank + 1) * G] += local_bias
    if w.get("protocol") == "threshold":
        # python/brt/router/protocol/threshold.py:23-39; every kept route weighs 1
        score = torch.sigmoid(logits)
        mask = (score > w["threshold"]).to(torch.int32)
        return dict(name=name, spec=w, x=x, logits=logits, score=score, mask=mask,
                    gates=mask.to(torch.float32), cap=capacity_of(w))
    score = torch.softmax(logits, dim=1)
    vals, picks = torch.topk(score, k, dim=1)
    mask = torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1)
    if k > 1:
        denom = torch.clamp(vals.sum(dim=1, keepdim=True), min=torch.finfo(torch.float32).eps)
        gates = torch.zeros_like(score).scatter_(1, picks, vals / denom)
    else:
        gates = score
    return dict(name=name, spec=w, x=x, logits=logits, score=score, mask=mask, gates=gates,
                cap=capacity_of(w))


def algorithmic_bytes(w, idx: np.ndarray, loads: np.ndarray, total_rows: int):
    """Minimum HBM bytes of each op for this routing: R kept routes, T_r cells
    with at least one kept route, L output rows."""
    T, d, E = w["T"], w["d"], w["E"]
    s = 4 if w["dtype"] == "f32" else 2
    kept = (idx > 0) & (idx <= loads[None, :])
    R = int(kept.sum())
    Tr = int(kept.any(axis=1).sum())
    return {
        "throttle": 8 * T * E + 12 * E,
        "indices": 8 * T * E + (16 * E if w["cap"] != "none" else 4 * E),
        "dispatch": Tr * d * s + total_rows * d * s + 4 * T * E,
        "combine": R * d * s + T * d * s + 8 * T * E,
        # the two kernels of a dispatch: rows moved to their routes, rows nobody landed on
        "dispatch_move": Tr * d * s + R * d * s + 4 * T * E,
        "dispatch_zero_fill": (total_rows - R) * d * s + total_rows,
        "R": R, "T_r": Tr, "L": total_rows,
    }


def config_of(name: str, world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    w = WORKLOADS[name]
    s = 4 if w["dtype"] == "f32" else 2
    distributed = world > 1
    return {"workload": f"{name}: {w['desc']}",
            "step": "throttle + seat indices/loads (one fused scan when a capacity applies) + "
                    "dispatch + "
                    + ("sparse all-to-all forward and back + " if distributed else "")
                    + "weighted combine",
            "l2": "inputs and outputs of a step exceed the 126 MB L2"
                  if (w["T"] * w["d"] * s * 3) > 126e6 else
                  "working set fits in L2; numbers are L2-assisted",
            "parallelism": f"ep{world}" if distributed else "single"}


# --------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6),
                                  ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if f[col].lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm),
                       reasons=sorted(reasons))
        return out


# --------------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=dev)
    from brainstorm_b200._C import router as R
    from brainstorm_b200.router import GatherRouter, ScatterRouter
    from brainstorm_b200.runtime import distributed as brt_dist

    wl = make_workload(args.workload, rank=rank, local_bias=args.local_bias, world=world)
    w = wl["spec"]
    T, d, E = w["T"], w["d"], w["E"]
    cap = wl["cap"]
    padded = cap > 0
    x = wl["x"].to(dev)
    mask = wl["mask"].to(dev)
    gates = wl["gates"].to(dev)
    caps = torch.full((E,), cap, dtype=torch.int32, device=dev) if padded else None
    zeros_e = torch.zeros((E,), dtype=torch.int32, device=dev)
    distributed = world > 1
    if distributed:
        assert E % world == 0
        brt_dist.is_nccl_activated()

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(8)] for _ in range(args.steps)]
    a2a_bytes = [0]
    fused_used = [False]
    pulled = [False]

    def step(i=None):
        rec = (lambda j: ev[i][j].record()) if i is not None else (lambda j: None)
        rec(0)
        rec(1)
        if padded:
            # throttle_hotmask + generate_indices_and_loads of the throttled mask, one pass
            prefix = torch.zeros_like(zeros_e)
            idx, loads, _ = R.throttle_and_generate_indices(mask, prefix, caps, caps)
        else:
            idx, loads = R.generate_indices_and_loads(mask, caps)
        rec(2)
        fused = None
        if distributed and not args.no_fused_exchange:
            # dispatch and forward exchange as one kernel (what the distributed fabric runs):
            # there is no separate dispatch to time, the forward leg includes it
            rec(3)
            fused = brt_dist.dispatch_group_sparse_a2a(x, idx, loads, padded, cap)
            if fused is None:
                (routed,) = R.dispatch_with_indices_and_loads(x, idx, loads, None, False, None,
                                                              padded, cap)
        else:
            (routed,) = R.dispatch_with_indices_and_loads(x, idx, loads, None, False, None,
                                                          padded, cap)
            rec(3)
        if distributed:
            if fused is not None:
                recv, out_loads, in_loads = fused
            else:
                recv, out_loads, in_loads = brt_dist.group_sparse_a2a(routed, loads, padded, cap)
            rec(4)
            # rows this rank really sends to OTHER ranks (in_loads: my send sizes, [W, G])
            sent = in_loads.reshape(world, -1)
            a2a_bytes[0] = int(sent.sum() - sent[rank].sum()) * d * x.element_size()
            fused_used[0] = fused is not None
            out = None
            if args.pull_combine:
                # inverse exchange and combine as one kernel that pulls the rows from the
                # peers (an option of the distributed combine fabric): no separate inverse leg
                rec(5)
                out = brt_dist.combine_group_sparse_a2a(recv, idx, gates, out_loads, in_loads,
                                                        padded)
                routed = recv
            pulled[0] = out is not None
            if out is None:
                routed = brt_dist.size_known_group_sparse_a2a(recv, out_loads, in_loads, padded)
                rec(5)
                (out,) = R.combine_with_indices_and_loads(routed, idx, loads, gates, None,
                                                          padded)
        else:
            rec(4)
            rec(5)
            (out,) = R.combine_with_indices_and_loads(routed, idx, loads, gates, None, padded)
        rec(6)
        return out, idx, loads, routed

    def step_replayable():
        """The expert-parallel step without a host synchronisation: the exchange's size
        tensors stay on the device (an expert would read its loads there), so the whole step
        can be captured in a CUDA graph, as the single-GPU step is."""
        if padded:
            prefix = torch.zeros_like(zeros_e)
            idx, loads, _ = R.throttle_and_generate_indices(mask, prefix, caps, caps)
        else:
            idx, loads = R.generate_indices_and_loads(mask, caps)
        with brt_dist.replayable_exchanges():
            recv, out_loads, in_loads = brt_dist.dispatch_group_sparse_a2a_device(
                x, idx, loads, padded, cap)
            out = brt_dist.combine_group_sparse_a2a(recv, idx, gates, out_loads, in_loads,
                                                    padded) if args.pull_combine else None
            routed = recv
            if out is None:
                routed = brt_dist.size_known_group_sparse_a2a(recv, out_loads, in_loads, padded)
        if out is None:
            (out,) = R.combine_with_indices_and_loads(routed, idx, loads, gates, None, padded)
        return out, idx, loads, routed

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        out, idx, loads, routed = step()
    barrier()

    # The padded single-GPU step has no host synchronisation, so it is captured once into a
    # CUDA graph and the timed region replays it: launch latency of the Python wrappers is
    # not part of the device-side number (the eager number is reported next to it).  The
    # un-padded step reads loads.sum() on the host to size its output and stays eager.
    graph = None
    if not distributed and not args.no_graph and padded:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out, idx, loads, routed = step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(warmup):
            graph.replay()
        barrier()
    graph_note = None
    if distributed and not args.no_graph and not args.no_fused_exchange:
        # every rank captures, or none does: a rank that replays cannot meet one that issues
        from brainstorm_b200.runtime import p2p as brt_p2p
        eager_out = out.clone()
        captured, why = None, ""
        try:
            if brt_p2p.arena() is None:
                raise RuntimeError("no peer-memory arena")
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_replayable()
                side.synchronize()
                captured = torch.cuda.CUDAGraph()
                with torch.cuda.graph(captured, stream=side):
                    g_out, g_idx, g_loads, g_routed = step_replayable()
            torch.cuda.current_stream().wait_stream(side)
        except Exception as exc:  # noqa: BLE001
            captured, why = None, f"{type(exc).__name__}: {exc}"[:200]
        agreed = torch.tensor([1 if captured is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 1:
            graph = captured
            for _ in range(warmup):
                graph.replay()
            barrier()
            same = torch.tensor([int(torch.equal(g_out, eager_out))], device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            graph_note = {"replayed_step_equals_eager_step": bool(same.item())}
            out, idx, loads = g_out, g_idx, g_loads
        else:
            graph_note = {"not_captured": why or "another rank could not capture"}
            del captured
        barrier()

    exchange_trace = None
    if distributed:
        from brainstorm_b200.runtime import p2p as brt_p2p
        if brt_p2p.arena() is not None:
            # where the two landing kernels of a step spend their time: waiting for the other
            # ranks to enter the exchange (skew) or moving rows (device clock, one step at a
            # time with a synchronisation after each; outside the timed region)
            rows_t = []
            for _ in range(10):
                if graph is not None:
                    graph.replay()
                else:
                    step()
                rows_t.append(brt_p2p.arena().trace())
            mean_t = torch.tensor([statistics.mean(r[k] for r in rows_t) for k in range(10)],
                                  device=dev, dtype=torch.float64)
            worst = mean_t.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            keys = ("wait", "move", "plan", "first_cta_out", "last_cta_out")
            exchange_trace = {"unit": "us", "steps": len(rows_t)}
            for leg, base in (("forward", 0), ("inverse", 5)):
                exchange_trace["rank0_" + leg] = {k: round(float(mean_t[base + i]), 2)
                                                  for i, k in enumerate(keys)}
                exchange_trace["slowest_rank_" + leg + "_move"] = round(float(worst[base + 1]), 2)
            exchange_trace["note"] = (
                "wait = CTA 0 of the landing kernel from its start until every rank has "
                "entered the exchange; the rest counts from that instant: move = until the "
                "arrival flags are raised, plan = CTA 0 has placed its buckets, first / "
                "last_cta_out = when the first / last CTA leaves its copy loop")
        barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for i in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            out, idx, loads, routed = step()
    t_end.record()
    barrier()
    total_ms = t_start.elapsed_time(t_end)
    if distributed:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps

    # Host-inclusive time of the eager Python API, for reference.
    # The library counts its own kernel launches; the eager steps give launches per step
    # (a graph replay issues the same kernels without passing through the entry points).
    from brainstorm_b200 import _lib
    h0 = torch.cuda.Event(enable_timing=True)
    h1 = torch.cuda.Event(enable_timing=True)
    launches_before = _lib.query("brt_kernel_launch_count")
    h0.record()
    for _ in range(args.steps):
        step()
    h1.record()
    barrier()
    launches_per_step = (_lib.query("brt_kernel_launch_count") - launches_before) / args.steps
    eager_host_ms = h0.elapsed_time(h1) / args.steps

    # Per-op device times: the same steps, eagerly, with events between the ops.  A spin
    # kernel holds the GPU while the host enqueues every step, so the event intervals hold
    # device time only, not host launch time.
    if not distributed:
        try:
            torch.cuda._sleep(int(60e6))
        except Exception:
            pass
    e_start = torch.cuda.Event(enable_timing=True)
    e_end = torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(args.steps):
        out, idx, loads, routed = step(i)
    e_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    eager_ms = e_start.elapsed_time(e_end) / args.steps

    # Per-kernel device times: the library brackets each of its hot kernels with CUDA events
    # on the launching stream while profiling is on (one more eager pass, same spin trick).
    from brainstorm_b200 import _lib as brt_lib
    import ctypes
    brt_lib.query("brt_profile_enable", 1)
    if not distributed:
        try:
            torch.cuda._sleep(int(60e6))
        except Exception:
            pass
    for i in range(args.steps):
        step()
    barrier()
    brt_lib.query("brt_profile_enable", 0)
    report = ctypes.create_string_buffer(8192)
    brt_lib.call("brt_profile_report", report, len(report))
    timed = json.loads(report.value.decode())

    names = ["throttle", "indices", "dispatch", "a2a_forward", "a2a_backward", "combine"]
    op_ms = {n: statistics.mean(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(args.steps))
             for j, n in enumerate(names)}
    ab = algorithmic_bytes(w, idx.cpu().numpy(), loads.cpu().numpy(), routed.size(0))
    peaks = {}
    try:
        peaks = json.load(open(ROOT / "MEASURED_PEAKS.json"))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    kernels = {}
    for n in ("indices", "dispatch", "combine"):
        if op_ms[n] > 0 and not (n == "dispatch" and fused_used[0]):
            gbs = ab[n] / (op_ms[n] * 1e-3) / 1e9
            kernels[n] = {"ms": round(op_ms[n], 5), "algorithmic_bytes": ab[n],
                          "achieved_gbs": round(gbs, 1), "frac": round(gbs / peak, 4)}
    dc_ms = op_ms["dispatch"] + op_ms["combine"]
    # which algorithmic byte count belongs to which timed kernel
    kernel_bytes = {"throttle_chain_kernel": ab["throttle"], "throttle_split_kernels": ab["throttle"],
                    "index_chain_kernel": ab["indices"], "index_split_kernels": ab["indices"],
                    "throttle_index_chain_kernel": ab["indices"],
                    "dispatch_kernel": ab["dispatch"],
                    "dispatch_move_kernel": ab["dispatch_move"],
                    "dispatch_zero_fill_kernel": ab["dispatch_zero_fill"],
                    "combine_kernel": ab["combine"]}
    device_kernels = {}
    for name, t in timed.items():
        if t["launches"] == 0:
            continue
        if name.startswith("p2p_") or name in ("dispatch_land_kernel", "combine_land_kernel"):
            # exchange kernels: bound by NVLink, not by HBM
            device_kernels[name] = {"launches": t["launches"],
                                    "ms": round(t["total_ms"] / t["launches"], 5)}
            continue
        if name not in kernel_bytes:
            continue
        ms = t["total_ms"] / t["launches"]
        gbs = kernel_bytes[name] / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        device_kernels[name] = {"launches": t["launches"], "ms": round(ms, 5),
                                "algorithmic_bytes": kernel_bytes[name],
                                "achieved_gbs": round(gbs, 1), "frac": round(gbs / peak, 4)}
    dominant = max((n for n in device_kernels if "algorithmic_bytes" in device_kernels[n]),
                   key=lambda n: device_kernels[n]["ms"])
    dominant_op = {"dispatch_move_kernel": "dispatch", "dispatch_zero_fill_kernel": "dispatch",
                   "dispatch_kernel": "dispatch",
                   "combine_kernel": "combine"}.get(dominant, "indices")

    # ---- the two big kernels launched back to back: the events that bracket every launch
    # above keep the next launch from overlapping the previous kernel's tail and add their
    # own few microseconds, which is a tenth of a 40 us kernel.  Here ONE pair of events spans
    # `reps` consecutive launches of the same kernel (a CUDA graph holds them, so the host is
    # not in the way); each launch moves more bytes than L2 holds.
    back_to_back = None
    if not distributed and padded and not args.no_graph:
        def consecutive(fn, reps=8):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(reps):
                        fn()
            torch.cuda.current_stream().wait_stream(side)
            ts = []
            for _ in range(8):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) / reps)
            return statistics.median(ts[3:])

        try:
            d_ms = consecutive(lambda: R.dispatch_with_indices_and_loads(
                x, idx, loads, None, False, None, padded, cap))
            c_ms = consecutive(lambda: R.combine_with_indices_and_loads(
                routed, idx, loads, gates, None, padded))
            back_to_back = {}
            for n, ms_ in (("dispatch", d_ms), ("combine", c_ms)):
                gbs = ab[n] / (ms_ * 1e-3) / 1e9
                back_to_back[n] = {"ms": round(ms_, 5), "achieved_gbs": round(gbs, 1),
                                   "frac": round(gbs / peak, 4)}
            back_to_back["timing"] = ("one pair of CUDA events around 8 consecutive launches "
                                      "of the kernel (a CUDA graph), median of 5, per launch")
        except Exception as exc:  # noqa: BLE001
            back_to_back = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}

    # ---- the gate in front of the path: scores -> mask (-> indices), torch ops of the
    # reference's protocol beside the library's single-launch gate
    gate = measure_gate(wl, dev, w, R, padded, caps)

    # ---- end to end through the router API with host buffers
    e2e = measure_e2e(wl, dev, args, ScatterRouter, GatherRouter, distributed, world)

    result = {
        "metric": METRIC, "value": world * T / (ms_per_step * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": config_of(args.workload, world),
        "dispatch_combine_only": {"tokens_per_s": world * T / (dc_ms * 1e-3), "ms": dc_ms},
        "roofline": {"bound": "hbm", "kernel": dominant,
                     "achieved": device_kernels[dominant]["achieved_gbs"], "peak": peak,
                     "unit": "GB/s", "frac": device_kernels[dominant]["frac"],
                     "traffic": NCU_DRAM_KERNEL_TRAFFIC.get(args.workload, {}).get(dominant),
                     "traffic_note": "ncu DRAM counters of one launch; writes still held in "
                                     "L2 at kernel end are not counted",
                     "peak_kind": f"{peak_kind} copy bandwidth",
                     "timing": "CUDA events around each launch of the kernel, on its stream",
                     "nominal_frac_of_8000":
                         round(device_kernels[dominant]["achieved_gbs"] / 8000, 4),
                     "whole_op": {"op": dominant_op, **kernels[dominant_op]}},
        "device_kernels": device_kernels,
        "kernels_back_to_back": back_to_back,
        "gate": gate,
        "kernels": kernels,
        "routing": {"kept_routes": ab["R"], "cells_routed": ab["T_r"], "output_rows": ab["L"]},
        "gpu_launches": int(round(args.steps * launches_per_step)),
        "gpu_launches_per_step": launches_per_step,
        "clocks": clocks, "e2e": e2e,
        "timed_region": ("CUDA graph replay of the step" + (
                             " (exchanges with device-resident sizes, no host synchronisation)"
                             if distributed else "")) if graph is not None
                        else "eager launches of the step",
        "eager_ms_per_step": eager_host_ms, "eager_device_ms_per_step": eager_ms,
        # `value` is a graph replay wherever the step can be captured (at N > 1: with the
        # exchange's size tensors left on the device); this is the figure of the eager
        # Python API at every N (at N > 1 the forward exchange hands CPU size tensors to the
        # host, as the reference's op does)
        "value_eager": world * T / (eager_host_ms * 1e-3),
    }
    if distributed:
        result["checks"] = exchange_checks(dev, rank, world, x, mask, gates, caps, cap, padded,
                                           R, brt_dist)
        if exchange_trace is not None:
            result["exchange_trace_us"] = exchange_trace
        if graph_note is not None:
            if "replayed_step_equals_eager_step" in graph_note:
                result["checks"].update(graph_note)
            else:
                result["graph"] = graph_note
        plain = measure_a2a_cfg4(dev, rank, world, R, brt_dist, 0.0, uniform_loads=True)
        plain.pop("loads_rank")
        result["a2a_cfg4"] = plain
        hot = measure_a2a_cfg4(dev, rank, world, R, brt_dist, 0.0)
        hot.pop("loads_rank")
        result["a2a_cfg4_hot_experts"] = hot
        bias = bias_for_local_fraction(world, 0.6)
        skewed = measure_a2a_cfg4(dev, rank, world, R, brt_dist, bias)
        skew_loads = skewed.pop("loads_rank")
        skewed["locality"] = measure_locality(skew_loads, world, dev, brt_dist)
        # the same bias towards the NEXT rank's experts (every rank's favourite experts live
        # elsewhere, the case of benchmark/micro/distributed/placement_a2a.py:54-64): here the
        # rank matching has something to find
        shifted = measure_a2a_cfg4(dev, rank, world, R, brt_dist, bias, favour_shift=1,
                                   loads_only=True)
        skewed["locality_when_the_favoured_experts_sit_on_the_next_rank"] = measure_locality(
            shifted["loads_rank"], world, dev, brt_dist)
        result["locality_cfg4"] = skewed
        result["checks"]["a2a_cfg4_round_trip_bit_exact"] = bool(
            plain["round_trip_bit_exact"] and hot["round_trip_bit_exact"]
            and skewed["round_trip_bit_exact"])
        result["locality"] = measure_locality(loads, world, dev, brt_dist)
        try:
            result["balanced_placement"] = measure_balanced_placement(
                dev, rank, world, x, mask, gates, caps, cap, padded, R, brt_dist, args.steps)
        except Exception as exc:  # noqa: BLE001  (an extra, never the reason a run fails)
            result["balanced_placement"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:160]}
        fwd = a2a_bytes[0]
        land_name = "dispatch_land_kernel" if fused_used[0] else "p2p_land_forward_kernel"
        land = device_kernels.get(land_name)
        if land is not None and land["ms"] > 0:
            # at N > 1 the step is bound by the exchange: its landing kernel against NVLink
            gbs = fwd / (land["ms"] * 1e-3) / 1e9
            result["roofline_hbm_kernel"] = result["roofline"]
            result["roofline"] = {
                "bound": "nvlink", "kernel": land_name, "achieved": round(gbs, 1),
                "peak": 900.0, "unit": "GB/s", "frac": round(gbs / 900.0, 4), "traffic": None,
                "peak_kind": "nominal NVLink 5 bandwidth per direction per GPU; a peer copy "
                             "on this pool measures 770 GB/s",
                "frac_of_measured_peer_copy": round(gbs / 770.0, 4),
                "timing": "CUDA events around each launch of the kernel, on its stream; "
                          "bytes = what this rank sends to other ranks in one exchange"}
            if exchange_trace is not None:
                # the same launch by the device's own clock, from "every rank has entered the
                # exchange" to "arrival flags raised" (no launch or event overhead, no skew)
                move = exchange_trace["rank0_forward"]["move"]
                if move > 0:
                    result["roofline"]["by_device_clock"] = {
                        "move_us": move, "achieved": round(fwd / (move * 1e-6) / 1e9, 1),
                        "frac": round(fwd / (move * 1e-6) / 1e9 / 900.0, 4)}
        # with the combine that pulls its rows from the peers the inverse leg IS the combine
        back_ms = op_ms["combine"] if pulled[0] else op_ms["a2a_backward"]
        result["a2a"] = {
            "forward_ms": op_ms["a2a_forward"], "backward_ms": back_ms,
            "remote_bytes_per_rank_per_direction": a2a_bytes[0],
            "bus_gbs_forward": fwd / (op_ms["a2a_forward"] * 1e-3) / 1e9,
            "bus_gbs_backward": fwd / (back_ms * 1e-3) / 1e9,
            "backward_includes_combine": pulled[0],
            "nvlink_peak_gbs_per_direction": 900.0,
            "transport": "peer-memory landing kernels over NVLink"
                         if __import__("brainstorm_b200.runtime.p2p", fromlist=["arena"]).arena()
                         is not None else "nccl send/recv",
            "forward_includes_dispatch": fused_used[0],
        }
    if world == 1:
        result["expert_gemm"] = measure_expert_gemm(wl, dev, loads, cap, peaks)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(wl, budget_s=args.cpu_seconds)
    if rank == 0:
        print(json.dumps(result))
    failed = distributed and not all(v for v in result["checks"].values() if isinstance(v, bool))
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("bench.py: an exchange check failed (see \"checks\" in the line above)")


def exchange_checks(dev, rank, world, x, mask, gates, caps, cap, padded, R, brt_dist):
    """Correctness of the expert-parallel step on THIS run's ranks, outside any timed region:
    (1) the round trip forward -> inverse returns the dispatched rows bit for bit;
    (2) every row lands where the reference's walk puts it (src/distributed/collective.cc:
        142-182): rows that carry (source rank, source row) are exchanged and the receiver
        checks each [local expert][source] segment against the size matrix of all ranks;
    (3) the step's output equals the same step without any exchange (identity expert).
    Every verdict is the AND over all ranks."""
    import torch.distributed as dist

    m = mask
    if padded:
        m, _ = R.throttle_hotmask(mask, torch.zeros_like(caps), caps)
    idx, loads = R.generate_indices_and_loads(m, caps)
    (routed,) = R.dispatch_with_indices_and_loads(x, idx, loads, None, False, None, padded, cap)
    (local_out,) = R.combine_with_indices_and_loads(routed, idx, loads, gates, None, padded)
    recv, out_loads, in_loads = brt_dist.group_sparse_a2a(routed, loads, padded, cap)
    back = brt_dist.size_known_group_sparse_a2a(recv, out_loads, in_loads, padded)
    round_trip = bool(torch.equal(back, routed))
    (ep_out,) = R.combine_with_indices_and_loads(back, idx, loads, gates, None, padded)
    same_as_local = bool(torch.equal(ep_out, local_out))

    # (2) landing layout, with 16-byte rows that name their origin
    E = loads.numel()
    G = E // world
    n_rows = routed.size(0)
    ident = torch.empty((n_rows, 4), dtype=torch.int32, device=dev)
    ident[:, 0] = rank
    ident[:, 1] = torch.arange(n_rows, dtype=torch.int32, device=dev)
    ident[:, 2:] = 0
    got, _, _ = brt_dist.group_sparse_a2a(ident, loads, padded, cap)
    all_loads = [torch.empty_like(loads) for _ in range(world)]
    dist.all_gather(all_loads, loads.contiguous())
    S = torch.stack(all_loads).cpu().numpy().astype(np.int64)       # [source][global expert]
    starts = np.zeros_like(S)
    if padded:
        starts[:] = np.arange(E)[None, :] * cap
    else:
        starts[:, 1:] = np.cumsum(S, axis=1)[:, :-1]
    want_rank, want_row, at = [], [], []
    cursor = 0
    for j in range(G):
        for src in range(world):
            e = rank * G + j
            cnt = int(min(S[src, e], cap) if padded else S[src, e])
            want_rank.append(np.full(cnt, src, dtype=np.int32))
            want_row.append(starts[src, e] + np.arange(cnt))
            at.append((cursor if not padded else (j * world + src) * cap) + np.arange(cnt))
            cursor += cnt
    at = torch.from_numpy(np.concatenate(at)).to(dev)
    want_rank = torch.from_numpy(np.concatenate(want_rank)).to(dev)
    want_row = torch.from_numpy(np.concatenate(want_row).astype(np.int32)).to(dev)
    rows_ok = got.size(0) == (E * cap if padded else cursor)
    layout = bool(rows_ok and torch.equal(got[at, 0], want_rank)
                  and torch.equal(got[at, 1], want_row))
    # (4) the dispatch that stores its rows straight into the peers equals the two steps
    fused = brt_dist.dispatch_group_sparse_a2a(x, idx, loads, padded, cap)
    fused_same = True
    if fused is not None:
        two = brt_dist.group_sparse_a2a(routed, loads, padded, cap)
        if padded:
            valid = torch.zeros(two[0].size(0), dtype=torch.bool, device=dev)
            for b, cnt in enumerate(two[1].tolist()):
                valid[b * cap:b * cap + min(cnt, cap)] = True
            fused_same = bool(torch.equal(fused[0][valid], two[0][valid]))
        else:
            fused_same = bool(torch.equal(fused[0], two[0]))
        fused_same = fused_same and bool(torch.equal(fused[1], two[1]))
    # (5) the combine that pulls its rows from the peers equals inverse exchange + combine
    pull_same, pull_ran = True, False
    fwd3 = brt_dist.group_sparse_a2a(routed, loads, padded, cap)
    pulled_out = brt_dist.combine_group_sparse_a2a(fwd3[0], idx, gates, fwd3[1], fwd3[2], padded)
    if pulled_out is not None:
        pull_ran = True
        pull_same = bool(torch.equal(pulled_out, local_out))
    else:
        brt_dist.size_known_group_sparse_a2a(fwd3[0], fwd3[1], fwd3[2], padded)
    verdict = torch.tensor([int(round_trip), int(layout), int(same_as_local), int(fused_same),
                            int(pull_same)], device=dev)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    v = verdict.tolist()
    return {"round_trip_bit_exact": bool(v[0]), "forward_layout_matches_reference_walk": bool(v[1]),
            "step_equals_single_rank_step": bool(v[2]),
            "fused_dispatch_exchange_equals_two_steps": bool(v[3]),
            "fused_exchange_combine_equals_two_steps": bool(v[4]),
            "fused_exchange_combine": "ran" if pull_ran
            else "not available on this transport (two steps)",
            "fused_dispatch_exchange": "ran" if fused is not None
            else "not available on this transport (two steps)", "ranks": world,
            "rows_exchanged_per_rank": int(n_rows)}


def bias_for_local_fraction(world: int, target: float = 0.6) -> float:
    """The value to add to the logits of ONE rank's experts so that about ``target`` of the
    cfg4 top-2 picks go to them (the workload states 60 %); found by bisection on a sample
    that every rank draws alike."""
    w = WORKLOADS["cfg4"]
    E, k = w["E"], w["k"]
    G = E // world
    g = torch.Generator(device="cpu").manual_seed(4242)
    logits = torch.randn((8192, E), generator=g) + torch.randn(
        (E,), generator=torch.Generator(device="cpu").manual_seed(4999))
    lo, hi = 0.0, 8.0
    for _ in range(24):
        mid = 0.5 * (lo + hi)
        biased = logits.clone()
        biased[:, :G] += mid
        local = float((torch.topk(biased, k, dim=1).indices < G).float().mean())
        if local < target:
            lo = mid
        else:
            hi = mid
    return round(0.5 * (lo + hi), 3)


def measure_a2a_cfg4(dev, rank, world, R, brt_dist, local_bias: float, iters: int = 10,
                     favour_shift: int = 0, loads_only: bool = False,
                     uniform_loads: bool = False):
    """The exchange the metric's all-to-all figure is quoted on (cfg4: T = 65536 tokens per
    rank, d = 2048 bf16, 64 experts, top-2, packed buckets), forward and back, with the timing
    protocol of benchmark/micro/distributed/sparse_a2a.py:53-100: CUDA events around
    group_sparse_a2a and size_known_group_sparse_a2a, host work of the calls included.
    Bus GB/s = bytes this rank sends to OTHER ranks / time; the slowest rank counts.
    ``uniform_loads``: the bucket sizes are drawn as that script draws them
    (``torch.randint(load, (world * local_expert,))`` seeded by the rank, sparse_a2a.py:56-60)
    with ``load`` = 2 x the mean cfg4 bucket, so a rank holds T * k rows on average; otherwise
    they come from top-2 picks on gate logits that carry a per-expert bias shared by all
    ranks (hot experts, so some rank receives well above the mean).
    ``local_bias`` > 0 skews each rank's picks towards its own experts
    (benchmark/micro/distributed/placement_a2a.py:54-80 measures that case)."""
    import torch.distributed as dist
    from brainstorm_b200 import _lib as brt_lib

    w = WORKLOADS["cfg4"]
    T, d, E, k = w["T"], w["d"], w["E"], w["k"]
    G = E // world
    g = torch.Generator(device="cpu").manual_seed(4000 + rank)
    gb = torch.Generator(device="cpu").manual_seed(4999)
    logits = torch.randn((T, E), generator=g) + torch.randn((E,), generator=gb)
    if local_bias:
        favoured = (rank + favour_shift) % world
        logits[:, favoured * G:(favoured + 1) * G] += local_bias
    if uniform_loads:
        gu = torch.Generator(device="cpu").manual_seed(rank)
        loads = torch.randint(2 * T * k // E, (E,), generator=gu, dtype=torch.int32).to(dev)
    else:
        picks = torch.topk(logits, k, dim=1).indices
        mask = torch.zeros((T, E), dtype=torch.int32).scatter_(1, picks, 1).to(dev)
        _, loads = R.generate_indices_and_loads(mask)
    if loads_only:
        return {"loads_rank": loads}
    rows = int(loads.sum().item())
    x = torch.empty((rows, d), dtype=torch.bfloat16, device=dev).normal_()
    sent = loads.reshape(world, G).sum(dim=1)
    remote = int((sent.sum() - sent[rank]).item()) * d * 2

    def once(record=None):
        if record:
            record[0].record()
        recv, out_loads, in_loads = brt_dist.group_sparse_a2a(x, loads)
        if record:
            record[1].record()
        back = brt_dist.size_known_group_sparse_a2a(recv, out_loads, in_loads)
        if record:
            record[2].record()
        return back

    for _ in range(3):
        back = once()
    ok = bool(torch.equal(back, x))
    dist.barrier()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(iters)]
    brt_lib.query("brt_profile_enable", 1)
    for i in range(iters):
        once(evs[i])
    torch.cuda.synchronize()
    brt_lib.query("brt_profile_enable", 0)
    import ctypes
    report = ctypes.create_string_buffer(8192)
    brt_lib.call("brt_profile_report", report, len(report))
    timed = json.loads(report.value.decode())
    fwd = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    # bytes every rank sends to / receives from OTHER ranks in one direction of the exchange
    _, recv_sizes, _ = brt_dist.group_sparse_a2a(x, loads)
    got = recv_sizes.reshape(G, world).sum(dim=0)
    received = int((got.sum() - got[rank]).item()) * d * 2
    mine = torch.tensor([float(remote), float(received)], device=dev, dtype=torch.float64)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    per_rank = torch.stack(everyone).cpu()
    mean_remote = float(per_rank[:, 0].mean())
    busiest = float(per_rank.max())
    stats = torch.tensor([fwd, bwd], device=dev, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    fwd, bwd = stats.tolist()
    all_ok = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(all_ok, op=dist.ReduceOp.MIN)
    kernels = {name: round(t["total_ms"] / max(t["launches"], 1), 5)
               for name, t in timed.items() if name.startswith("p2p_")}
    from brainstorm_b200.runtime import p2p
    return {
        "workload": "cfg4 exchange: d=2048 bf16, E=64, packed buckets; "
                    + ("bucket sizes ~ randint(4096) seeded by the rank (T*k = 131072 rows per "
                       "rank on average), the draw of the reference's sparse_a2a.py"
                       if uniform_loads else
                       "T=65536 per rank, top-2 picks on logits with a per-expert bias shared "
                       "by all ranks (hot experts)")
                    + (f", logits of a rank's own experts +{local_bias}" if local_bias else ""),
        "forward_ms": fwd, "backward_ms": bwd, "iterations": iters,
        "remote_bytes_per_rank_per_direction": {
            "mean": mean_remote, "sent_min": float(per_rank[:, 0].min()),
            "sent_max": float(per_rank[:, 0].max()), "received_max": float(per_rank[:, 1].max())},
        "bus_gbs_forward": mean_remote / (fwd * 1e-3) / 1e9,
        "bus_gbs_backward": mean_remote / (bwd * 1e-3) / 1e9,
        "frac_of_900_forward": mean_remote / (fwd * 1e-3) / 1e9 / 900.0,
        "frac_of_900_backward": mean_remote / (bwd * 1e-3) / 1e9 / 900.0,
        "busiest_link_gbs_forward": busiest / (fwd * 1e-3) / 1e9,
        "busiest_link_gbs_backward": busiest / (bwd * 1e-3) / 1e9,
        "busiest_link_frac_of_900": busiest / (max(fwd, bwd) * 1e-3) / 1e9 / 900.0,
        "bytes_note": "bus GB/s = mean over ranks of the bytes a rank sends to OTHER ranks per "
                      "direction / the slowest rank's time of the op (host work included). "
                      "Where the buckets are uneven some rank receives (forward) and sends "
                      "back (inverse) more than the mean: busiest_link is that rank's bytes "
                      "over the same time, the figure the link ceiling applies to",
        "kernel_ms_rank0": kernels,
        "round_trip_bit_exact": bool(all_ok.item()),
        "transport": "peer-memory landing kernels over NVLink" if p2p.arena() is not None
                     else "nccl send/recv",
        "loads_rank": loads,
    }


def measure_balanced_placement(dev, rank, world, x, mask, gates, caps, cap, padded, R, brt_dist,
                               steps: int):
    """The same step with the experts re-placed so that every rank hosts about the same number
    of routed rows (what a placement search is for: python/brt/runtime/placement.py:139-357
    searches placements from captured loads).  The exchange is bound by the busiest receiver's
    link; with popular experts spread over the ranks that receiver is an average one.  Experts
    are dealt to ranks greedily, most popular first, each rank taking E / W of them
    (``runtime.placement.load_balanced_placement``); the columns of the hot mask and of the
    gates are permuted accordingly.  Returns the step time
    (CUDA graph replay when every rank could capture, else eager) and the busiest receiver's
    share before and after."""
    import torch.distributed as dist
    from brainstorm_b200.runtime import p2p as brt_p2p

    E = mask.size(1)
    G = E // world
    if padded:
        m, _ = R.throttle_hotmask(mask, torch.zeros_like(caps), caps)
    else:
        m = mask
    mine = m.sum(dim=0).to(torch.int64)
    per_rank = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(per_rank, mine)
    S = torch.stack(per_rank).cpu()              # [source rank][expert]
    totals = S.sum(dim=0).tolist()

    def busiest_over_mean(assign):               # assign[p] = expert at position p
        S_perm = S[:, assign].reshape(world, world, G).sum(dim=2).clone()   # [source][dest]
        S_perm.fill_diagonal_(0)
        return float(S_perm.sum(dim=0).max()) / max(float(S_perm.sum(dim=1).float().mean()), 1.0)

    from brainstorm_b200.runtime.placement import load_balanced_placement
    assign = [e for hosted in load_balanced_placement(totals, world) for e in hosted]
    perm = torch.tensor(assign, dtype=torch.int64, device=dev)
    mask_b = mask.index_select(1, perm).contiguous()
    gates_b = gates.index_select(1, perm).contiguous()
    zeros_e = torch.zeros((E,), dtype=torch.int32, device=dev)

    def step():
        if padded:
            idx, loads, _ = R.throttle_and_generate_indices(mask_b, torch.zeros_like(zeros_e),
                                                            caps, caps)
        else:
            idx, loads = R.generate_indices_and_loads(mask_b, caps)
        with brt_dist.replayable_exchanges():
            recv, out_loads, in_loads = brt_dist.dispatch_group_sparse_a2a_device(
                x, idx, loads, padded, cap)
            back = brt_dist.size_known_group_sparse_a2a(recv, out_loads, in_loads, padded)
        (out,) = R.combine_with_indices_and_loads(back, idx, loads, gates_b, None, padded)
        return out

    graph, why = None, ""
    try:
        if brt_p2p.arena() is None:
            raise RuntimeError("no peer-memory arena")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
    except Exception as exc:  # noqa: BLE001
        graph, why = None, f"{type(exc).__name__}: {exc}"[:160]
    agreed = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
    if int(agreed.item()) != 1:
        return {"unavailable": why or "another rank could not capture the step"}
    for _ in range(3):
        graph.replay()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"ms_per_step": float(t.item()),
            "busiest_receiver_over_mean": {"block_placement": round(busiest_over_mean(list(range(E))), 3),
                                           "balanced_placement": round(busiest_over_mean(assign), 3)},
            "note": "same cells, gates and capacities; experts dealt to ranks most popular "
                    "first so that every rank receives about the mean (the headline value "
                    "keeps the block placement of the stated config)"}


def measure_locality(loads, world, dev, brt_dist):
    """The greedy rank matching on the gathered [W, W, G] load matrix: kernel time (CUDA
    events, median of 11) and the rows that stay on their own rank before and after it."""
    import torch.distributed as dist
    from brainstorm_b200._C import distributed as D

    G = loads.numel() // world
    mine = loads.to(torch.int32).contiguous()
    rows = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(rows, mine)
    matrix = torch.stack(rows).reshape(world, world, G).contiguous()
    ts = []
    for _ in range(14):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        reordered, order = D.group_locality_reorder(matrix, world, G)
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    total = int(matrix.sum())
    diag = lambda m: int(sum(int(m[i, i].sum()) for i in range(world)))
    return {"reorder_kernel_us": round(sorted(ts[3:])[5], 2),
            "local_rows_fraction": round(diag(matrix) / max(total, 1), 4),
            "local_rows_fraction_after_reorder": round(diag(reordered) / max(total, 1), 4),
            "reorder_indices": order.tolist()}


def measure_gate(wl, dev, w, R, padded, caps):
    """Device time (CUDA events, median of 11, L2 flushed in between) of turning the fp32
    score matrix into seat indices: the reference's protocol as torch ops (topk, zeros,
    scatter_) followed by this library's throttle and index ops, beside the library's gate
    kernel, which takes the scores straight to the (throttled) mask or to the indices."""
    score = wl["score"].to(dev)
    if not R.route_scores_supported(score):
        return None
    T, E, k = w["T"], w["E"], w["k"]
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)

    threshold = w.get("threshold") if w.get("protocol") == "threshold" else None
    decide = dict(decision="threshold", threshold=threshold) if threshold is not None else \
        dict(decision="topk", top_k=k)

    def torch_protocol():
        if threshold is not None:
            mask = (score > threshold).to(torch.int32)
        else:
            picks = torch.topk(score, k, dim=1).indices
            mask = torch.zeros((T, E), dtype=torch.int32, device=dev).scatter_(1, picks, 1)
        if padded:
            mask, _ = R.throttle_hotmask(mask, torch.zeros(E, dtype=torch.int32, device=dev), caps)
        return R.generate_indices_and_loads(mask, caps)

    def gate_kernel():
        if padded:  # decision, throttle and index scan in one launch
            i, l, _ = R.route_scores(score, output="throttled_seat_indices",
                                     prefix=torch.zeros(E, dtype=torch.int32, device=dev),
                                     throttle_capacity=caps, supported_capacities=caps, **decide)
            return i, l
        return R.route_scores(score, output="seat_indices", **decide)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(11):
            flush.zero_()
            try:
                torch.cuda._sleep(400000)  # lets the host enqueue the whole chain first
            except Exception:
                pass
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2], out

    t_torch, (i0, l0) = timed(torch_protocol)
    t_gate, (i1, l1) = timed(gate_kernel)
    return {"scores_to_indices_ms": {"torch_protocol_then_index_ops": round(t_torch, 5),
                                     "gate_kernel": round(t_gate, 5)},
            "same_result": bool(torch.equal(i0, i1) and torch.equal(l0, l1)),
            "launches": {"torch_protocol_then_index_ops":
                         ("compare, cast" if threshold is not None else "topk, zeros, scatter_")
                         + (", throttle, indices" if padded else ", indices"),
                         "gate_kernel": "route_scores(throttled seat indices)" if padded
                         else "route_scores(seat indices)"}}


def measure_expert_gemm(wl, dev, idx_loads, cap, peaks):
    """The expert side of the dispatched layout (not part of the routing step): a grouped
    linear layer [d -> 4d] over the rows this workload dispatches, on the tensor cores, with
    the per-expert loads staying on the device.  CUDA events, median of 7, against the measured
    sustained bf16 GEMM rate of this pool's B200s."""
    from brainstorm_b200._C import expert as X

    w = wl["spec"]
    if w["dtype"] != "bf16" or w["d"] % 128 != 0 or w["E"] > 1024:
        return None
    E, d = w["E"], w["d"]
    loads = idx_loads
    padded = cap > 0
    L = cap * E if padded else int(loads.sum().item())
    if L * 4 * d * 2 > 8e9:
        return None
    rows = torch.empty((L, d), dtype=torch.bfloat16, device=dev).normal_()
    weights = torch.empty((E, 4 * d, d), dtype=torch.bfloat16, device=dev).normal_(0, d ** -0.5)
    for _ in range(3):
        X.grouped_expert_linear(rows, weights, loads, padded, cap, True)
    X.check_status()
    ts = []
    for _ in range(7):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        X.grouped_expert_linear(rows, weights, loads, padded, cap, True)
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ms = sorted(ts)[3]
    kept = loads.clamp(max=cap) if padded else loads
    flops = 2.0 * float(kept.sum().item()) * d * 4 * d
    tf = flops / (ms * 1e-3) / 1e12
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    return {"op": f"grouped expert linear {d} -> {4 * d} with ReLU over the dispatched rows "
                  f"({int(kept.sum().item())} rows in {E} experts)",
            "ms": round(ms, 4), "tflops": round(tf, 1), "peak_tflops": peak,
            "peak_kind": "measured sustained cuBLAS bf16" if "bf16_tflops_sustained" in peaks
                         else "fallback",
            "frac": round(tf / peak, 4), "kernel": "expert_gemm_kernel (tcgen05.mma, TMA, TMEM)"}


def measure_e2e(wl, dev, args, ScatterRouter, GatherRouter, distributed, world):
    """Same routing through ScatterRouter / GatherRouter, inputs in pinned host memory, the
    combined result copied back to the host, all inside the timed region."""
    import torch.distributed as dist

    w = wl["spec"]
    T, E = w["T"], w["E"]
    cap = wl["cap"]
    padded = cap > 0
    kind = "distributed_fused" if distributed else "fused"
    fkw = {"max_path_padding": padded, "max_path_load": cap}
    if padded:
        fkw["supported_capacities"] = [cap]
    if w.get("protocol") == "threshold":
        proto, pkw = "threshold", {"threshold": w["threshold"]}
    else:
        proto, pkw = "topk", {"top_k": w["k"]}
    scatter = ScatterRouter(protocol_type=proto, fabric_type=f"{kind}_dispatch",
                            protocol_kwargs=pkw, fabric_kwargs=fkw).to(dev)
    gather = GatherRouter(fabric_type=f"{kind}_combine",
                          fabric_kwargs={"transform": True, "max_path_padding": padded}).to(dev)
    x_h = wl["x"].pin_memory()
    score_h = wl["score"].pin_memory()
    gates_h = wl["gates"].pin_memory()
    out_h = torch.empty_like(wl["x"]).pin_memory()
    from brainstorm_b200.runtime.grid_tensor import init_grid_tensor

    def step():
        x = init_grid_tensor(x_h.to(dev, non_blocking=True), [None], [None])
        score = score_h.to(dev, non_blocking=True)
        gates = gates_h.to(dev, non_blocking=True)
        routed = scatter(x, score)
        out = gather(routed, None, gates)
        out_h.copy_(out, non_blocking=True)

    def timed(run_steps, steps):
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        run_steps(steps)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        if distributed:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(3):
        step()
    steps = max(3, min(args.steps, 20))
    serial_ms = timed(lambda n: [step() for _ in range(n)], steps)

    # The same steps as a three-stage pipeline, the way a serving loop feeds a GPU: step i+1's
    # inputs go up on a copy stream and step i-1's result comes down on another while step i
    # routes.  Every step still copies its own inputs in and its own result out; two device
    # input slots and two pinned output slots are reused in turn.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    slots = [{"x": torch.empty_like(wl["x"], device=dev),
              "score": torch.empty_like(wl["score"], device=dev),
              "gates": torch.empty_like(wl["gates"], device=dev),
              "out_h": torch.empty_like(wl["x"]).pin_memory(),
              "loaded": torch.cuda.Event(), "consumed": torch.cuda.Event(),
              "drained": torch.cuda.Event()} for _ in range(2)]

    def copy_in(i):
        sl = slots[i % 2]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(sl["consumed"])
            sl["x"].copy_(x_h, non_blocking=True)
            sl["score"].copy_(score_h, non_blocking=True)
            sl["gates"].copy_(gates_h, non_blocking=True)
            sl["loaded"].record(s_in)

    def pipelined(n):
        copy_in(0)
        for i in range(n):
            sl = slots[i % 2]
            if i + 1 < n:
                # the next step's inputs go up while this step routes; enqueued before the one
                # point of a step where the host may wait (the sizes of an exchange)
                copy_in(i + 1)
            main.wait_event(sl["loaded"])
            x = init_grid_tensor(sl["x"], [None], [None])
            routed = scatter(x, sl["score"])
            out = gather(routed, None, sl["gates"])
            sl["consumed"].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(sl["consumed"])
                if i >= 2:
                    s_out.wait_event(sl["drained"])
                out.record_stream(s_out)
                sl["out_h"].copy_(out, non_blocking=True)
                sl["drained"].record(s_out)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    pipelined(4)
    ms = timed(pipelined, steps)
    h2d = sum(t.numel() * t.element_size() for t in (x_h, score_h, gates_h))
    d2h = out_h.numel() * out_h.element_size()
    return {"value": world * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "api": f"ScatterRouter({proto}, {kind}_dispatch) -> GatherRouter({kind}_combine)",
            "schedule": "copy-in, route and copy-out of consecutive steps overlap (2 slots)",
            "serial_ms_per_step": serial_ms,
            "serial_value": world * T / (serial_ms * 1e-3)}


# --------------------------------------------------------------------------------- CPU arm
def cpu_pass(wl, oracle):
    w = wl["spec"]
    cap = wl["cap"]
    padded = cap > 0
    dt = w["dtype"]
    x = wl["x_bits"]
    mask = wl["mask_np"]
    caps = [cap] * w["E"] if padded else None
    m = mask
    if padded:
        m, _ = oracle.throttle_hotmask(mask, np.zeros(w["E"], dtype=np.int32),
                                       np.full(w["E"], cap, dtype=np.int32))
    idx, loads = oracle.generate_indices_and_loads(m, caps)
    (routed,) = oracle.dispatch_with_indices_and_loads(x, idx, loads, max_path_padding=padded,
                                                       max_path_load=cap, dtype=dt)
    (out,) = oracle.combine_with_indices_and_loads(routed, idx, loads, wl["gates_np"],
                                                   max_path_padding=padded, dtype=dt)
    return out


def cpu_baseline(wl, budget_s: float = 15.0, min_passes: int = 2):
    """The reference has no CPU implementation of the fused router ops; the baseline is the
    CPU restatement in oracle/ (C + OpenMP) on all host cores."""
    import oracle

    w = wl["spec"]
    cores = os.cpu_count() or 1
    oracle.set_threads(cores)
    if "x_bits" not in wl:
        xt = wl["x"]
        wl["x_bits"] = xt.numpy() if w["dtype"] == "f32" else \
            xt.view(torch.int16).numpy().view(np.uint16)
        wl["mask_np"] = wl["mask"].numpy()
        wl["gates_np"] = wl["gates"].numpy()
    cpu_pass(wl, oracle)  # warm-up
    times = []
    t_all = time.perf_counter()
    while len(times) < min_passes or (time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter()
        cpu_pass(wl, oracle)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": w["T"] / best, "unit": UNIT, "cores": min(cores, oracle.max_threads()),
            "kind": "port",
            "sample": f"whole batch of {w['T']} tokens, best of {len(times)} passes "
                      f"({sum(times):.1f} s of CPU work)",
            "ms_per_step": best * 1e3}


def run_reference(args):
    """Reference arm: the CPU restatement of the reference's router on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload)
    w = wl["spec"]
    import oracle

    cores = os.cpu_count() or 1
    oracle.set_threads(cores)
    xt = wl["x"]
    wl["x_bits"] = xt.numpy() if w["dtype"] == "f32" else \
        xt.view(torch.int16).numpy().view(np.uint16)
    wl["mask_np"] = wl["mask"].numpy()
    wl["gates_np"] = wl["gates"].numpy()
    warm = max(args.warmup, 3)  # the same rule as the GPU arm
    for _ in range(warm):
        cpu_pass(wl, oracle)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_pass(wl, oracle)
    ms = (time.perf_counter() - t0) / steps * 1e3
    value = w["T"] / (ms * 1e-3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"],
        "data": "synthetic",
        "config": config_of(args.workload, max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": UNIT,
                         "cores": min(cores, oracle.max_threads()), "kind": "port",
                         "sample": f"whole batch of {w['T']} tokens per step, {steps} steps",
                         "note": "the reference has no CPU implementation of its fused router "
                                 "ops (every op asserts CUDA tensors); this is its algorithm "
                                 "restated in C + OpenMP (oracle/), on all host cores, one "
                                 "rank's batch"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--local-bias", type=float, default=0.0,
                    help="added to the logits of a rank's own experts in the timed step's workload "
                         "(N>1); the locality_cfg4 block calibrates its own bias to 60%% local "
                         "picks at the world size it runs on")
    ap.add_argument("--no-fused-exchange", action="store_true",
                    help="at N>1 run dispatch and the forward exchange as two ops instead of the "
                         "one kernel that stores the dispatched rows straight into the peers")
    ap.add_argument("--pull-combine", action="store_true",
                    help="at N>1 run the inverse exchange and the combine as the one kernel that "
                         "pulls the expert outputs from the peers (checked either way; the "
                         "default, rows pushed back and combined locally, measured faster)")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of a CUDA graph replay")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
