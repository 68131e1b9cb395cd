"""Regenerates the fixtures in this directory from the reference tree.

Run where the reference project is checked out (its location comes from
BRT_REFERENCE_ROOT) and the reference extensions have been built by
``python oracle/build.py --ref``:

    python tests/golden/make_golden.py

Writes
  notebook_vectors.json   saved cell outputs of sample/router/generate_indices.ipynb
                          (mask -> seat indices; throttle_hotmask in/out) parsed as text
  ref_python_vectors.npz  outputs of the reference's *Python* code run on CPU tensors:
                          its torch oracle FabricCPPTest.pt_generate_indices
                          (test/python/fabric_test.py:35-92) and its protocol classes
                          (python/brt/router/protocol/{topk,threshold}.py)

Nothing here is needed at test time except the two output files.
"""
import json
import os
import re
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(os.environ.get("BRT_REFERENCE_ROOT", str(REPO.parent / "reference")))


def _tensor_literals(text):
    """All ``tensor([...])`` literals of a printed cell output, as nested lists."""
    out = []
    for m in re.finditer(r"tensor\(", text):
        i = m.end()
        depth = 0
        j = i
        while j < len(text):
            if text[j] == "[":
                depth += 1
            elif text[j] == "]":
                depth -= 1
                if depth == 0:
                    break
            j += 1
        out.append(json.loads(re.sub(r"\s+", "", text[i:j + 1])))
    return out


def notebook_vectors():
    nb = json.load(open(REF / "sample/router/generate_indices.ipynb"))
    cells = nb["cells"]

    def text_of(c):
        return "".join("".join(o.get("text", "")) for o in c.get("outputs", []))

    mask = _tensor_literals(text_of(cells[0]))[0]
    seat, legacy_src = _tensor_literals(text_of(cells[1]))[:2]
    shuffled, loads, converted = _tensor_literals(text_of(cells[2]))[:3]
    t = _tensor_literals(text_of(cells[4]))
    src = "".join(cells[4]["source"])
    prefix_in = json.loads(re.search(r"prefix = torch\.tensor\((\[[^\]]*\])", src).group(1))
    threshold = json.loads(re.search(r"threshold = torch\.tensor\((\[[^\]]*\])", src).group(1))
    return {
        "source": "sample/router/generate_indices.ipynb",
        "indices": {
            "hot_mask": mask,
            "seat_indices": seat,
            # printed by an older API whose tag ("src") indices were 0-based cell ids with 0
            # doubling as "empty"; kept for the record, current kernels write cell+1
            "legacy_src_indices_zero_based": legacy_src,
            "shuffled_seat_indices": shuffled,
            "shuffled_loads": loads,
            "legacy_converted_zero_based": converted,
        },
        "throttle": {
            "hot_mask": t[0],
            "column_sums": t[1],
            "prefix_in": prefix_in,
            "threshold": threshold,
            "throttled_mask": t[2],
            "kept_counts": t[3],
            "prefix_out": t[4],
        },
    }


def _import_reference_python():
    """Make ``import brt...`` resolve to the reference's Python sources, with its compiled
    extension replaced by the build in oracle/_ref and its one missing dependency (nni)
    replaced by identity decorators."""
    sys.path.insert(0, str(REPO / "oracle" / "_ref"))
    import brt_ref_distributed
    import brt_ref_router

    nni = types.ModuleType("nni")
    common = types.ModuleType("nni.common")
    ser = types.ModuleType("nni.common.serializer")
    ser.trace = lambda cls=None, **kw: cls if cls is not None else (lambda c: c)
    ser.is_traceable = lambda x: False
    ser.is_wrapped_with_trace = lambda x: False
    sys.modules.update({"nni": nni, "nni.common": common, "nni.common.serializer": ser})
    sys.path.insert(0, str(REF / "python"))
    cpkg = types.ModuleType("brt._C")
    cpkg.__path__ = []
    cpkg.router = brt_ref_router
    sys.modules["brt._C"] = cpkg
    cpkg.distributed = brt_ref_distributed
    sys.modules["brt._C.router"] = brt_ref_router
    sys.modules["brt._C.distributed"] = brt_ref_distributed


def ref_python_vectors():
    _import_reference_python()
    sys.path.insert(0, str(REF / "test" / "python"))
    from fabric_test import FabricCPPTest
    from brt.router.protocol.threshold import ThresholdProtocol
    from brt.router.protocol.topk import TopKProtocol

    t = FabricCPPTest()
    g = torch.Generator().manual_seed(20231)
    out = {}
    cases = [
        # name, T, E, k, capacities, capacity_padding, path_wise_padding
        ("plain_top1", 512, 16, 1, None, False, False),
        ("plain_top4", 512, 16, 4, None, False, False),
        ("caps_top4", 512, 8, 4, [1, 2, 4, 8, 16, 32, 64, 128, 256, 512], False, False),
        ("caps_overflow", 512, 8, 4, [1, 2, 4, 8, 16, 32, 64, 128], False, False),
        ("pad_top1", 512, 8, 1, [1, 2, 4, 8, 16, 32, 64, 128, 256, 512], True, False),
        ("pad_overflow", 300, 4, 2, [16, 32, 100], True, False),
        ("pathwise", 256, 8, 4, [2, 4, 8, 16, 32, 64, 128, 256], True, True),
        ("ragged", 1037, 5, 2, None, False, False),
    ]
    for name, T, E, k, caps, cpad, pwise in cases:
        score = torch.randn((T, E), generator=g)
        idx = torch.topk(score, k, dim=1).indices
        mask = torch.zeros((T, E), dtype=torch.int32).scatter(1, idx, 1)
        caps_t = None if caps is None else torch.tensor(caps, dtype=torch.int32)
        out[f"idx/{name}/mask"] = mask.numpy()
        out[f"idx/{name}/caps"] = np.array([] if caps is None else caps, dtype=np.int32)
        out[f"idx/{name}/flags"] = np.array([cpad, pwise], dtype=np.int32)
        for tag in (False, True):
            i, l = t.pt_generate_indices(mask.clone(), caps_t, cpad, pwise, tag)
            out[f"idx/{name}/{'tag' if tag else 'seat'}_indices"] = i.numpy()
            out[f"idx/{name}/{'tag' if tag else 'seat'}_loads"] = l.numpy()
    # protocols
    score = torch.softmax(torch.randn((64, 8), generator=g), dim=1)
    out["proto/score"] = score.numpy()
    for k in (1, 2, 3):
        out[f"proto/topk{k}"] = TopKProtocol(top_k=k)(score).numpy()
    sig = torch.sigmoid(torch.randn((64, 8), generator=g))
    out["proto/sigmoid"] = sig.numpy()
    out["proto/threshold_0.5"] = ThresholdProtocol(threshold=0.5)(sig).numpy()
    out["proto/threshold_0.8_residual3"] = ThresholdProtocol(threshold=0.8, residual_path=3)(
        sig).numpy()
    return out


if __name__ == "__main__":
    json.dump(notebook_vectors(), open(HERE / "notebook_vectors.json", "w"), indent=1)
    np.savez_compressed(HERE / "ref_python_vectors.npz", **ref_python_vectors())
    print("wrote", HERE / "notebook_vectors.json", HERE / "ref_python_vectors.npz")
