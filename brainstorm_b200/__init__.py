"""brainstorm_b200 — B200-native routing hot path behind Brainstorm's router API.

The package mirrors the part of the reference's ``brt`` Python package that sits on the
token/sample routing path:

    brainstorm_b200._C.router        <->  brt._C.router        (index/load/dispatch/combine ops)
    brainstorm_b200._C.distributed   <->  brt._C.distributed   (variable-size all-to-all, reorder)
    brainstorm_b200.router           <->  brt.router           (ScatterRouter / GatherRouter, ...)
    brainstorm_b200.runtime          <->  brt.runtime          (GridTensor, Annotator, wrappers)

``install_as_brt()`` registers these modules under the reference's names so that code written
against ``import brt...`` runs unchanged.
"""
import importlib
import sys

__version__ = "0.1.0"

from .runtime.annotate import Annotator  # noqa: E402,F401
from .runtime.grid_tensor import GridTensor, to_grid_tensor, to_torch_tensor  # noqa: E402,F401

_ALIASES = (
    "", "_C", "_C.router", "_C.distributed", "router", "router.base", "router.scatter",
    "router.gather", "router.utils", "router.protocol", "router.protocol.base",
    "router.protocol.topk", "router.protocol.threshold", "router.protocol.switch",
    "router.protocol.swin_moe", "router.fabric", "router.fabric.base", "router.fabric.generic",
    "router.fabric.fused", "router.fabric.distributed", "router.fabric.distributed_slots", "runtime", "runtime.grid_tensor",
    "runtime.annotate", "runtime.registry", "runtime.distributed", "runtime.log",
    "runtime.placement",
)


def install_as_brt() -> None:
    """Make ``import brt``, ``import brt._C.router`` ... resolve to this package."""
    if "brt" in sys.modules and getattr(sys.modules["brt"], "__name__", "") != __name__:
        raise RuntimeError("another package named brt is already imported")
    for suffix in _ALIASES:
        name = __name__ + ("." + suffix if suffix else "")
        try:
            mod = importlib.import_module(name)
        except ModuleNotFoundError:
            continue
        sys.modules["brt" + ("." + suffix if suffix else "")] = mod
