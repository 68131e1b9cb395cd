"""Operator boundary: the same modules and function names the reference exposes as
``brt._C.router`` and ``brt._C.distributed`` (pybind11 extensions there; thin torch-facing
wrappers over the C ABI of ``libbrt_b200.so`` here)."""
from . import distributed, router  # noqa: F401
