"""ctypes binding of ``libbrt_b200.so`` (the C ABI declared in ``include/brt_b200.h``).

There is no fallback: if the library is missing or a call fails, a ``RuntimeError`` says
so.  Pointers are passed as integers (``tensor.data_ptr()``), streams as
``torch.cuda.current_stream().cuda_stream``.
"""
import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libbrt_b200.so"

_lib = None

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_int = ctypes.c_int
_sz = ctypes.c_size_t
_u64 = ctypes.c_uint64

# name -> (restype, argtypes); kept in step with include/brt_b200.h
SIGNATURES = {
    "brt_abi_version": (_int, []),
    "brt_last_error": (ctypes.c_char_p, []),
    "brt_kernel_launch_count": (ctypes.c_uint64, []),
    "brt_profile_enable": (None, [_int]),
    "brt_profile_report": (_int, [_vp, _sz]),
    "brt_index_scratch_bytes": (_sz, [_i64, _int]),
    "brt_generate_indices_and_loads": (
        _int, [_vp, _vp, _vp, _vp, _i64, _int, _vp, _int, _int, _int, _int, _vp, _sz, _vp]),
    "brt_static_index_scratch_bytes": (_sz, []),
    "brt_generate_indices_and_loads_static": (
        _int, [_vp, _vp, _vp, _i64, _int, _vp, _int, _int, _int, _int, _vp]),
    "brt_index_status": (_int, []),
    "brt_index_status_reset": (None, []),
    "brt_index_set_test_hooks": (None, [_int, _int]),
    "brt_route_scores": (
        _int, [_vp, _i64, _int, _int, _int, ctypes.c_float, _int, _int, _vp, _vp, _vp, _vp, _int,
               _int, _int, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "brt_throttle_hotmask": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _vp, _sz, _vp]),
    "brt_throttle_and_generate_indices": (
        _int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _vp, _int, _int, _int, _vp, _sz,
               _vp]),
    "brt_convert_index_format": (_int, [_vp, _vp, _vp, _i64, _int, _int, _vp]),
    "brt_dispatch_scratch_bytes": (_sz, [_i64, _int]),
    "brt_dispatch_with_indices_and_loads": (
        _int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _i32, _i64, _int, _int,
               _int, _vp, _vp, _sz, _vp]),
    "brt_combine_with_indices_and_loads": (
        _int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _i32, _int, _int, _int, _vp]),
    "brt_sum_rows_scratch_bytes": (_sz, [_i64, _i64]),
    "brt_sum_rows_by_index": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "brt_grouped_expert_gemm": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i32, _i64, _i64, _int,
                                       _vp, _vp]),
    "brt_locality_reorder": (_int, [_vp, _int, _vp, _vp, _vp]),
    "brt_group_locality_reorder": (_int, [_vp, _int, _int, _vp, _vp, _vp]),
    "brt_nccl_get_unique_id": (_int, [_vp]),
    "brt_nccl_init": (_int, [_vp, _int, _int]),
    "brt_nccl_is_initialized": (_int, []),
    "brt_nccl_world": (_int, [ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "brt_nccl_destroy": (_int, []),
    "brt_broadcast": (_int, [_vp, _vp, _i64, _int, _vp]),
    "brt_exchange": (_int, [_vp, _vp, _i64, _int, _int, _vp]),
    "brt_scatter": (_int, [_vp, _vp, _i64, _int, _vp]),
    "brt_gather": (_int, [_vp, _vp, _i64, _int, _vp]),
    "brt_all_to_all": (_int, [_vp, _vp, _i64, _vp]),
    "brt_group_asymmetry_all_to_all": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "brt_group_sparse_all_to_all": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "brt_p2p_alloc": (_int, [_sz, ctypes.POINTER(_vp), _vp]),
    "brt_p2p_open": (_int, [_vp, ctypes.POINTER(_vp)]),
    "brt_p2p_close": (_int, [_vp]),
    "brt_p2p_free": (_int, [_vp]),
    "brt_p2p_push": (_int, [_vp, _int, _vp, _vp, _vp, _int, _int, _u64, _vp, _vp, _vp]),
    "brt_p2p_post": (_int, [_vp, _int, _int, _int, _u64, _vp, _vp, _vp]),
    "brt_p2p_land": (_int, [_vp, _vp, _vp, _int, _int, _int, _int, _int, _i64, _i64, _i64, _vp, _u64,
                            _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "brt_p2p_wait": (_int, [_vp, _int, _int, _u64, _vp, _vp, _u64, _vp]),
    "brt_p2p_control_bytes": (_sz, []),
    "brt_p2p_ctx_create": (_int, [_int, _int, _vp, _vp, _sz, _vp]),
    "brt_p2p_ctx_destroy": (None, [_vp]),
    "brt_p2p_ctx_set_wait_limit": (_int, [_vp, _u64]),
    "brt_p2p_ctx_status": (_int, [_vp]),
    "brt_p2p_ctx_reset_status": (_int, [_vp]),
    "brt_p2p_ctx_exchanges": (_u64, [_vp]),
    "brt_p2p_sparse_forward_begin": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _int, _vp, _vp,
                                            _int]),
    "brt_p2p_dispatch_forward_begin": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _i64,
                                              _vp, _vp, _int]),
    "brt_p2p_dispatch_land": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _int, _int, _int, _i64,
                                     _i64, _vp, _u64, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "brt_p2p_ctx_trace": (_int, [_vp, _vp]),
    "brt_p2p_combine_backward": (_int, [_vp, _u64, _int, _i64, _i64, _i64, _vp, _vp, _int, _int,
                                        _i64, _vp, _vp, _int]),
    "brt_p2p_ctx_replay_begin": (_int, [_vp]),
    "brt_p2p_ctx_replay_end": (_int, [_vp]),
    "brt_p2p_forward_device_sizes": (_int, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "brt_p2p_sparse_forward_sizes": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "brt_p2p_sparse_backward": (_int, [_vp, _u64, _int, _i64, _i64, _int, _int, _vp, _vp, _int,
                                       _vp, _vp]),
}


class BrtError(RuntimeError):
    """A failed library call; ``status`` is the brt_status code (0 when not from the library)."""

    def __init__(self, message: str, status: int = 0):
        super().__init__(message)
        self.status = status


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise BrtError(
            f"{LIB_PATH} is missing: build it with `python -m brainstorm_b200.build` "
            "(there is no CPU or eager fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue  # reported by exported_symbols()/call()
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def exported(name: str) -> bool:
    return hasattr(load(), name)


_fns = {}


def _fn(name: str):
    fn = _fns.get(name)
    if fn is None:
        fn = getattr(load(), name, None)
        if fn is None:
            raise BrtError(f"libbrt_b200.so does not export {name}")
        _fns[name] = fn
    return fn


def call(name: str, *args):
    """Call a status-returning entry point; raise BrtError with the library's message."""
    rc = _fn(name)(*args)
    if rc != 0:
        msg = load().brt_last_error().decode("utf-8", "replace")
        raise BrtError(f"{name} failed (status {rc}): {msg}", rc)


def query(name: str, *args):
    """Call an entry point that returns a value rather than a status."""
    return _fn(name)(*args)


# The ops sit on the host's critical path of an eager step (three launches of 15 to 40 us each),
# so the two per-call lookups they need are taken the short way: the raw handle of torch's
# current stream and a device guard that does nothing when the device is already current.
def raw_stream(device=None) -> int:
    """``torch.cuda.current_stream(device).cuda_stream`` without building a Stream object."""
    import torch

    index = None if device is None else getattr(device, "index", device)
    if index is None:
        index = torch.cuda.current_device()
    try:
        return torch._C._cuda_getCurrentRawStream(index)
    except AttributeError:  # a torch build without the shortcut
        return torch.cuda.current_stream(index).cuda_stream


class device_guard:
    """``with torch.cuda.device(device)`` for a device that usually is the current one."""

    __slots__ = ("index", "prev")

    def __init__(self, device):
        self.index = getattr(device, "index", device)
        self.prev = -1

    def __enter__(self):
        import torch

        if self.index is not None and self.index != torch.cuda.current_device():
            self.prev = torch.cuda.current_device()
            torch.cuda.set_device(self.index)
        return self

    def __exit__(self, exc_type, exc, tb):
        if self.prev >= 0:
            import torch

            torch.cuda.set_device(self.prev)
        return False
