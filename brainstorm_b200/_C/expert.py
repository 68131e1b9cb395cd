"""The expert side of the dispatched layout: a grouped linear layer on the tensor cores.

No counterpart in the reference's ``brt._C.router``: there the experts run as horizontally
fused kernels compiled by its JIT (``brt._C.jit`` ``homo_invoke``,
src/backend/torch/jit.cc:54-75; benchmark/switch_moe/switch_expert.py:62-99 builds the FFN of
a Switch layer from them).  This op consumes the same buffer and the same per-expert loads,
with the loads staying on the device.
"""
import torch

from .. import _lib

_error_words = {}


def _error_word(device: torch.device) -> torch.Tensor:
    word = _error_words.get(device.index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[device.index] = word
    return word


def grouped_expert_linear(rows: torch.Tensor, weights: torch.Tensor, loads: torch.Tensor,
                          max_path_padding: bool = False, max_path_load: int = 0,
                          relu: bool = False, out: torch.Tensor = None) -> torch.Tensor:
    """``out[r] = act(rows[r] @ weights[e].T)`` for the first ``loads[e]`` rows of every expert
    ``e`` of a dispatched buffer.

    ``rows`` [L, in] bf16 as ``dispatch_with_indices_and_loads`` returns it (padded to
    ``max_path_load`` rows per expert with ``max_path_padding``, else packed), ``weights``
    [E, out, in] bf16, ``loads`` [E] int32 on the device.  Returns [L, out] bf16; rows beyond an
    expert's load are left unwritten (combine never reads them).  ``in`` must be a multiple of
    64 and ``out`` of 128 (``NotImplementedError`` otherwise).  ``out``: a contiguous [L, out]
    bf16 tensor to write instead of a new one (e.g. ``expert_output_buffer`` of the
    expert-parallel exchange, which the fused combine pulls from)."""
    if not rows.is_cuda or not weights.is_cuda or not loads.is_cuda:
        raise RuntimeError("rows, weights and loads must be CUDA tensors")
    if rows.dtype != torch.bfloat16 or weights.dtype != torch.bfloat16:
        raise NotImplementedError("the tensor-core expert GEMM takes bf16 rows and weights")
    if rows.dim() != 2 or weights.dim() != 3 or weights.size(2) != rows.size(1) or \
            loads.numel() != weights.size(0):
        raise RuntimeError("expected rows [L, in], weights [E, out, in] and loads [E]")
    E, n_out, n_in = weights.shape
    L = rows.size(0)
    if max_path_padding:
        mpl = int(max_path_load) if max_path_load > 0 else L // E
        if mpl * E != L:
            raise RuntimeError("a padded buffer must hold max_path_load rows per expert")
    else:
        mpl = 0
    dev = rows.device
    with _lib.device_guard(dev):
        x = rows if rows.is_contiguous() else rows.contiguous()
        w = weights if weights.is_contiguous() else weights.contiguous()
        counts = loads if (loads.dtype == torch.int32 and loads.is_contiguous()) \
            else loads.to(torch.int32).contiguous()
        if out is None:
            out = torch.empty((L, n_out), dtype=torch.bfloat16, device=dev)
        elif out.shape != (L, n_out) or out.dtype != torch.bfloat16 or \
                not out.is_contiguous() or out.device != dev:
            raise RuntimeError("out must be a contiguous [L, out_features] bf16 tensor on the "
                               "device of the rows")
        try:
            _lib.call("brt_grouped_expert_gemm", x.data_ptr(), w.data_ptr(), out.data_ptr(),
                      counts.data_ptr(), E, L, mpl, n_in, n_out, int(bool(relu)),
                      _error_word(dev).data_ptr(), _lib.raw_stream(dev))
        except _lib.BrtError as exc:
            if exc.status == 4:  # BRT_ERR_UNSUPPORTED: feature counts the tiles do not divide
                raise NotImplementedError(str(exc)) from None
            raise
    return out


def check_status(device=None) -> None:
    """Synchronise and raise if a bounded wait inside an expert GEMM ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    word = _error_words.get(dev.index)
    if word is not None and int(word.item()) != 0:
        word.zero_()
        raise _lib.BrtError("an expert GEMM gave up a bounded wait; its output is incomplete", 7)
