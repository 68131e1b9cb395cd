"""CPU checker for the routing hot path.  TEST INFRASTRUCTURE ONLY.

numpy-level restatement of the reference's operator semantics (shape logic of the
torch binding + the C row loops in ``brt_oracle.c``).  Only ``tests/``, the smoke
test and the benchmark's CPU-baseline leg may import this package; the shipped
package never does.

Parity status: pinned against the reference's saved notebook outputs and sample
scripts (``tests/test_oracle_golden.py``) and, on a GPU box, against the
reference's own kernels built by ``oracle/build.py --ref``.

Arrays are numpy; 16-bit floating point travels as ``uint16`` bit patterns with
an explicit ``dtype`` argument ("f32", "f16", "bf16").
"""
import ctypes
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import build as _build

_DT = {"f32": 0, "f16": 1, "bf16": 2}
_ES = {"f32": 4, "f16": 2, "bf16": 2}
_NP = {"f32": np.float32, "f16": np.uint16, "bf16": np.uint16}

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        _lib = ctypes.CDLL(str(path))
        _lib.brt_oracle_generate_indices_and_loads.restype = ctypes.c_int
        _lib.brt_oracle_max_threads.restype = ctypes.c_int
    return _lib


def max_threads() -> int:
    return int(lib().brt_oracle_max_threads())


def set_threads(n: int) -> None:
    lib().brt_oracle_set_threads(ctypes.c_int(n))


def _p(a: Optional[np.ndarray]):
    if a is None:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.int32)


# --------------------------------------------------------------------------- 16-bit helpers


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_bits(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 array -> storage array of ``dtype``."""
    if dtype == "f32":
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "f16":
        return np.ascontiguousarray(x.astype(np.float16)).view(np.uint16)
    return f32_to_bf16_bits(x)


def from_bits(b: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f32":
        return b
    if dtype == "f16":
        return b.view(np.float16).astype(np.float32)
    return bf16_bits_to_f32(b)


# --------------------------------------------------------------------------- protocols


def topk_hot_mask(score: np.ndarray, top_k: int) -> np.ndarray:
    """python/brt/router/protocol/topk.py:26-31 — ones at the k largest scores of each row.
    Ties are not pinned by the reference's tests; inputs used for parity have none."""
    T, E = score.shape
    order = np.argsort(-score, axis=1, kind="stable")[:, :top_k]
    mask = np.zeros((T, E), dtype=np.int32)
    np.put_along_axis(mask, order, 1, axis=1)
    return mask


def threshold_hot_mask(score: np.ndarray, threshold: float, residual_path: int = -1) -> np.ndarray:
    """python/brt/router/protocol/threshold.py:23-39."""
    mask = (score > threshold).astype(np.int32)
    if residual_path >= 0:
        empty = (mask.sum(axis=1) == 0).astype(np.int32)
        mask[:, residual_path] += empty
    return mask


def softmax(logits: np.ndarray) -> np.ndarray:
    z = logits.astype(np.float32)
    z = z - z.max(axis=1, keepdims=True)
    e = np.exp(z)
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def renormalised_topk_score(score: np.ndarray, top_k: int) -> np.ndarray:
    """python/brt/router/protocol/swin_moe.py:193-204 — the top-k scores of each row divided
    by their sum (clamped at float32 eps, summed in pick order), zeros elsewhere."""
    T, E = score.shape
    order = np.argsort(-score, axis=1, kind="stable")[:, :top_k]
    vals = np.take_along_axis(score, order, axis=1).astype(np.float32)
    denom = np.zeros((T,), dtype=np.float32)
    for j in range(vals.shape[1]):
        denom = (denom + vals[:, j]).astype(np.float32)
    denom = np.maximum(denom, np.finfo(np.float32).eps)
    out = np.zeros((T, E), dtype=np.float32)
    np.put_along_axis(out, order, (vals / denom[:, None]).astype(np.float32), axis=1)
    return out


def route_scores(score: np.ndarray, decision: str = "topk", top_k: int = 1,
                 threshold: float = 0.0, residual_path: int = -1, output: str = "mask",
                 supported_capacities=None, capacity_padding: bool = False,
                 path_wise_padding: bool = False, prefix=None, throttle_capacity=None):
    """A protocol of python/brt/router/protocol/ (topk.py:26-31, threshold.py:23-39) followed
    by nothing ("mask": mask and cells per path), by throttle_hotmask ("throttled_mask") or
    by generate_indices_and_loads ("seat_indices"), composed from the functions of this file."""
    if decision == "topk":
        mask = topk_hot_mask(score, top_k)
    else:
        mask = threshold_hot_mask(score, threshold, residual_path)
    if output == "mask":
        return mask, mask.sum(axis=0).astype(np.int32)
    if output == "throttled_mask":
        return throttle_hotmask(mask, prefix, throttle_capacity)
    return generate_indices_and_loads(mask, supported_capacities, capacity_padding,
                                      path_wise_padding, False)


# --------------------------------------------------------------------------- index generation


def generate_indices_and_loads(
    hot_mask: np.ndarray,
    supported_capacities: Optional[Sequence[int]] = None,
    capacity_padding: bool = False,
    path_wise_padding: bool = False,
    is_tag_index: bool = False,
) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/torch/router.cc:48-80 over src/router/location.cu:212-257,335-379."""
    mask = _i32(hot_mask)
    T, E = mask.shape
    indices = np.zeros((T, E), dtype=np.int32)
    loads = np.zeros((E,), dtype=np.int32)
    if mask.size == 0:
        return indices, loads
    caps = None if supported_capacities is None else _i32(supported_capacities)
    rc = lib().brt_oracle_generate_indices_and_loads(
        _p(mask), _p(indices), _p(loads), ctypes.c_int64(T), ctypes.c_int(E), _p(caps),
        ctypes.c_int(0 if caps is None else caps.shape[0]), ctypes.c_int(bool(capacity_padding)),
        ctypes.c_int(bool(path_wise_padding)), ctypes.c_int(bool(is_tag_index)))
    if rc != 0:
        raise RuntimeError("capacity_padding needs at least one supported capacity")
    return indices, loads


def generate_indices_and_loads_numpy(hot_mask, supported_capacities=None, capacity_padding=False,
                                     path_wise_padding=False, is_tag_index=False):
    """Second, independent restatement in the style of the reference's own torch oracle
    (test/python/fabric_test.py:35-92): cumsum*mask, column sums, capacity mapping loop.
    Used to cross-check the C loops.  Unlike that test oracle (which skips empty paths
    before looking at path_wise_padding), loads follow the kernel."""
    mask = _i32(hot_mask)
    T, E = mask.shape
    csum = np.cumsum(mask, axis=0, dtype=np.int32)
    real = mask.sum(axis=0, dtype=np.int32)
    if not is_tag_index:
        indices = (csum * mask).astype(np.int32)
    else:
        indices = np.zeros_like(mask)
        for e in range(E):
            cells = np.nonzero(mask[:, e])[0]
            indices[: cells.size, e] = cells + 1
    loads = real.copy()
    caps = None if supported_capacities is None else list(np.asarray(supported_capacities))
    for e in range(E):
        if capacity_padding and path_wise_padding:
            loads[e] = caps[e]
            continue
        if real[e] == 0:
            loads[e] = 0
            continue
        if caps is None or len(caps) == 0:
            continue
        fit = [c for c in caps if real[e] <= c]
        if fit:
            loads[e] = fit[0] if capacity_padding else real[e]
        else:
            loads[e] = caps[-1]
    return indices, loads


def throttle_hotmask(hot_mask, prefix, threshold) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/torch/router.cc:15-31 over src/router/location.cu:59-130.
    Returns (throttled mask, updated prefix); ``prefix`` itself is updated in place when it
    is an int32 numpy array, as the reference mutates its argument."""
    mask = _i32(hot_mask)
    T, E = mask.shape
    pre = prefix if isinstance(prefix, np.ndarray) and prefix.dtype == np.int32 else _i32(prefix)
    thr = _i32(threshold)
    assert pre.shape[0] == E and thr.shape[0] == E
    out = np.zeros_like(mask)
    lib().brt_oracle_throttle_hotmask(_p(mask), _p(out), _p(pre), _p(thr), ctypes.c_int64(T),
                                      ctypes.c_int(E))
    return out, pre


def convert_index_format(origin_indices, loads, is_to_tag: bool) -> np.ndarray:
    """src/backend/torch/router.cc:90-110.  The binding forwards ``is_to_tag`` into the
    launcher's ``tag_to_seat`` slot (src/router/location.cu:317-333), so ``True`` runs the
    tag->seat kernel."""
    origin = _i32(origin_indices)
    T, E = origin.shape
    out = np.zeros_like(origin)
    lib().brt_oracle_convert_index_format(_p(origin), _p(out), _p(_i32(loads)), ctypes.c_int64(T),
                                          ctypes.c_int(E), ctypes.c_int(bool(is_to_tag)))
    return out


# --------------------------------------------------------------------------- dispatch / combine


def _cell_size(arr: np.ndarray, rows: int) -> int:
    return int(arr.size // rows) if rows else 0


def dispatch_with_indices_and_loads(
    in_data: np.ndarray,
    route_indices: np.ndarray,
    loads: np.ndarray,
    gates: Optional[np.ndarray] = None,
    tag_generating: bool = False,
    tags: Optional[np.ndarray] = None,
    max_path_padding: bool = False,
    max_path_load: int = 0,
    is_1d_routing: bool = True,
    is_tag_index: bool = False,
    dtype: str = "f32",
) -> List[np.ndarray]:
    """src/backend/torch/router.cc:131-273 over src/router/route.cu:13-206,284-465."""
    indices = _i32(route_indices)
    loads = _i32(loads)
    T = in_data.shape[0]
    E = indices.shape[1]
    if T == 0:
        shape = list(in_data.shape)
        if is_1d_routing:
            shape[0] = 0
        else:
            if len(shape) == 2:
                shape.append(1)
            shape[1] = 0
            shape = shape[1:]
        out = [np.zeros(shape, dtype=in_data.dtype)]
        if tag_generating:
            out.append(np.zeros((0,), dtype=np.int32))
        return out
    cell_size = _cell_size(in_data, T)
    if not is_1d_routing:
        cell_size //= E
    if max_path_padding:
        mpl = int(max_path_load) if max_path_load > 0 else int(loads.max())
        total = mpl * E
    else:
        mpl = 0
        total = int(loads.sum())
    shape = list(in_data.shape)
    if is_1d_routing:
        shape[0] = total
    else:
        if len(shape) == 2:
            shape.append(1)
        shape[1] = total
        shape = shape[1:]
    out = np.zeros(shape, dtype=in_data.dtype)
    if gates is not None:
        assert is_1d_routing
        gates = np.ascontiguousarray(gates)
    old_tags = new_tags = None
    if tag_generating:
        old_tags = np.arange(1, T + 1, dtype=np.int32) if tags is None else _i32(tags)
        new_tags = np.zeros((total,), dtype=np.int32)
    fn = lib().brt_oracle_dispatch_tag if is_tag_index else lib().brt_oracle_dispatch_seat
    src = np.ascontiguousarray(in_data)
    fn(_p(src), _p(out), _p(gates), _p(indices), _p(loads), _p(old_tags), _p(new_tags),
       ctypes.c_int64(T), ctypes.c_int64(cell_size), ctypes.c_int(E), ctypes.c_int32(mpl),
       ctypes.c_int(bool(is_1d_routing)), ctypes.c_int(_DT[dtype]))
    return [out, new_tags] if tag_generating else [out]


def split_fused_cells_to_paths(in_data, loads, max_path_padding=False, is_load_split=False,
                               is_tag_split=False, tags=None):
    """src/backend/torch/router.cc:285-335."""
    loads = _i32(loads)
    E = loads.size
    if is_tag_split:
        is_load_split = True
        assert tags is not None
    datas, loads_l, tags_l = [], [], []
    start = 0
    for e in range(E):
        n = in_data.shape[0] // E if max_path_padding else int(loads[e])
        s = e * n if max_path_padding else start
        datas.append(in_data[s:s + n])
        if is_load_split:
            loads_l.append(loads[e:e + 1])
        if is_tag_split:
            tags_l.append(tags[s:s + n])
        start += n
    if is_tag_split:
        return [datas, loads_l, tags_l]
    if is_load_split:
        return [datas, loads_l]
    return [datas]


def fuse_split_cells_from_paths(in_data, is_load_fuse=False, is_tag_fuse=False, loads=None,
                                tags=None):
    """src/backend/torch/router.cc:348-369."""
    out = np.concatenate(in_data, axis=0)
    if is_load_fuse:
        return [out, np.concatenate(loads, axis=0)]
    if is_tag_fuse:
        all_tags = np.concatenate(tags, axis=0)
        uniq, inverse = np.unique(all_tags, return_inverse=True)
        return [out, uniq.astype(all_tags.dtype), inverse.astype(np.int64)]
    return [out]


def combine_with_indices_and_loads(
    in_data: np.ndarray,
    route_indices: np.ndarray,
    loads: Optional[np.ndarray] = None,
    gates: Optional[np.ndarray] = None,
    out_data: Optional[np.ndarray] = None,
    max_path_padding: bool = False,
    ever_padded: bool = True,
    is_tag_index: bool = False,
    tags: Optional[np.ndarray] = None,
    dtype: str = "f32",
    gates_dtype: str = "f32",
) -> List[np.ndarray]:
    """src/backend/torch/router.cc:372-473 over src/router/route.cu:208-282,467-522.
    With ``out_data`` the array is mutated and returned (residual semantics)."""
    T = route_indices.shape[0]
    if T == 0:
        if not is_tag_index:
            return [out_data if out_data is not None else np.empty_like(in_data)]
        return [np.empty_like(in_data), np.empty_like(tags), np.zeros_like(tags)]
    if T == 1:
        if not is_tag_index:
            if out_data is not None:
                s = from_bits(out_data, dtype) + from_bits(in_data, dtype)
                return [to_bits(s, dtype).reshape(out_data.shape)]
            return [in_data]
        return [in_data, tags, np.ones_like(tags)]
    if not is_tag_index:
        indices = _i32(route_indices)
        E = indices.shape[1]
        loads = _i32(loads)
        cell_size = _cell_size(in_data, in_data.shape[0])
        mpl = in_data.shape[0] // E if max_path_padding else 0
        src = np.ascontiguousarray(in_data)
        if out_data is not None:
            out, residual = out_data, True
            assert out.flags["C_CONTIGUOUS"]
        else:
            out = np.zeros((T,) + tuple(in_data.shape[1:]), dtype=in_data.dtype)
            residual = False
        g = None if gates is None else np.ascontiguousarray(gates)
        lib().brt_oracle_combine_seat(
            _p(src), _p(out), _p(g), _p(indices), _p(loads), ctypes.c_int64(T),
            ctypes.c_int64(cell_size), ctypes.c_int(E), ctypes.c_int32(mpl),
            ctypes.c_int(residual), ctypes.c_int(_DT[dtype]), ctypes.c_int(_DT[gates_dtype]))
        return [out]
    # tag branch: per-unique-tag sum of rows, src/backend/torch/router.cc:449-472.
    inverse = np.asarray(route_indices).reshape(-1)
    n = tags.shape[0]
    vals = from_bits(in_data, dtype).reshape(in_data.shape[0], -1)
    if out_data is not None:
        # the functional scatter_reduce result is discarded: out_data returned unchanged
        out = out_data
        tags_v = tags
    else:
        acc = np.zeros((n, vals.shape[1]), dtype=np.float32)
        for i in range(vals.shape[0]):  # ascending row order
            acc[inverse[i]] = acc[inverse[i]] + vals[i]
        tags_v = tags
        if ever_padded and int(tags[0]) == 0:
            acc = acc[1:]
            tags_v = tags[1:]
        out = to_bits(acc, dtype).reshape((acc.shape[0],) + tuple(in_data.shape[1:]))
    return [out, tags_v, np.array([tags_v.size], dtype=np.int32)]


# --------------------------------------------------------------------------- distributed


def locality_reorder(loads: np.ndarray, world_size: int) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/torch/distributed.cc:43-55 over src/distributed/local_reorder.cu:15-63."""
    l = _i32(loads).reshape(-1)
    out = np.zeros_like(l)
    idx = np.zeros((world_size,), dtype=np.int32)
    lib().brt_oracle_locality_reorder(_p(l), ctypes.c_int(world_size), _p(idx), _p(out))
    return out.reshape(np.asarray(loads).shape), idx


def group_locality_reorder(loads: np.ndarray, world_size: int, group_size: int = 1):
    """src/backend/torch/distributed.cc:57-69 over src/distributed/local_reorder.cu:65-141."""
    l = _i32(loads).reshape(-1)
    out = np.zeros_like(l)
    idx = np.zeros((world_size,), dtype=np.int32)
    lib().brt_oracle_group_locality_reorder(_p(l), ctypes.c_int(group_size),
                                            ctypes.c_int(world_size), _p(idx), _p(out))
    return out.reshape(np.asarray(loads).shape), idx


def sim_group_sparse_all_to_all(in_datas: List[np.ndarray], send_sizes: List[np.ndarray],
                                max_path_padding: bool = False, max_path_load: int = 0):
    """All W ranks of ``group_sparse_all_to_all`` at once
    (src/backend/torch/distributed.cc:755-841, src/distributed/collective.cc:142-182).
    Rank r sends bucket (i, j) — rows for rank i's local expert j, packed in that order —
    and receives into segments ordered [local expert j][source rank i].
    Returns per rank (out_data, recv_sizes laid out [G, W], send_sizes)."""
    W = len(in_datas)
    G = send_sizes[0].size // W
    send = [_i32(s).reshape(W, G) for s in send_sizes]
    results = []
    for me in range(W):
        recv = np.stack([send[i][me] for i in range(W)], axis=0)  # [W(src), G]
        recv_gw = np.ascontiguousarray(recv.T)  # [G, W]
        if max_path_padding:
            mpl = int(max_path_load) if max_path_load else int(recv_gw.max())
            n = mpl * W * G
        else:
            mpl = 0
            n = int(recv_gw.sum())
        out = np.zeros((n,) + tuple(in_datas[me].shape[1:]), dtype=in_datas[me].dtype)
        cur = 0
        for j in range(G):
            for i in range(W):
                cnt = int(send[i][me, j])
                # where bucket (me, j) starts in rank i's packed send buffer
                if max_path_padding:
                    off = (me * G + j) * mpl
                else:
                    off = int(send[i].reshape(-1)[: me * G + j].sum())
                out[cur:cur + cnt] = in_datas[i][off:off + cnt]
                cur += mpl if max_path_padding else cnt
        results.append((out, recv_gw.reshape(-1).copy(), send[me].reshape(-1).copy()))
    return results


def sim_size_known_group_sparse_all_to_all(in_datas, send_sizes, recv_sizes,
                                           max_path_padding: bool = False):
    """All W ranks of ``size_known_group_sparse_all_to_all``
    (src/backend/torch/distributed.cc:843-898, src/distributed/collective.cc:184-224):
    the inverse walk.  ``send_sizes[r]`` is laid out [G, W] (what rank r got in the forward
    pass), ``recv_sizes[r]`` is laid out [W, G] (what rank r sent in the forward pass)."""
    W = len(in_datas)
    G = send_sizes[0].size // W
    send = [_i32(s).reshape(G, W) for s in send_sizes]
    recv = [_i32(s).reshape(W, G) for s in recv_sizes]
    outs = []
    for me in range(W):
        if max_path_padding:
            n = in_datas[me].shape[0]
            mpl = n // (W * G)
        else:
            n = int(recv[me].sum())
            mpl = 0
        out = np.zeros((n,) + tuple(in_datas[me].shape[1:]), dtype=in_datas[me].dtype)
        cur = 0
        for i in range(W):
            for j in range(G):
                cnt = int(recv[me][i, j])
                # bucket (j, me) in rank i's [G, W]-ordered buffer
                if max_path_padding:
                    off = (j * W + me) * mpl
                else:
                    off = int(send[i].reshape(-1)[: j * W + me].sum())
                out[cur:cur + cnt] = in_datas[i][off:off + cnt]
                cur += mpl if max_path_padding else cnt
        outs.append(out)
    return outs


def sim_group_asymmetry_all_to_all(in_datas, send_sizes):
    """All W ranks of the padded-slot exchange (src/distributed/collective.cc:90-140):
    the buffer is W*G equal slots; slot (i, j) sends its first send[i, j] rows to rank i,
    and slot (i, j) of the output receives what rank i sent from its slot (me, j).
    Rows of an output slot beyond the received count are unspecified in the reference
    (``empty_like``); here they are zero.  Returns per rank (out, recv_sizes)."""
    W = len(in_datas)
    S = send_sizes[0].size
    G = S // W
    send = [_i32(s).reshape(W, G) for s in send_sizes]
    res = []
    for me in range(W):
        x = in_datas[me]
        slot = x.shape[0] // S
        out = np.zeros_like(x)
        recv = np.zeros((W, G), dtype=np.int32)
        for i in range(W):
            for j in range(G):
                cnt = int(send[i][me, j])
                recv[i, j] = cnt
                src0 = (me * G + j) * slot
                dst0 = (i * G + j) * slot
                out[dst0:dst0 + cnt] = in_datas[i][src0:src0 + cnt]
        res.append((out, recv.reshape(-1)))
    return res
