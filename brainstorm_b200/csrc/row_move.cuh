// Device-side building blocks of the row-moving kernels (dispatch, combine and the dispatch
// that lands its rows straight in the peers' arenas): index-row scans, route tables, 16-byte
// chunk arithmetic, item cursors and the dense-column bookkeeping.
#pragma once

#include "common.cuh"

namespace brt_b200 {
namespace rows {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxPaths = 4096;
constexpr int kPieceVecs = 128;    // vectors per dispatch item (2 KB at 16 bytes)
constexpr int kCopyUnroll = kPieceVecs / 32;
constexpr int kMaxRoutes = 2;      // routes per combine item staged in shared memory (the
                                   // fold below is written out for exactly two)
constexpr int kFoldVecs = 128;     // vectors per combine item (2 KB at 16 bytes)
constexpr int kFoldUnroll = kFoldVecs / 32;
constexpr int kStages = 2;

struct RouteSlot {
  int row;     // output row (dispatch) / input row (combine)
  float gate;  // gate as fp32; for 2-D dispatch the path id, bit-cast
};

// The index row of one cell is scanned IV paths per lane: one coalesced 16-byte load per
// lane covers 128 paths when the row is 16-byte aligned (IV = 4), otherwise one path per
// lane (IV = 1).
template <int IV>
__device__ __forceinline__ void load_index_chunk(const int* __restrict__ indices, int64_t cell,
                                                 int path_num, int chunk, int lane,
                                                 int (&v)[IV]) {
  const int e0 = (chunk * 32 + lane) * IV;
  if constexpr (IV == 4) {
    if (e0 < path_num) {
      const int4 q = *reinterpret_cast<const int4*>(indices + cell * path_num + e0);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
      v[0] = v[1] = v[2] = v[3] = 0;
    }
  } else {
    v[0] = e0 < path_num ? indices[cell * path_num + e0] : 0;
  }
}

// Gate rows travel with the index rows.  GK: 0 = no gates, 1 = fp32, 2 = stored as DT.
template <int IV, int GK, int DT>
__device__ __forceinline__ void load_gate_chunk(const void* __restrict__ gates, int64_t cell,
                                                int path_num, int chunk, int lane,
                                                float (&g)[IV]) {
#pragma unroll
  for (int j = 0; j < IV; j++) g[j] = 1.f;
  if constexpr (GK == 0) return;
  const int e0 = (chunk * 32 + lane) * IV;
  if (e0 >= path_num) return;
  if constexpr (GK == 1) {
    const float* p = static_cast<const float*>(gates) + cell * path_num + e0;
    if constexpr (IV == 4) {
      const float4 q = *reinterpret_cast<const float4*>(p);
      g[0] = q.x; g[1] = q.y; g[2] = q.z; g[3] = q.w;
    } else {
      g[0] = *p;
    }
  } else {
    using E = typename Elem<DT>::type;
    const E* p = static_cast<const E*>(gates) + cell * path_num + e0;
    if constexpr (IV == 4 && sizeof(E) == 2) {
      alignas(8) E e[4];
      *reinterpret_cast<uint2*>(e) = *reinterpret_cast<const uint2*>(p);
#pragma unroll
      for (int j = 0; j < 4; j++) g[j] = Elem<DT>::to_f32(e[j]);
    } else {
#pragma unroll
      for (int j = 0; j < IV; j++) g[j] = Elem<DT>::to_f32(p[j]);
    }
  }
}

// s_loads[e], s_base[e] for every path; called by all threads of the CTA.
__device__ __forceinline__ void setup_paths(const int* __restrict__ loads, int path_num,
                                            int max_path_load, int* s_loads, int* s_base) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int p = 0; p < path_num; p += 32) {
      const int e = p + lane;
      const int v = e < path_num ? loads[e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (e < path_num) {
        s_loads[e] = v;
        s_base[e] = max_path_load != 0 ? e * max_path_load : carry + incl - v;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
}

// Dense seat columns (what the index kernels write): column e holds every seat
// 1 .. counts[e] exactly once, so the rows of path e that receive a cell are exactly the first
// min(counts[e], loads[e]) of its slot and the rest of the slot is known to stay empty
// without looking at the indices.  s_written[e] = rows of path e that get a cell,
// s_fill[e] = exclusive prefix of the empty rows per path (s_fill[path_num] = their total).
// Called by all threads of the CTA after setup_paths.
__device__ __forceinline__ void setup_fill(const int* __restrict__ counts, int path_num,
                                           int max_path_load, const int* s_loads,
                                           int* s_written, int* s_fill) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int p = 0; p < path_num; p += 32) {
      const int e = p + lane;
      int written = 0, empty = 0;
      if (e < path_num) {
        const int load = s_loads[e] > 0 ? s_loads[e] : 0;
        const int have = counts[e] > 0 ? counts[e] : 0;
        written = have < load ? have : load;
        const int slot = max_path_load != 0 ? max_path_load : load;
        empty = slot > written ? slot - written : 0;
      }
      int incl = empty;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (e < path_num) {
        s_written[e] = written;
        s_fill[e] = carry + incl - empty;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_fill[path_num] = carry;
  }
  __syncthreads();
}

template <int VB, int DT>
struct Lanes {
  using V = typename Chunk<VB>::type;
  using E = typename Elem<DT>::type;
  static constexpr int N = VB / (int)sizeof(E);
};

// 16-byte chunk <-> fp32 lanes.  16-bit types convert two at a time (the scalar
// float -> bf16/half conversions run at a quarter of the packed rate).
template <int VB, int DT>
__device__ __forceinline__ void unpack_chunk(const typename Chunk<VB>::type& row,
                                             float (&f)[Lanes<VB, DT>::N]) {
  using L = Lanes<VB, DT>;
  if constexpr (VB == 16 && DT == BRT_BF16) {
    const uint32_t w[4] = {row.x, row.y, row.z, row.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else if constexpr (VB == 16 && DT == BRT_F16) {
    const uint32_t w[4] = {row.x, row.y, row.z, row.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  } else {
    alignas(VB) typename L::E el[L::N];
    *reinterpret_cast<typename L::V*>(el) = row;
#pragma unroll
    for (int i = 0; i < L::N; i++) f[i] = Elem<DT>::to_f32(el[i]);
  }
}

template <int VB, int DT>
__device__ __forceinline__ typename Chunk<VB>::type pack_chunk(
    const float (&f)[Lanes<VB, DT>::N]) {
  using L = Lanes<VB, DT>;
  if constexpr (VB == 16 && DT == BRT_BF16) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  } else if constexpr (VB == 16 && DT == BRT_F16) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    alignas(VB) typename L::E el[L::N];
#pragma unroll
    for (int i = 0; i < L::N; i++) el[i] = Elem<DT>::from_f32(f[i]);
    return *reinterpret_cast<typename L::V*>(el);
  }
}

// x * g element-wise in the storage type: exact product in fp32, one rounding.
template <int VB, int DT>
__device__ __forceinline__ typename Chunk<VB>::type scale_chunk(typename Chunk<VB>::type x,
                                                                float g) {
  float f[Lanes<VB, DT>::N];
  unpack_chunk<VB, DT>(x, f);
#pragma unroll
  for (int i = 0; i < Lanes<VB, DT>::N; i++) f[i] = __fmul_rn(f[i], g);
  return pack_chunk<VB, DT>(f);
}

struct MoveArgs {
  const void* src;
  void* dst;
  const void* gates;
  const int* indices;
  const int* loads;
  const int* old_tags;       // dispatch only
  int* new_tags;             // dispatch only
  unsigned char* row_marks;  // dispatch only (general index tensors)
  const int* dense_counts;   // dispatch only: seat columns are dense, see setup_fill
  int keep_rows_cached;      // dispatch: write rows with the default cache policy (the next
                             // op reads them) instead of evict-first
  int loads_evict_first;     // dispatch: source rows leave L2 first (they are read once)
  int newest_first;          // combine: visit the cells from the last to the first, so that
                             // the rows written most recently are read while still in L2
  int64_t cell_num;
  int64_t row_vecs;  // vectors per row
  int64_t pieces_per_row;
  int path_num;
  int max_path_load;
  int64_t total_rows;  // dispatch: output rows
  int is_residual;     // combine only
};

// Position of a warp in the (cell, piece) item space.  Items are visited with a fixed
// stride, so the position advances by a precomputed (cells, pieces) step with one carry
// instead of a 64-bit division per item.
struct ItemCursor {
  int64_t cell;
  int piece;
};
struct ItemStep {
  int64_t cells;
  int pieces;
  int pieces_per_row;
};
__device__ __forceinline__ ItemCursor cursor_at(int64_t item, int64_t pieces_per_row) {
  ItemCursor c;
  c.cell = item / pieces_per_row;
  c.piece = (int)(item - c.cell * pieces_per_row);
  return c;
}
__device__ __forceinline__ ItemStep step_of(int64_t stride, int64_t pieces_per_row) {
  ItemStep s;
  s.cells = stride / pieces_per_row;
  s.pieces = (int)(stride - s.cells * pieces_per_row);
  s.pieces_per_row = (int)pieces_per_row;
  return s;
}
__device__ __forceinline__ ItemCursor advance(ItemCursor c, const ItemStep& s) {
  c.cell += s.cells;
  c.piece += s.pieces;
  if (c.piece >= s.pieces_per_row) {
    c.piece -= s.pieces_per_row;
    c.cell += 1;
  }
  return c;
}

// Scan the index row of `cell` (first chunk already in seat/gate registers) and write its
// kept routes to slots[0..kMaxRoutes) in ascending path order; returns their total count.
// kStorePath: keep the path id in the slot's gate field (2-D dispatch needs it).
template <int IV, int GK, int DT, bool kStorePath>
__device__ __forceinline__ int build_routes(const MoveArgs& a, int64_t cell,
                                            const int (&first_seat)[IV],
                                            const float (&first_gate)[IV], const int* s_loads,
                                            const int* s_base, RouteSlot* slots, int lane,
                                            int max_slots = kMaxRoutes) {
  const int E = a.path_num;
  const int chunks = (E + 32 * IV - 1) / (32 * IV);
  int count = 0;
  for (int c = 0; c < chunks; c++) {
    int seat[IV];
    float gate[IV];
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < IV; j++) { seat[j] = first_seat[j]; gate[j] = first_gate[j]; }
    } else {
      load_index_chunk<IV>(a.indices, cell, E, c, lane, seat);
      load_gate_chunk<IV, GK, DT>(a.gates, cell, E, c, lane, gate);
    }
    unsigned mine = 0;
#pragma unroll
    for (int j = 0; j < IV; j++) {
      const int e = (c * 32 + lane) * IV + j;
      const bool keep = e < E && seat[j] > 0 && seat[j] <= s_loads[e];
      mine |= (keep ? 1u : 0u) << j;
    }
    unsigned any = __ballot_sync(0xffffffffu, mine != 0);
    while (any) {  // lanes, then paths within a lane: ascending path order
      const int l = __ffs(any) - 1;
      any &= any - 1;
      const unsigned theirs = __shfl_sync(0xffffffffu, mine, l);
#pragma unroll
      for (int j = 0; j < IV; j++) {
        if ((theirs >> j) & 1u) {  // warp-uniform
          const int e = (c * 32 + l) * IV + j;
          const int seat_b = __shfl_sync(0xffffffffu, seat[j], l);
          const float g = __shfl_sync(0xffffffffu, gate[j], l);
          if (count < max_slots && lane == 0) {
            slots[count].row = s_base[e] + seat_b - 1;
            slots[count].gate = kStorePath ? __int_as_float(e) : g;
          }
          count++;
        }
      }
    }
  }
  return count;
}

// Zero one (empty row, 2 KB piece) of a dense dispatch; `item` counts the pieces of the empty
// rows in path order.  Called by a whole warp.
template <int VB>
__device__ __forceinline__ void fill_item(const MoveArgs& a, const int* s_base,
                                          const int* s_written, const int* s_fill, int64_t item,
                                          int lane) {
  using V = typename Chunk<VB>::type;
  const int64_t nth = item / a.pieces_per_row;
  const int piece = (int)(item - nth * a.pieces_per_row);
  int lo = 0, hi = a.path_num - 1;  // last path whose first empty row is <= nth
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((int64_t)s_fill[mid] <= nth) lo = mid; else hi = mid - 1;
  }
  const int64_t row = (int64_t)s_base[lo] + s_written[lo] + (nth - s_fill[lo]);
  V* dp = static_cast<V*>(a.dst) + row * a.row_vecs;
  const V zero = zero_chunk<V>();
  const int64_t v0 = (int64_t)piece * kPieceVecs + lane;
#pragma unroll
  for (int u = 0; u < kCopyUnroll; u++) {
    const int64_t v = v0 + u * 32;
    if (v < a.row_vecs) store_stream(dp + v, zero);
  }
  if (piece == 0 && lane == 0 && a.new_tags != nullptr) a.new_tags[row] = 0;
}

// A warp's share of the empty-row pieces, spread evenly between its move items so that the
// writes of zeros mix with the row traffic instead of trailing it.
struct FillPacer {
  int64_t next, end, stride;  // items next, next + stride, ... < end
  int64_t moves, fills, acc;
  __device__ __forceinline__ FillPacer(int64_t move_items, int64_t fill_items, int64_t warp,
                                       int64_t warps) {
    next = warp;
    end = fill_items;
    stride = warps;
    moves = move_items > warp ? (move_items - warp + warps - 1) / warps : 0;
    fills = fill_items > warp ? (fill_items - warp + warps - 1) / warps : 0;
    acc = 0;
  }
  // how many fill items are due after one more move item
  __device__ __forceinline__ int due() {
    acc += fills;
    int n = 0;
    while (acc >= moves && moves > 0) { acc -= moves; n++; }
    return n;
  }
};

// ------------------------------------------------------------------------------ combine parts
// (The packed fp32 instructions of sm_100, mul.rn.f32x2 / add.rn.f32x2, were tried here: the
// results differed from the scalar sequence in the last bit and the kernel ran slower, so the
// fold stays scalar.)
template <int VB, int DT, int GMODE>
__device__ __forceinline__ void fold_chunk(float (&acc)[Lanes<VB, DT>::N],
                                           const typename Chunk<VB>::type& row, float g) {
  using L = Lanes<VB, DT>;
  float x[L::N];
  unpack_chunk<VB, DT>(row, x);
#pragma unroll
  for (int i = 0; i < L::N; i++) {
    if constexpr (GMODE != 0) x[i] = __fmul_rn(x[i], g);
    acc[i] = __fadd_rn(acc[i], x[i]);
  }
}

template <int DT, int GMODE>
__device__ __forceinline__ float gate_at(const void* gates, int64_t at) {
  if constexpr (GMODE == 1) return static_cast<const float*>(gates)[at];
  if constexpr (GMODE == 2)
    return Elem<DT>::to_f32(static_cast<const typename Elem<DT>::type*>(gates)[at]);
  return 1.f;
}

// Per-warp staging area: kStages x (route table + kMaxRoutes row pieces of 2 KB).
struct alignas(16) FoldStage {
  uint4 rows[kMaxRoutes][kFoldVecs];
  RouteSlot route[kMaxRoutes];
  int count;
  int pad[3];
};

constexpr int kCopyRoutes = 4;  // destinations per dispatch item kept in the route table

// Per-warp staging area of the pipelined dispatch: one 2 KB source piece and its routes.
struct alignas(16) CopyStage {
  uint4 row[kPieceVecs];
  RouteSlot route[kCopyRoutes];
  int count;
  int pad[3];
};

}  // namespace rows
}  // namespace brt_b200
