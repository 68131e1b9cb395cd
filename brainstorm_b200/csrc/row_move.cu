// Token dispatch and weighted combine for sm_100a.
//
// Both are pure data movement, so the design goal is HBM traffic equal to the algorithmic
// minimum and enough independent 16-byte accesses in flight to cover HBM latency.
//
//   dispatch : source-major.  One warp owns (cell, 2 KB piece of its row): it scans the
//              cell's index row with one coalesced 16-byte load per lane (128 paths per
//              load), keeps the piece in registers and stores it to every path that kept
//              the cell (times the gate when weighted), so a source row crosses HBM once
//              however many copies are made.  The index row of the warp's next item is
//              fetched before the current one is moved.  Rows of the output that no cell
//              lands on (capacity padding, dropped seats) are found through a byte map that
//              the move pass marks, and are written as zeros by a second launch: the output
//              is never memset as a whole and no row is written twice.
//   combine  : destination-major.  One warp owns (cell, 2 KB piece).  The rows of the
//              cell's kept routes are brought into shared memory with asynchronous 16-byte
//              copies (cp.async) - the copies of the warp's NEXT item are issued before
//              the current item is folded, so every warp keeps two items of row traffic in
//              flight without spending registers on it.  The fold walks the routes in
//              ascending path order with separate fp32 multiply and add roundings (the
//              order and rounding of the reference's atomicAdd sequence, without atomics)
//              and writes the row once.  Rows that are not 16-byte aligned take a simpler
//              register-only kernel.
//
// Per-path base rows (prefix sum of loads, or e * max_path_load) are computed once per CTA
// into shared memory.  Cells with more routes than the staging buffers hold (2) finish
// through a slower serial walk of the index row, so any number of routes is correct.
#include "row_move.cuh"

#include <cstdlib>
#include <cstring>
#include <initializer_list>

namespace brt_b200 {
namespace {

using namespace rows;


// ---------------------------------------------------------------------------------- dispatch
template <int VB, int DT, bool WEIGHTED, bool IS_1D, int IV>
__global__ void __launch_bounds__(kThreads, 4) dispatch_seat_kernel(const MoveArgs a) {
  using V = typename Chunk<VB>::type;
  constexpr int U = kCopyUnroll;
  constexpr int GK = WEIGHTED ? 2 : 0;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  int* s_written = s_base + a.path_num;
  int* s_fill = s_written + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);
  const bool dense = a.dense_counts != nullptr;
  if (dense) setup_fill(a.dense_counts, a.path_num, a.max_path_load, s_loads, s_written, s_fill);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;
  const int chunks = (E + 32 * IV - 1) / (32 * IV);
  FillPacer pace(items, dense ? (int64_t)s_fill[E] * a.pieces_per_row : 0, warp, warps);

  const ItemStep step = step_of(warps, a.pieces_per_row);
  ItemCursor at = cursor_at(warp < items ? warp : 0, a.pieces_per_row);
  if (warp >= items) at.cell = a.cell_num;
  ItemCursor ahead = advance(at, step);
  int cur[IV];
#pragma unroll
  for (int j = 0; j < IV; j++) cur[j] = 0;
  if (at.cell < a.cell_num) load_index_chunk<IV>(a.indices, at.cell, E, 0, lane, cur);
  while (at.cell < a.cell_num) {
    int nxt[IV];
#pragma unroll
    for (int j = 0; j < IV; j++) nxt[j] = 0;
    if (ahead.cell < a.cell_num) load_index_chunk<IV>(a.indices, ahead.cell, E, 0, lane, nxt);

    const int64_t cell = at.cell;
    const int piece = at.piece;
    const int64_t v0 = (int64_t)piece * kPieceVecs + lane;
    V regs[U];
    bool loaded = false;
    for (int c = 0; c < chunks; c++) {
      int seat[IV];
      if (c == 0) {
#pragma unroll
        for (int j = 0; j < IV; j++) seat[j] = cur[j];
      } else {
        load_index_chunk<IV>(a.indices, cell, E, c, lane, seat);
      }
      unsigned mine = 0;
#pragma unroll
      for (int j = 0; j < IV; j++) {
        const int e = (c * 32 + lane) * IV + j;
        const bool keep = e < E && seat[j] > 0 && seat[j] <= s_loads[e];
        mine |= (keep ? 1u : 0u) << j;
      }
      float gate[IV];
      if (mine != 0)
        load_gate_chunk<IV, GK, DT>(a.gates, cell, E, c, lane, gate);
      else {
#pragma unroll
        for (int j = 0; j < IV; j++) gate[j] = 1.f;
      }
      unsigned any = __ballot_sync(0xffffffffu, mine != 0);
      while (any) {
        const int l = __ffs(any) - 1;
        any &= any - 1;
        const unsigned theirs = __shfl_sync(0xffffffffu, mine, l);
#pragma unroll
        for (int j = 0; j < IV; j++) {
          if ((theirs >> j) & 1u) {  // warp-uniform
            const int e = (c * 32 + l) * IV + j;
            const int seat_b = __shfl_sync(0xffffffffu, seat[j], l);
            const int64_t row = (int64_t)s_base[e] + seat_b - 1;
            if (!IS_1D || !loaded) {
              const int64_t src_row = IS_1D ? cell : cell * E + e;
              const V* sp = src + src_row * a.row_vecs;
#pragma unroll
              for (int u = 0; u < U; u++) {
                const int64_t v = v0 + u * 32;
                if (v < a.row_vecs) regs[u] = load_stream(sp + v);
              }
              loaded = true;
            }
            V* dp = dst + row * a.row_vecs;
            if constexpr (WEIGHTED) {
              const float g = __shfl_sync(0xffffffffu, gate[j], l);
#pragma unroll
              for (int u = 0; u < U; u++) {
                const int64_t v = v0 + u * 32;
                if (v < a.row_vecs) store_stream(dp + v, scale_chunk<VB, DT>(regs[u], g));
              }
            } else {
#pragma unroll
              for (int u = 0; u < U; u++) {
                const int64_t v = v0 + u * 32;
                if (v < a.row_vecs) store_stream(dp + v, regs[u]);
              }
            }
            if (piece == 0 && lane == 0) {
              if (!dense) a.row_marks[row] = 1;
              if (a.new_tags != nullptr) a.new_tags[row] = a.old_tags[cell];
            }
          }
        }
      }
    }
    if (dense)
      for (int n = pace.due(); n > 0 && pace.next < pace.end; n--, pace.next += pace.stride)
        fill_item<VB>(a, s_base, s_written, s_fill, pace.next, lane);
#pragma unroll
    for (int j = 0; j < IV; j++) cur[j] = nxt[j];
    at = ahead;
    ahead = advance(ahead, step);
  }
  for (; pace.next < pace.end; pace.next += pace.stride)
    fill_item<VB>(a, s_base, s_written, s_fill, pace.next, lane);
}

// Writes zeros to every row (and tag) the move pass did not mark.  A warp owns the items
// (row, 2 KB piece) warp, warp + warps, ...; its lanes fetch the marks of the next 32 of
// them with one load, so a fully occupied output costs one mark latency per 32 items.
template <int VB>
__global__ void __launch_bounds__(kThreads) dispatch_zero_fill_kernel(const MoveArgs a) {
  using V = typename Chunk<VB>::type;
  constexpr int kUnroll = kCopyUnroll;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.total_rows * a.pieces_per_row;
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const V zero = zero_chunk<V>();
  const ItemStep step = step_of(warps, a.pieces_per_row);
  ItemCursor at = cursor_at(warp < items ? warp : 0, a.pieces_per_row);
  if (warp >= items) at.cell = a.total_rows;
  for (int64_t first = warp; first < items; first += 32 * warps) {
    // lane l looks at item first + l * warps
    const int64_t mine = first + (int64_t)lane * warps;
    const bool empty = mine < items && a.row_marks[mine / a.pieces_per_row] == 0;
    const unsigned todo = __ballot_sync(0xffffffffu, empty);
    if (todo == 0) {  // nothing to fill among these 32 items: skip them in one step
      const int64_t next = first + 32 * warps;
      if (next < items) at = cursor_at(next, a.pieces_per_row);
      continue;
    }
    for (int k = 0; k < 32 && at.cell < a.total_rows; k++, at = advance(at, step)) {
      if (!((todo >> k) & 1u)) continue;
      const int64_t row = at.cell;
      V* dp = dst + row * a.row_vecs;
      const int64_t v0 = (int64_t)at.piece * kPieceVecs + lane;
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) store_stream(dp + v, zero);
      }
      if (at.piece == 0 && lane == 0 && a.new_tags != nullptr) a.new_tags[row] = 0;
    }
  }
}

// Tag-index dispatch: output-major.  One warp owns (output row, piece); row i of path e
// pulls cell tag-1 when i < loads[e] and the tag is non-zero, otherwise it is zeroed.
template <int VB, int DT, bool WEIGHTED, bool IS_1D>
__global__ void __launch_bounds__(kThreads) dispatch_tag_kernel(const MoveArgs a) {
  using V = typename Chunk<VB>::type;
  constexpr int kUnroll = kCopyUnroll;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.total_rows * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;
  const V zero = zero_chunk<V>();

  for (int64_t item = warp; item < items; item += warps) {
    const int64_t row = item / a.pieces_per_row;
    const int64_t piece = item - row * a.pieces_per_row;
    // path of this row: last e with s_base[e] <= row (binary search; equal bases of empty
    // paths resolve to the last one, whose slot is the one that contains the row)
    int lo = 0, hi = E - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((int64_t)s_base[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int e = lo;
    const int64_t i = row - s_base[e];
    int tag = 0;
    if (i < s_loads[e] && i < a.cell_num) tag = a.indices[i * E + e];
    const int64_t cell = (int64_t)tag - 1;
    const bool pull = tag != 0 && cell >= 0 && cell < a.cell_num;
    V* dp = dst + row * a.row_vecs;
    const int64_t v0 = piece * kPieceVecs + lane;
    if (pull) {
      const int64_t src_row = IS_1D ? cell : cell * E + e;
      const V* sp = src + src_row * a.row_vecs;
      V regs[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) regs[u] = load_stream(sp + v);
      }
      float g = 1.f;
      if constexpr (WEIGHTED)
        g = Elem<DT>::to_f32(static_cast<const typename Elem<DT>::type*>(a.gates)[cell * E + e]);
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) {
          if constexpr (WEIGHTED)
            store_stream(dp + v, scale_chunk<VB, DT>(regs[u], g));
          else
            store_stream(dp + v, regs[u]);
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) store_stream(dp + v, zero);
      }
    }
    if (piece == 0 && lane == 0 && a.new_tags != nullptr)
      a.new_tags[row] = pull ? a.old_tags[cell] : 0;
  }
}

// ---------------------------------------------------------------------------------- combine
// GMODE: 0 = no gates, 1 = fp32 gates, 2 = gates stored in the data type.
// 16-byte rows only (VB == 16).
template <int DT, int GMODE, int IV>
__global__ void __launch_bounds__(kThreads, 3) combine_seat_async_kernel(const MoveArgs a) {
  constexpr int VB = 16;
  using L = Lanes<VB, DT>;
  using V = typename L::V;
  extern __shared__ __align__(16) unsigned char s_raw[];
  FoldStage* s_stage = reinterpret_cast<FoldStage*>(s_raw);  // [kWarps][kStages]
  int* s_loads = reinterpret_cast<int*>(s_raw + sizeof(FoldStage) * kWarps * kStages);
  int* s_base = s_loads + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + warp_in_cta;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;
  FoldStage* my = s_stage + warp_in_cta * kStages;

  int seat[IV];
  float gate[IV];
  // the cell an item position stands for (positions are walked upwards either way)
  auto cell_at = [&](int64_t pos) { return a.newest_first ? a.cell_num - 1 - pos : pos; };
  auto fetch = [&](const ItemCursor& c) {
#pragma unroll
    for (int j = 0; j < IV; j++) { seat[j] = 0; gate[j] = 1.f; }
    if (c.cell < a.cell_num) {
      load_index_chunk<IV>(a.indices, cell_at(c.cell), E, 0, lane, seat);
      load_gate_chunk<IV, GMODE, DT>(a.gates, cell_at(c.cell), E, 0, lane, gate);
    }
  };
  // Build the route table of an item from the registers fetched for it and start the
  // asynchronous copies of its rows; always closes exactly one copy group.
  auto issue = [&](FoldStage& st, const ItemCursor& c) {
    if (c.cell < a.cell_num) {
      const int count = build_routes<IV, GMODE, DT, false>(a, cell_at(c.cell), seat, gate,
                                                           s_loads, s_base, st.route, lane);
      if (lane == 0) st.count = count;
      __syncwarp();
      const int staged = count < kMaxRoutes ? count : kMaxRoutes;
      const int64_t first = (int64_t)c.piece * kFoldVecs;
      for (int r = 0; r < staged; r++) {
        const V* sp = src + (int64_t)st.route[r].row * a.row_vecs + first;
#pragma unroll
        for (int u = 0; u < kFoldUnroll; u++) {
          const int v = u * 32 + lane;
          if (first + v < a.row_vecs) cp_async_16(&st.rows[r][v], sp + v);
        }
      }
    }
    cp_async_commit();
  };

  const ItemStep step = step_of(warps, a.pieces_per_row);
  ItemCursor at = cursor_at(warp < items ? warp : 0, a.pieces_per_row);
  if (warp >= items) at.cell = a.cell_num;
  ItemCursor ahead = advance(at, step);
  ItemCursor ahead2 = advance(ahead, step);
  int stage = 0;
  fetch(at);
  issue(my[0], at);
  fetch(ahead);
  while (at.cell < a.cell_num) {
    issue(my[stage ^ 1], ahead);
    fetch(ahead2);
    cp_async_wait<1>();
    __syncwarp();

    const FoldStage& st = my[stage];
    const int64_t cell = cell_at(at.cell);
    const int64_t first = (int64_t)at.piece * kFoldVecs;
    const int count = st.count;
    V* dp = dst + cell * a.row_vecs + first + lane;
    const uint4* r0 = &st.rows[0][lane];
    const uint4* r1 = &st.rows[1][lane];
    const float g0 = st.route[0].gate;
    const float g1 = st.route[1].gate;
    const bool full = first + kFoldVecs <= a.row_vecs;
    if (count <= kMaxRoutes && (count > 0 || !a.is_residual)) {
      // common case: every route of the cell is staged
#pragma unroll
      for (int u = 0; u < kFoldUnroll; u++) {
        if (!full && first + u * 32 + lane >= a.row_vecs) continue;
        float acc[L::N];
#pragma unroll
        for (int n = 0; n < L::N; n++) acc[n] = 0.f;
        if (count >= 1) fold_chunk<VB, DT, GMODE>(acc, r0[u * 32], g0);
        if (count >= 2) fold_chunk<VB, DT, GMODE>(acc, r1[u * 32], g1);
        store_stream(dp + u * 32, pack_chunk<VB, DT>(acc));
      }
    } else if (count > kMaxRoutes) {
      // More routes than the staging area holds: the rest is fetched straight from global
      // memory, two 512-byte chunks of the piece at a time; the loads of a route are issued
      // before the previous route is folded, so one route's latency hides behind the other's
      // arithmetic.  The order stays ascending in the path index.
#pragma unroll 1
      for (int h = 0; h < kFoldUnroll; h += 2) {
        const int v0 = h * 32 + lane, v1 = v0 + 32;
        const bool in0 = first + v0 < a.row_vecs, in1 = first + v1 < a.row_vecs;
        float acc0[L::N], acc1[L::N];
#pragma unroll
        for (int n = 0; n < L::N; n++) acc0[n] = acc1[n] = 0.f;
        fold_chunk<VB, DT, GMODE>(acc0, r0[h * 32], g0);
        fold_chunk<VB, DT, GMODE>(acc1, r0[h * 32 + 32], g0);
        fold_chunk<VB, DT, GMODE>(acc0, r1[h * 32], g1);
        fold_chunk<VB, DT, GMODE>(acc1, r1[h * 32 + 32], g1);
        V held0 = zero_chunk<V>(), held1 = zero_chunk<V>();
        float held_gate = 0.f;
        bool pending = false;
        int seen = 0;
        for (int e = 0; e < E; e++) {
          const int s = a.indices[cell * E + e];
          if (s <= 0 || s > s_loads[e]) continue;
          if (seen++ < kMaxRoutes) continue;
          const V* rp = src + ((int64_t)s_base[e] + s - 1) * a.row_vecs + first;
          const V next0 = in0 ? load_stream(rp + v0) : zero_chunk<V>();
          const V next1 = in1 ? load_stream(rp + v1) : zero_chunk<V>();
          const float next_gate = gate_at<DT, GMODE>(a.gates, cell * E + e);
          if (pending) {
            fold_chunk<VB, DT, GMODE>(acc0, held0, held_gate);
            fold_chunk<VB, DT, GMODE>(acc1, held1, held_gate);
          }
          held0 = next0;
          held1 = next1;
          held_gate = next_gate;
          pending = true;
        }
        if (pending) {
          fold_chunk<VB, DT, GMODE>(acc0, held0, held_gate);
          fold_chunk<VB, DT, GMODE>(acc1, held1, held_gate);
        }
        if (in0) store_stream(dp + h * 32, pack_chunk<VB, DT>(acc0));
        if (in1) store_stream(dp + h * 32 + 32, pack_chunk<VB, DT>(acc1));
      }
    }
    __syncwarp();
    at = ahead;
    ahead = ahead2;
    ahead2 = advance(ahead2, step);
    stage ^= 1;
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------- dispatch (async)

// 1-D seat-index dispatch of 16-byte rows.  Same ownership as dispatch_seat_kernel (a warp
// owns a (cell, 2 KB piece)), but the piece travels through shared memory: the asynchronous
// copy of the warp's NEXT item is in flight while the current one is stored to its routes,
// and cells that no path kept are never read.
template <int DT, bool WEIGHTED, int IV>
__global__ void __launch_bounds__(kThreads, WEIGHTED ? 3 : 4) dispatch_seat_async_kernel(const MoveArgs a) {
  constexpr int VB = 16;
  constexpr int GK = WEIGHTED ? 2 : 0;
  using V = uint4;
  extern __shared__ __align__(16) unsigned char s_raw[];
  CopyStage* s_stage = reinterpret_cast<CopyStage*>(s_raw);  // [kWarps][kStages]
  int* s_loads = reinterpret_cast<int*>(s_raw + sizeof(CopyStage) * kWarps * kStages);
  int* s_base = s_loads + a.path_num;
  int* s_written = s_base + a.path_num;
  int* s_fill = s_written + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);
  const bool dense = a.dense_counts != nullptr;
  if (dense) setup_fill(a.dense_counts, a.path_num, a.max_path_load, s_loads, s_written, s_fill);

  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + warp_in_cta;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;
  CopyStage* my = s_stage + warp_in_cta * kStages;
  const unsigned long long evict_first = l2_evict_first_policy();
  FillPacer pace(items, dense ? (int64_t)s_fill[E] * a.pieces_per_row : 0, warp, warps);

  int seat[IV];
  float gate[IV];
  auto fetch = [&](const ItemCursor& c) {
#pragma unroll
    for (int j = 0; j < IV; j++) { seat[j] = 0; gate[j] = 1.f; }
    if (c.cell < a.cell_num) {
      load_index_chunk<IV>(a.indices, c.cell, E, 0, lane, seat);
      load_gate_chunk<IV, GK, DT>(a.gates, c.cell, E, 0, lane, gate);
    }
  };
  auto issue = [&](CopyStage& st, const ItemCursor& c) {
    if (c.cell < a.cell_num) {
      const int count = build_routes<IV, GK, DT, false>(a, c.cell, seat, gate, s_loads, s_base,
                                                        st.route, lane, kCopyRoutes);
      if (lane == 0) st.count = count;
      if (count > 0) {
        const int64_t first = (int64_t)c.piece * kPieceVecs;
        const V* sp = src + c.cell * a.row_vecs + first;
#pragma unroll
        for (int u = 0; u < kCopyUnroll; u++) {
          const int v = u * 32 + lane;
          if (first + v < a.row_vecs) {
            if (a.loads_evict_first)
              cp_async_16_hint(&st.row[v], sp + v, evict_first);
            else
              cp_async_16(&st.row[v], sp + v);
          }
        }
      }
    }
    cp_async_commit();
  };

  const ItemStep step = step_of(warps, a.pieces_per_row);
  ItemCursor at = cursor_at(warp < items ? warp : 0, a.pieces_per_row);
  if (warp >= items) at.cell = a.cell_num;
  ItemCursor ahead = advance(at, step);
  ItemCursor ahead2 = advance(ahead, step);
  int stage = 0;
  fetch(at);
  issue(my[0], at);
  fetch(ahead);
  while (at.cell < a.cell_num) {
    issue(my[stage ^ 1], ahead);
    fetch(ahead2);
    cp_async_wait<1>();
    __syncwarp();

    const CopyStage& st = my[stage];
    const int64_t cell = at.cell;
    const int64_t first = (int64_t)at.piece * kPieceVecs;
    const int count = st.count;
    if (count > 0) {
      const bool full = first + kPieceVecs <= a.row_vecs;
      V regs[kCopyUnroll];
#pragma unroll
      for (int u = 0; u < kCopyUnroll; u++) regs[u] = st.row[u * 32 + lane];
      const int staged = count < kCopyRoutes ? count : kCopyRoutes;
      for (int r = 0; r < staged; r++) {
        const RouteSlot slot = st.route[r];
        V* dp = dst + (int64_t)slot.row * a.row_vecs + first + lane;
#pragma unroll
        for (int u = 0; u < kCopyUnroll; u++) {
          if (!full && first + u * 32 + lane >= a.row_vecs) continue;
          V out = regs[u];
          if constexpr (WEIGHTED) out = scale_chunk<VB, DT>(regs[u], slot.gate);
          if (a.keep_rows_cached)
            dp[u * 32] = out;
          else
            store_stream(dp + u * 32, out);
        }
        if (at.piece == 0 && lane == 0) {
          if (!dense) a.row_marks[slot.row] = 1;
          if (a.new_tags != nullptr) a.new_tags[slot.row] = a.old_tags[cell];
        }
      }
      if (count > kCopyRoutes) {
        // more routes than the table holds: walk the index row for the rest (warp-uniform)
        int seen = 0;
        for (int e = 0; e < E; e++) {
          const int s = a.indices[cell * E + e];
          if (s <= 0 || s > s_loads[e]) continue;
          if (seen++ < kCopyRoutes) continue;
          const int64_t row = (int64_t)s_base[e] + s - 1;
          float g = 1.f;
          if constexpr (WEIGHTED) g = gate_at<DT, 2>(a.gates, cell * E + e);
          V* dp = dst + row * a.row_vecs + first + lane;
#pragma unroll
          for (int u = 0; u < kCopyUnroll; u++) {
            if (!full && first + u * 32 + lane >= a.row_vecs) continue;
            if constexpr (WEIGHTED)
              store_stream(dp + u * 32, scale_chunk<VB, DT>(regs[u], g));
            else
              store_stream(dp + u * 32, regs[u]);
          }
          if (at.piece == 0 && lane == 0) {
            if (!dense) a.row_marks[row] = 1;
            if (a.new_tags != nullptr) a.new_tags[row] = a.old_tags[cell];
          }
        }
      }
    }
    if (dense)
      for (int n = pace.due(); n > 0 && pace.next < pace.end; n--, pace.next += pace.stride)
        fill_item<VB>(a, s_base, s_written, s_fill, pace.next, lane);
    __syncwarp();
    at = ahead;
    ahead = ahead2;
    ahead2 = advance(ahead2, step);
    stage ^= 1;
  }
  cp_async_wait<0>();
  for (; pace.next < pace.end; pace.next += pace.stride)
    fill_item<VB>(a, s_base, s_written, s_fill, pace.next, lane);
}

// Register-only combine for rows that cannot be moved 16 bytes at a time.
template <int VB, int DT, int GMODE>
__global__ void __launch_bounds__(kThreads) combine_seat_kernel(const MoveArgs a) {
  using L = Lanes<VB, DT>;
  using V = typename L::V;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;

  for (int64_t item = warp; item < items; item += warps) {
    const int64_t cell = item / a.pieces_per_row;
    const int64_t piece = item - cell * a.pieces_per_row;
    float acc[kFoldUnroll][L::N];
#pragma unroll
    for (int u = 0; u < kFoldUnroll; u++)
#pragma unroll
      for (int n = 0; n < L::N; n++) acc[u][n] = 0.f;
    bool routed = false;
    for (int p = 0; p < E; p += 32) {
      const int e_lane = p + lane;
      int seat = 0;
      if (e_lane < E) seat = a.indices[cell * E + e_lane];
      const bool keep = e_lane < E && seat > 0 && seat <= s_loads[e_lane];
      float gate = 1.f;
      if (keep) gate = gate_at<DT, GMODE>(a.gates, cell * E + e_lane);
      unsigned ballot = __ballot_sync(0xffffffffu, keep);
      while (ballot) {
        const int b = __ffs(ballot) - 1;
        ballot &= ballot - 1;
        const int seat_b = __shfl_sync(0xffffffffu, seat, b);
        const float g = __shfl_sync(0xffffffffu, gate, b);
        const V* sp = src + ((int64_t)s_base[p + b] + seat_b - 1) * a.row_vecs;
#pragma unroll
        for (int u = 0; u < kFoldUnroll; u++) {
          const int64_t vec = piece * kFoldVecs + u * 32 + lane;
          if (vec < a.row_vecs) fold_chunk<VB, DT, GMODE>(acc[u], load_stream(sp + vec), g);
        }
        routed = true;
      }
    }
    if (routed || !a.is_residual) {
#pragma unroll
      for (int u = 0; u < kFoldUnroll; u++) {
        const int64_t vec = piece * kFoldVecs + u * 32 + lane;
        if (vec < a.row_vecs)
          store_stream(dst + cell * a.row_vecs + vec, pack_chunk<VB, DT>(acc[u]));
      }
    }
  }
}

// ---------------------------------------------------------------------------------- launch
// Cache behaviour of the two big kernels (read once; the defaults are what measured best on
// the routing step, the variables exist for experiments):
//   BRT_DISPATCH_STORES = cached | stream   rows written with the default policy or evict-first
//   BRT_COMBINE_ORDER   = newest | oldest   cells visited last-to-first or first-to-last
//   BRT_DISPATCH_LOADS  = evict_first | normal   L2 policy of the source rows of a dispatch
bool env_is(const char* name, const char* value, bool otherwise) {
  const char* v = getenv(name);
  return v == nullptr ? otherwise : strcmp(v, value) == 0;
}
int64_t l2_bytes() {
  static thread_local int cached_dev = -1;
  static thread_local int64_t cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrL2CacheSize, dev) != cudaSuccess) n = 0;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}
bool dispatch_keeps_rows_cached() {
  static const bool on = env_is("BRT_DISPATCH_STORES", "cached", true);
  return on;
}
bool dispatch_loads_evict_first() {
  static const bool on = env_is("BRT_DISPATCH_LOADS", "evict_first", true);
  return on;
}
bool combine_newest_first() {
  static const bool on = env_is("BRT_COMBINE_ORDER", "newest", true);
  return on;
}

int pick_vec_bytes(int64_t row_bytes, std::initializer_list<const void*> ptrs, int min_bytes) {
  for (int vb : {16, 8, 4, 2}) {
    if (vb < min_bytes) break;
    if (row_bytes % vb != 0) continue;
    bool ok = true;
    for (const void* p : ptrs)
      if (p != nullptr && !aligned_to(p, vb)) ok = false;
    if (ok) return vb;
  }
  return 0;
}

// warp-per-item kernels
unsigned grid_for_items(int64_t items) {
  int64_t blocks = (items + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

unsigned grid_for_resident(int64_t items, int ctas_per_sm) {
  int64_t blocks = (items + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// 16-byte scans of index (and gate) rows need path_num % 4 == 0 and aligned arrays.
bool wide_rows(const int* indices, const void* gates, int gate_elem_bytes, int path_num) {
  if (path_num % 4 != 0 || !aligned_to(indices, 16)) return false;
  if (gates != nullptr && !aligned_to(gates, (size_t)4 * gate_elem_bytes)) return false;
  return true;
}

// Opt a kernel into more than 48 KB of dynamic shared memory (once per kernel and device).
template <void (*kKernel)(const MoveArgs)>
void configure_smem(size_t stage_bytes) {
  static thread_local int configured_device = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || configured_device == dev) return;
  cudaFuncSetAttribute(kKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       (int)(stage_bytes + ((size_t)kMaxPaths * 4 + 4) * sizeof(int)));
  configured_device = dev;
}

template <int VB, int DT, bool WEIGHTED, bool IS_1D>
void launch_dispatch(const MoveArgs& a, bool is_tag, cudaStream_t st) {
  const KernelTimer timer(is_tag ? "dispatch_tag_kernel"
                                 : a.dense_counts != nullptr ? "dispatch_kernel"
                                                             : "dispatch_move_kernel",
                          st);
  const size_t smem = (a.dense_counts != nullptr ? (size_t)a.path_num * 4 + 4
                                                 : (size_t)a.path_num * 2) * sizeof(int);
  if (is_tag) {
    dispatch_tag_kernel<VB, DT, WEIGHTED, IS_1D>
        <<<grid_for_items(a.total_rows * a.pieces_per_row), kThreads, smem, st>>>(a), note_launch();
  } else if (VB == 16 && IS_1D) {
    if constexpr (VB == 16 && IS_1D) {
      const size_t smem_async = sizeof(CopyStage) * kWarps * kStages + smem;
      const int64_t work = (a.cell_num + (a.dense_counts != nullptr ? a.total_rows : 0)) *
                           a.pieces_per_row;
      const unsigned grid = grid_for_resident(work, WEIGHTED ? 3 : 4);
      if (wide_rows(a.indices, a.gates, dtype_size(DT), a.path_num)) {
        configure_smem<dispatch_seat_async_kernel<DT, WEIGHTED, 4>>(sizeof(CopyStage) * kWarps *
                                                                    kStages);
        dispatch_seat_async_kernel<DT, WEIGHTED, 4><<<grid, kThreads, smem_async, st>>>(a), note_launch();
      } else {
        configure_smem<dispatch_seat_async_kernel<DT, WEIGHTED, 1>>(sizeof(CopyStage) * kWarps *
                                                                    kStages);
        dispatch_seat_async_kernel<DT, WEIGHTED, 1><<<grid, kThreads, smem_async, st>>>(a), note_launch();
      }
    }
  } else {
    const int64_t work = (a.cell_num + (a.dense_counts != nullptr ? a.total_rows : 0)) *
                         a.pieces_per_row;
    if (wide_rows(a.indices, a.gates, dtype_size(DT), a.path_num))
      dispatch_seat_kernel<VB, DT, WEIGHTED, IS_1D, 4>
          <<<grid_for_items(work), kThreads, smem, st>>>(a), note_launch();
    else
      dispatch_seat_kernel<VB, DT, WEIGHTED, IS_1D, 1>
          <<<grid_for_items(work), kThreads, smem, st>>>(a), note_launch();
  }
}

template <int VB>
int dispatch_by_flags(const MoveArgs& a, int dtype, bool weighted, bool is_1d, bool is_tag,
                      cudaStream_t st) {
  if (!weighted) {
    // an unweighted move is a byte copy: the element type does not matter
    if (is_1d)
      launch_dispatch<VB, BRT_BF16, false, true>(a, is_tag, st);
    else
      launch_dispatch<VB, BRT_BF16, false, false>(a, is_tag, st);
    return BRT_OK;
  }
  if (dtype == BRT_F32) {
    if constexpr (VB >= 4) {
      launch_dispatch<VB, BRT_F32, true, true>(a, is_tag, st);
      return BRT_OK;
    }
    return set_error(BRT_ERR_INVALID_ARGUMENT, "fp32 rows must be 4-byte aligned");
  }
  if (dtype == BRT_F16)
    launch_dispatch<VB, BRT_F16, true, true>(a, is_tag, st);
  else
    launch_dispatch<VB, BRT_BF16, true, true>(a, is_tag, st);
  return BRT_OK;
}

template <int VB>
void launch_zero_fill(const MoveArgs& a, cudaStream_t st) {
  const KernelTimer timer("dispatch_zero_fill_kernel", st);
  dispatch_zero_fill_kernel<VB>
      <<<grid_for_items(a.total_rows * a.pieces_per_row), kThreads, 0, st>>>(a), note_launch();
}

template <int DT, int GMODE, int IV>
int launch_combine_async(const MoveArgs& a, cudaStream_t st) {
  const size_t smem = sizeof(FoldStage) * kWarps * kStages + (size_t)a.path_num * 2 * sizeof(int);
  static thread_local int configured_device = -1;
  int dev = 0;
  BRT_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    BRT_CUDA_TRY(cudaFuncSetAttribute(combine_seat_async_kernel<DT, GMODE, IV>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(sizeof(FoldStage) * kWarps * kStages +
                                            (size_t)kMaxPaths * 2 * sizeof(int))));
    configured_device = dev;
  }
  const KernelTimer timer("combine_kernel", st);
  combine_seat_async_kernel<DT, GMODE, IV>
      <<<grid_for_resident(a.cell_num * a.pieces_per_row, 3), kThreads, smem, st>>>(a), note_launch();
  return BRT_OK;
}

template <int VB, int DT, int GMODE>
int launch_combine(const MoveArgs& a, cudaStream_t st) {
  if constexpr (VB == 16) {
    const int gate_bytes = GMODE == 1 ? 4 : dtype_size(DT);
    if (wide_rows(a.indices, a.gates, gate_bytes, a.path_num))
      return launch_combine_async<DT, GMODE, 4>(a, st);
    return launch_combine_async<DT, GMODE, 1>(a, st);
  } else {
    const size_t smem = (size_t)a.path_num * 2 * sizeof(int);
    const KernelTimer timer("combine_kernel", st);
    combine_seat_kernel<VB, DT, GMODE>
        <<<grid_for_items(a.cell_num * a.pieces_per_row), kThreads, smem, st>>>(a), note_launch();
    return BRT_OK;
  }
}

template <int VB, int DT>
int combine_by_gates(const MoveArgs& a, int gmode, cudaStream_t st) {
  if (gmode == 0) return launch_combine<VB, DT, 0>(a, st);
  if (gmode == 1 || DT == BRT_F32) return launch_combine<VB, DT, 1>(a, st);
  return launch_combine<VB, DT, 2>(a, st);
}

template <int VB>
int combine_by_dtype(const MoveArgs& a, int dtype, int gmode, cudaStream_t st) {
  if (dtype == BRT_F32) {
    if constexpr (VB >= 4) return combine_by_gates<VB, BRT_F32>(a, gmode, st);
    return set_error(BRT_ERR_INVALID_ARGUMENT, "fp32 rows must be 4-byte aligned");
  }
  if (dtype == BRT_F16) return combine_by_gates<VB, BRT_F16>(a, gmode, st);
  return combine_by_gates<VB, BRT_BF16>(a, gmode, st);
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API size_t brt_dispatch_scratch_bytes(int64_t total_rows, int path_num) {
  (void)path_num;
  if (total_rows < 0) total_rows = 0;
  return round_up((size_t)total_rows + 1, 256);
}

BRT_API int brt_dispatch_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, const int32_t* old_tags, int32_t* new_tags, int64_t cell_num,
    int64_t cell_size, int path_num, int32_t max_path_load, int64_t total_rows,
    int is_1d_routing, int is_tag_index, int dtype, const int32_t* dense_counts, void* scratch,
    size_t scratch_bytes, void* stream) {
  clear_error();
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(cell_num >= 0 && cell_size >= 0 && total_rows >= 0, "negative size");
  BRT_REQUIRE(path_num > 0 && path_num <= kMaxPaths, "path_num %d outside [1, %d]", path_num,
              kMaxPaths);
  BRT_REQUIRE(max_path_load >= 0, "negative max_path_load");
  BRT_REQUIRE(total_rows <= 0x7fffffffLL, "more than 2^31-1 output rows");
  BRT_REQUIRE((old_tags == nullptr) == (new_tags == nullptr),
              "old_tags and new_tags must be given together");
  BRT_REQUIRE(gates == nullptr || is_1d_routing, "gates are only supported with 1-D routing");
  if (total_rows == 0 || cell_size == 0) return BRT_OK;
  BRT_REQUIRE(dst_data != nullptr && route_indices != nullptr && loads != nullptr,
              "null pointer argument");
  BRT_REQUIRE(cell_num == 0 || src_data != nullptr, "src_data is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int es = dtype_size(dtype);
  const int64_t row_bytes = cell_size * es;
  const int vb = pick_vec_bytes(row_bytes, {src_data, dst_data}, gates != nullptr ? es : 2);
  BRT_REQUIRE(vb != 0, "rows of %lld bytes cannot be moved: misaligned pointers",
              (long long)row_bytes);

  MoveArgs a;
  a.src = src_data;
  a.dst = dst_data;
  a.gates = gates;
  a.indices = route_indices;
  a.loads = loads;
  a.old_tags = old_tags;
  a.new_tags = new_tags;
  a.row_marks = static_cast<unsigned char*>(scratch);
  // the one-launch path for dense seat columns (its per-path tables live in shared memory)
  const bool dense = dense_counts != nullptr && !is_tag_index && path_num <= 2048;
  a.dense_counts = dense ? dense_counts : nullptr;
  // rows stay in L2 for the op that reads them next only when the output is of L2's order of
  // size; a larger output is streamed (measured: cached stores of a 512 MB output cost 30 %)
  a.keep_rows_cached =
      dispatch_keeps_rows_cached() && total_rows * row_bytes <= (int64_t)l2_bytes() * 5 / 4;
  a.loads_evict_first = dispatch_loads_evict_first() ? 1 : 0;
  a.newest_first = 0;
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / vb;
  a.pieces_per_row = (a.row_vecs + kPieceVecs - 1) / kPieceVecs;
  a.path_num = path_num;
  a.max_path_load = max_path_load;
  a.total_rows = total_rows;
  a.is_residual = 0;

  const bool is_tag = is_tag_index != 0;
  if (!is_tag && !dense) {
    const size_t need = brt_dispatch_scratch_bytes(total_rows, path_num);
    BRT_REQUIRE(scratch != nullptr, "scratch is null");
    if (scratch_bytes < need)
      return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                       scratch_bytes, need);
    BRT_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)total_rows, st));
  }
  int rc = BRT_OK;
  if (cell_num > 0 || is_tag || dense) {
    switch (vb) {
      case 16: rc = dispatch_by_flags<16>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      case 8: rc = dispatch_by_flags<8>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      case 4: rc = dispatch_by_flags<4>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      default: rc = dispatch_by_flags<2>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
    }
    if (rc != BRT_OK) return rc;
    BRT_LAUNCH_CHECK("dispatch kernel");
  }
  if (!is_tag && !dense) {
    switch (vb) {
      case 16: launch_zero_fill<16>(a, st); break;
      case 8: launch_zero_fill<8>(a, st); break;
      case 4: launch_zero_fill<4>(a, st); break;
      default: launch_zero_fill<2>(a, st); break;
    }
    BRT_LAUNCH_CHECK("dispatch_zero_fill_kernel");
  }
  return BRT_OK;
}

BRT_API int brt_combine_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, int64_t cell_num, int64_t cell_size, int path_num,
    int32_t max_path_load, int is_residual, int dtype, int gates_dtype, void* stream) {
  clear_error();
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(gates == nullptr || gates_dtype == BRT_F32 || gates_dtype == dtype,
              "gates must be fp32 or match the data type");
  BRT_REQUIRE(cell_num >= 0 && cell_size >= 0, "negative size");
  BRT_REQUIRE(path_num > 0 && path_num <= kMaxPaths, "path_num %d outside [1, %d]", path_num,
              kMaxPaths);
  BRT_REQUIRE(max_path_load >= 0, "negative max_path_load");
  if (cell_num == 0 || cell_size == 0) return BRT_OK;
  BRT_REQUIRE(dst_data != nullptr && route_indices != nullptr && loads != nullptr,
              "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype_size(dtype);
  const int64_t row_bytes = cell_size * es;
  const int vb = pick_vec_bytes(row_bytes, {src_data, dst_data}, es);
  BRT_REQUIRE(vb != 0, "rows of %lld bytes cannot be moved: misaligned pointers",
              (long long)row_bytes);
  MoveArgs a;
  a.src = src_data;
  a.dst = dst_data;
  a.gates = gates;
  a.indices = route_indices;
  a.loads = loads;
  a.old_tags = nullptr;
  a.new_tags = nullptr;
  a.row_marks = nullptr;
  a.dense_counts = nullptr;
  a.keep_rows_cached = 0;
  a.loads_evict_first = 0;
  a.newest_first = combine_newest_first() ? 1 : 0;
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / vb;
  a.pieces_per_row = (a.row_vecs + kFoldVecs - 1) / kFoldVecs;
  a.path_num = path_num;
  a.max_path_load = max_path_load;
  a.total_rows = 0;
  a.is_residual = is_residual;
  const int gmode = gates == nullptr ? 0 : (gates_dtype == BRT_F32 ? 1 : 2);
  int rc;
  switch (vb) {
    case 16: rc = combine_by_dtype<16>(a, dtype, gmode, st); break;
    case 8: rc = combine_by_dtype<8>(a, dtype, gmode, st); break;
    case 4: rc = combine_by_dtype<4>(a, dtype, gmode, st); break;
    default: rc = combine_by_dtype<2>(a, dtype, gmode, st); break;
  }
  if (rc != BRT_OK) return rc;
  BRT_LAUNCH_CHECK("combine_seat_kernel");
  return BRT_OK;
}

}  // extern "C"
