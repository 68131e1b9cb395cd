// Weighted combine fused with the inverse expert-parallel exchange.
//
// The unfused sequence is: a landing kernel stores every bucket of expert outputs back into its
// owner's rank-major layout, then combine reads those rows locally.  Here combine PULLS: for
// every kept route of a cell it reads the expert's output row straight from the arena of the
// rank that hosts the expert (plain 16-byte peer loads through cp.async; no TMA, no
// multicast), folds the routes in ascending path order and writes the cell once.  A row
// crosses NVLink once and is never written to or read from local HBM in between; on this
// hardware SM-issued peer loads also run faster than peer stores (about 2 us + bytes / 770 GB/s
// against 8 us + bytes / 718 GB/s).
//
//   prologue : wait (bounded) until every rank has posted this exchange (its expert outputs
//              are complete), then every CTA derives from the size matrix kept by the forward
//              exchange where the rows of each of MY buckets (destination rank i, its local
//              expert j) start in rank i's [local expert][source rank] layout and keeps one
//              pointer per global path in shared memory;
//   body     : the software-pipelined combine of row_move.cu (a warp owns a (cell, 2 KB piece);
//              the rows of the warp's next item are on their way into shared memory while the
//              current item is folded), with the row address taken from the per-path pointer.
//              Order and rounding of the fold are those of the local combine: ascending path,
//              fp32 multiply then add, one rounding to the storage type;
//   epilogue : the last CTA raises this rank's arrival flag at every rank: "I have finished
//              reading your rows".  The owner waits for all of them (the wait kernel that
//              follows) before anything may overwrite the rows.
//
// 16-byte-multiple rows, no residual input; the host side takes the unfused path for the rest.
#include "exchange_p2p.cuh"
#include "row_move.cuh"

namespace brt_b200 {
namespace {

using rows::FoldStage;
using rows::ItemCursor;
using rows::ItemStep;
using rows::kFoldUnroll;
using rows::kFoldVecs;
using rows::kMaxRoutes;
using rows::kStages;
using rows::kWarps;

constexpr int kThreads = rows::kThreads;
static_assert(rows::kThreads == p2p::kThreads, "both building blocks assume 256 threads");

struct CombineLandArgs {
  // the combine
  void* dst;
  const void* gates;
  const int* indices;
  int64_t cell_num;
  int64_t row_vecs;  // 16-byte vectors per row
  int64_t pieces_per_row;
  // the exchange
  int world_size, my_rank, group_size;
  long long stride_rows;  // 0: packed buckets
  unsigned long long epoch, limit_ns;
  unsigned long long* trace;                // see P2pReplay
  const unsigned long long* epoch_counter;  // see p2p::effective_epoch()
  const int* sizes;                         // [world][world * group]: the forward exchange's
  const unsigned long long* ready_flags;
  const char* rows_at[p2p::kMaxRanks];      // first expert-output row in every rank's arena
  unsigned long long* arrive_flags[p2p::kMaxRanks];
  unsigned int* done_counter;
  unsigned int* abort_word;
  p2p::StatusSink status;
};

__host__ __device__ inline size_t pull_plan_bytes(int n) {
  // s_ptr[n] (8 B) | s_loads[n] s_below[n] | s_aux[n+1] | s_warp[8]
  return (size_t)n * 8 + (size_t)n * 4 * 2 + (size_t)(n + 1) * 4 + 8 * 4 + 16;
}

// As rows::build_routes, but a slot keeps (path, seat - 1): the row's address comes from the
// per-path pointer.  Returns the total count of kept routes.
template <int IV, int GK, int DT>
__device__ __forceinline__ int build_pull_routes(const int* __restrict__ indices,
                                                 const void* __restrict__ gates, int E,
                                                 int64_t cell, const int (&first_seat)[IV],
                                                 const float (&first_gate)[IV],
                                                 const int* s_loads, rows::RouteSlot* slots,
                                                 int* paths, int lane) {
  const int chunks = (E + 32 * IV - 1) / (32 * IV);
  int count = 0;
  for (int c = 0; c < chunks; c++) {
    int seat[IV];
    float gate[IV];
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < IV; j++) { seat[j] = first_seat[j]; gate[j] = first_gate[j]; }
    } else {
      rows::load_index_chunk<IV>(indices, cell, E, c, lane, seat);
      rows::load_gate_chunk<IV, GK, DT>(gates, cell, E, c, lane, gate);
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
          if (count < kMaxRoutes && lane == 0) {
            slots[count].row = seat_b - 1;
            slots[count].gate = g;
            paths[count] = e;
          }
          count++;
        }
      }
    }
  }
  return count;
}

// GMODE: 0 = no gates, 1 = fp32 gates, 2 = gates stored in the data type.
template <int DT, int GMODE, int IV>
__global__ void __launch_bounds__(kThreads, 3)
combine_land_kernel(const __grid_constant__ CombineLandArgs a) {
  constexpr int VB = 16;
  using L = rows::Lanes<VB, DT>;
  using V = uint4;
  extern __shared__ __align__(16) unsigned char s_raw[];
  FoldStage* s_stage = reinterpret_cast<FoldStage*>(s_raw);  // [kWarps][kStages]
  int* s_paths = reinterpret_cast<int*>(s_raw + sizeof(FoldStage) * kWarps * kStages);
  unsigned char* at_plan = reinterpret_cast<unsigned char*>(s_paths + kWarps * kStages * kMaxRoutes);
  const int W = a.world_size, G = a.group_size, me = a.my_rank;
  const int n = W * G;
  const char** s_ptr = reinterpret_cast<const char**>(at_plan);
  int* s_loads = reinterpret_cast<int*>(at_plan + (size_t)n * 8);
  int* s_below = s_loads + n;
  int* s_aux = s_below + n;    // n + 1
  int* s_warp = s_aux + n + 1;  // 8
  const int tid = threadIdx.x;
  const long long grain = a.row_vecs * 16;

  const unsigned long long epoch = p2p::effective_epoch(a.epoch, a.epoch_counter);
  const bool tracer = a.trace != nullptr && blockIdx.x == 0 && tid == 0;
  if (tracer) {
    a.trace[0] = p2p::global_timer_ns();
    a.trace[4] = ~0ull;
    a.trace[5] = 0ull;
  }
  // every rank has posted this exchange: its expert outputs are in place
  const bool go = p2p::wait_for_flags(a.ready_flags, W, -1, epoch, a.limit_ns);
  if (tracer) a.trace[1] = p2p::global_timer_ns();
  if (!go && tid == 0) {
    p2p::report_timeout(a.status);
    atomicExch(a.abort_word, 1u);
  }
  if (go) {
    const int* S = a.sizes;
    for (int e = tid; e < n; e += kThreads) {
      int column = 0, below = 0;
      for (int s = 0; s < W; s++) {
        const int raw = __ldcg(S + s * n + e);
        const int v = raw > 0 ? raw : 0;
        column += v;
        if (s < me) below += v;
      }
      int mine = __ldcg(S + me * n + e);
      if (mine < 0) mine = 0;
      if (a.stride_rows != 0 && mine > a.stride_rows) mine = (int)a.stride_rows;
      s_aux[e] = column;
      s_below[e] = below;
      s_loads[e] = mine;
    }
    p2p::block_exclusive_scan(s_aux, n, s_warp);
    for (int e = tid; e < n; e += kThreads) {
      const int i = e / G, j = e - i * G;
      const long long row0 = a.stride_rows ? (long long)(j * W + me) * a.stride_rows
                                           : (long long)(s_aux[e] - s_aux[i * G] + s_below[e]);
      s_ptr[e] = a.rows_at[i] + row0 * grain;
    }
    __syncthreads();
  }
  if (tracer) a.trace[3] = p2p::global_timer_ns();

  if (go) {
    const int lane = tid & 31;
    const int warp_in_cta = tid >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + warp_in_cta;
    const int64_t warps = (int64_t)gridDim.x * kWarps;
    const int64_t items = a.cell_num * a.pieces_per_row;
    V* __restrict__ dst = static_cast<V*>(a.dst);
    const int E = n;
    FoldStage* my = s_stage + warp_in_cta * kStages;
    int* my_paths = s_paths + warp_in_cta * kStages * kMaxRoutes;

    int seat[IV];
    float gate[IV];
    auto fetch = [&](const ItemCursor& c) {
#pragma unroll
      for (int j = 0; j < IV; j++) { seat[j] = 0; gate[j] = 1.f; }
      if (c.cell < a.cell_num) {
        rows::load_index_chunk<IV>(a.indices, c.cell, E, 0, lane, seat);
        rows::load_gate_chunk<IV, GMODE, DT>(a.gates, c.cell, E, 0, lane, gate);
      }
    };
    // Build the route table of an item from the registers fetched for it and start the
    // asynchronous copies of its rows; always closes exactly one copy group.
    auto issue = [&](int stage, const ItemCursor& c) {
      FoldStage& st = my[stage];
      int* paths = my_paths + stage * kMaxRoutes;
      if (c.cell < a.cell_num) {
        const int count = build_pull_routes<IV, GMODE, DT>(a.indices, a.gates, E, c.cell, seat,
                                                           gate, s_loads, st.route, paths, lane);
        if (lane == 0) st.count = count;
        __syncwarp();
        const int staged = count < kMaxRoutes ? count : kMaxRoutes;
        const int64_t first = (int64_t)c.piece * kFoldVecs;
        for (int r = 0; r < staged; r++) {
          const V* sp = reinterpret_cast<const V*>(s_ptr[paths[r]]) +
                        (int64_t)st.route[r].row * a.row_vecs + first;
#pragma unroll
          for (int u = 0; u < kFoldUnroll; u++) {
            const int v = u * 32 + lane;
            if (first + v < a.row_vecs) cp_async_16(&st.rows[r][v], sp + v);
          }
        }
      }
      cp_async_commit();
    };

    const ItemStep step = rows::step_of(warps, a.pieces_per_row);
    ItemCursor at = rows::cursor_at(warp < items ? warp : 0, a.pieces_per_row);
    if (warp >= items) at.cell = a.cell_num;
    ItemCursor ahead = rows::advance(at, step);
    ItemCursor ahead2 = rows::advance(ahead, step);
    int stage = 0;
    fetch(at);
    issue(0, at);
    fetch(ahead);
    while (at.cell < a.cell_num) {
      issue(stage ^ 1, ahead);
      fetch(ahead2);
      cp_async_wait<1>();
      __syncwarp();

      const FoldStage& st = my[stage];
      const int64_t cell = at.cell;
      const int64_t first = (int64_t)at.piece * kFoldVecs;
      const int count = st.count;
      V* dp = dst + cell * a.row_vecs + first + lane;
      const uint4* r0 = &st.rows[0][lane];
      const uint4* r1 = &st.rows[1][lane];
      const float g0 = st.route[0].gate;
      const float g1 = st.route[1].gate;
      const bool full = first + kFoldVecs <= a.row_vecs;
      if (count <= kMaxRoutes) {
        // common case: every route of the cell is staged (no route: the cell is zero)
#pragma unroll
        for (int u = 0; u < kFoldUnroll; u++) {
          if (!full && first + u * 32 + lane >= a.row_vecs) continue;
          float acc[L::N];
#pragma unroll
          for (int k = 0; k < L::N; k++) acc[k] = 0.f;
          if (count >= 1) rows::fold_chunk<VB, DT, GMODE>(acc, r0[u * 32], g0);
          if (count >= 2) rows::fold_chunk<VB, DT, GMODE>(acc, r1[u * 32], g1);
          store_stream(dp + u * 32, rows::pack_chunk<VB, DT>(acc));
        }
      } else {
        // more routes than the staging area holds: the rest comes straight from the peers,
        // in ascending path order like the staged ones
#pragma unroll 1
        for (int u = 0; u < kFoldUnroll; u++) {
          const int v = u * 32 + lane;
          const bool in = first + v < a.row_vecs;
          float acc[L::N];
#pragma unroll
          for (int k = 0; k < L::N; k++) acc[k] = 0.f;
          rows::fold_chunk<VB, DT, GMODE>(acc, r0[u * 32], g0);
          rows::fold_chunk<VB, DT, GMODE>(acc, r1[u * 32], g1);
          int seen = 0;
          for (int e = 0; e < E; e++) {
            const int s = a.indices[cell * E + e];
            if (s <= 0 || s > s_loads[e]) continue;
            if (seen++ < kMaxRoutes) continue;
            const V* rp = reinterpret_cast<const V*>(s_ptr[e]) + (int64_t)(s - 1) * a.row_vecs +
                          first;
            const V row = in ? load_stream(rp + v) : zero_chunk<V>();
            rows::fold_chunk<VB, DT, GMODE>(acc, row,
                                            rows::gate_at<DT, GMODE>(a.gates, cell * E + e));
          }
          if (in) store_stream(dp + u * 32, rows::pack_chunk<VB, DT>(acc));
        }
      }
      __syncwarp();
      at = ahead;
      ahead = ahead2;
      ahead2 = rows::advance(ahead2, step);
      stage ^= 1;
    }
    cp_async_wait<0>();
  }

  // arrive: the last CTA to finish tells every rank that this rank has read its rows
  if (a.trace != nullptr) {
    __syncthreads();
    if (tid == 0) {
      const unsigned long long now = p2p::global_timer_ns();
      atomicMin(a.trace + 4, now);
      atomicMax(a.trace + 5, now);
    }
  }
  // Ordering the flag after every thread's accesses without a system-scope fence per thread
  // (or per CTA: those serialise device-wide and cost about 10 us per launch).  The CTA
  // barrier orders the CTA's accesses before thread 0; its device-scope fence and the counter
  // update release them to the CTA that finds the counter complete, whose single system-scope
  // fence precedes the flags: fences are cumulative, so the chain covers every access.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(a.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *a.done_counter = 0;
      const unsigned int aborted = atomicExch(a.abort_word, 0u);
      __threadfence_system();
      if (aborted == 0u)
        for (int r = 0; r < W; r++) p2p::store_release_sys(a.arrive_flags[r] + me, epoch);
      if (a.trace != nullptr) a.trace[2] = p2p::global_timer_ns();
    }
  }
}

template <int DT, int GMODE, int IV>
int launch(const CombineLandArgs& a, cudaStream_t st) {
  const int n = a.world_size * a.group_size;
  const size_t fixed = sizeof(FoldStage) * kWarps * kStages +
                       sizeof(int) * kWarps * kStages * kMaxRoutes;
  const size_t smem = fixed + pull_plan_bytes(n);
  static thread_local int configured_device = -1;
  int dev = 0;
  BRT_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    BRT_CUDA_TRY(cudaFuncSetAttribute(combine_land_kernel<DT, GMODE, IV>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(fixed + pull_plan_bytes(p2p::kMaxBuckets))));
    configured_device = dev;
  }
  const KernelTimer timer("combine_land_kernel", st);
  combine_land_kernel<DT, GMODE, IV><<<(unsigned)(sm_count() * 3), kThreads, smem, st>>>(a),
      note_launch();
  BRT_LAUNCH_CHECK("combine_land_kernel");
  return BRT_OK;
}

template <int DT, int GMODE>
int launch_by_width(const CombineLandArgs& a, int gate_bytes, cudaStream_t st) {
  const int n = a.world_size * a.group_size;
  // 16-byte scans of index (and gate) rows need a path count that is a multiple of 4 and
  // aligned arrays
  const bool wide = n % 4 == 0 && aligned_to(a.indices, 16) &&
                    (a.gates == nullptr || aligned_to(a.gates, (size_t)4 * gate_bytes));
  return wide ? launch<DT, GMODE, 4>(a, st) : launch<DT, GMODE, 1>(a, st);
}

template <int DT>
int launch_by_gates(const CombineLandArgs& a, int gmode, cudaStream_t st) {
  if (gmode == 0) return launch_by_width<DT, 0>(a, 4, st);
  if (gmode == 1 || DT == BRT_F32) return launch_by_width<DT, 1>(a, 4, st);
  return launch_by_width<DT, 2>(a, dtype_size(DT), st);
}

}  // namespace

int p2p_combine_land_launch(void* dst_data, const void* gates, int gates_dtype, int dtype,
                            const int32_t* route_indices, int64_t cell_num, int64_t row_bytes,
                            const int32_t* size_matrix, int world_size, int group_size,
                            int my_rank, int64_t stride_rows, const void* const* expert_rows,
                            uint64_t epoch, const void* my_ready_flags,
                            void* const* peer_arrive_flag_arrays, void* my_done_counter,
                            void* my_abort_word, void* status_word, void* host_status_word,
                            uint64_t wait_limit_ns, const P2pReplay& replay, void* stream) {
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(gates == nullptr || gates_dtype == BRT_F32 || gates_dtype == dtype,
              "gates must be fp32 or match the data type");
  BRT_REQUIRE(route_indices != nullptr && size_matrix != nullptr && expert_rows != nullptr &&
                  my_ready_flags != nullptr && peer_arrive_flag_arrays != nullptr &&
                  my_done_counter != nullptr && my_abort_word != nullptr &&
                  status_word != nullptr,
              "null pointers");
  BRT_REQUIRE(cell_num >= 0 && (cell_num == 0 || dst_data != nullptr), "dst_data is null");
  BRT_REQUIRE(world_size >= 1 && world_size <= p2p::kMaxRanks && my_rank >= 0 &&
                  my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(group_size >= 1 && (long long)world_size * group_size <= p2p::kMaxBuckets,
              "at most %d buckets per exchange", p2p::kMaxBuckets);
  BRT_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && aligned_to(dst_data, 16),
              "rows must be 16-byte multiples and the output 16-byte aligned");
  BRT_REQUIRE(stride_rows >= 0, "negative slot size");
  CombineLandArgs a;
  a.dst = dst_data;
  a.gates = gates;
  a.indices = route_indices;
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / 16;
  a.pieces_per_row = (a.row_vecs + kFoldVecs - 1) / kFoldVecs;
  a.world_size = world_size;
  a.my_rank = my_rank;
  a.group_size = group_size;
  a.stride_rows = stride_rows;
  a.epoch = epoch;
  a.limit_ns = wait_limit_ns;
  a.trace = static_cast<unsigned long long*>(replay.trace);
  a.epoch_counter = static_cast<const unsigned long long*>(replay.epoch_counter);
  a.sizes = size_matrix;
  a.ready_flags = static_cast<const unsigned long long*>(my_ready_flags);
  for (int r = 0; r < world_size; r++) {
    BRT_REQUIRE(expert_rows[r] != nullptr && aligned_to(expert_rows[r], 16),
                "expert rows of rank %d are null or not 16-byte aligned", r);
    a.rows_at[r] = static_cast<const char*>(expert_rows[r]);
    a.arrive_flags[r] = static_cast<unsigned long long*>(peer_arrive_flag_arrays[r]);
  }
  a.done_counter = static_cast<unsigned int*>(my_done_counter);
  a.abort_word = static_cast<unsigned int*>(my_abort_word);
  a.status.device_word = static_cast<int*>(status_word);
  a.status.host_word = static_cast<int*>(host_status_word);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int gmode = gates == nullptr ? 0 : (gates_dtype == BRT_F32 ? 1 : 2);
  switch (dtype) {
    case BRT_F32: return launch_by_gates<BRT_F32>(a, gmode, st);
    case BRT_F16: return launch_by_gates<BRT_F16>(a, gmode, st);
    default: return launch_by_gates<BRT_BF16>(a, gmode, st);
  }
}

}  // namespace brt_b200
