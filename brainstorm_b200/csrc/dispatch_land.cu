// Token dispatch fused with the forward expert-parallel exchange.
//
// The unfused sequence is: dispatch the cells into a local [path, seat] buffer, then a landing
// kernel reads that buffer and stores every bucket into its destination rank's output layout.
// Here the dispatch stores each kept copy of a cell STRAIGHT into the destination rank's
// landing half (plain 16-byte peer stores over NVLink; no TMA, no multicast): a source row is
// read once from local HBM and never written locally, the packed send buffer does not exist.
//
//   prologue : wait (bounded) until every rank has entered the exchange, then every CTA derives
//              from the size matrix on its board where each global path (destination rank,
//              its local expert) starts in that rank's [local expert][source rank] layout and
//              keeps one pointer per path in shared memory;
//   body     : the software-pipelined dispatch of row_move.cu (a warp owns a (cell, 2 KB
//              piece); the piece of the warp's next item is already on its way into shared
//              memory while the current one is stored to its routes), with the route's row
//              address taken from the per-path pointer.  Rows of a bucket that no cell fills
//              (loads padded above the cell counts) are written as zeros at the destination;
//   epilogue : the last CTA raises this rank's arrival flag at every rank.
//
// Unweighted 1-D routing of 16-byte-multiple rows with library-made (dense) seat indices only;
// the host side takes the unfused path for everything else.
#include "exchange_p2p.cuh"
#include "row_move.cuh"

namespace brt_b200 {
namespace {

using rows::CopyStage;
using rows::ItemCursor;
using rows::ItemStep;
using rows::kCopyRoutes;
using rows::kCopyUnroll;
using rows::kPieceVecs;
using rows::kStages;
using rows::kWarps;
using rows::RouteSlot;

constexpr int kThreads = rows::kThreads;
static_assert(rows::kThreads == p2p::kThreads, "both building blocks assume 256 threads");

struct DispatchLandArgs {
  // the dispatch
  const void* src;
  const int* indices;
  const int* dense_counts;
  int64_t cell_num;
  int64_t row_vecs;        // 16-byte vectors per row
  int64_t pieces_per_row;
  // the exchange
  int world_size, my_rank, group_size;
  long long stride_rows;   // 0: packed buckets
  long long half_bytes;
  unsigned long long epoch, limit_ns;
  unsigned long long* trace;                // see P2pReplay
  unsigned long long* work_counter;         // see P2pReplay
  const unsigned long long* epoch_counter;  // see p2p::effective_epoch()
  int strict;              // rows that do not fit are reported as an error
  const int* sizes;        // [world][world * group] on my board
  int* keep;
  const unsigned long long* ready_flags;
  char* land[p2p::kMaxRanks];
  unsigned long long* arrive_flags[p2p::kMaxRanks];
  unsigned int* done_counter;
  unsigned int* abort_word;
  p2p::StatusSink status;
};

__host__ __device__ inline size_t plan_bytes(int n) {
  // s_ptr[n] (8 B) | s_loads[n] s_written[n] s_zero[n] s_below[n] | s_fill[n+1] s_aux[n+1] |
  // s_warp[8]
  return (size_t)n * 8 + (size_t)n * 4 * 4 + (size_t)(n + 1) * 4 * 2 + 8 * 4 + 16;
}

template <int IV>
__global__ void __launch_bounds__(kThreads, 3)
dispatch_land_kernel(const __grid_constant__ DispatchLandArgs a) {
  using V = uint4;
  extern __shared__ __align__(16) unsigned char s_raw[];
  CopyStage* s_stage = reinterpret_cast<CopyStage*>(s_raw);  // [kWarps][kStages]
  unsigned char* at_plan = s_raw + sizeof(CopyStage) * kWarps * kStages;
  const int W = a.world_size, G = a.group_size, me = a.my_rank;
  const int n = W * G;
  char** s_ptr = reinterpret_cast<char**>(at_plan);
  int* s_loads = reinterpret_cast<int*>(at_plan + (size_t)n * 8);
  int* s_written = s_loads + n;
  int* s_zero = s_written + n;
  int* s_below = s_zero + n;
  int* s_fill = s_below + n;      // n + 1
  int* s_aux = s_fill + n + 1;    // n + 1
  int* s_warp = s_aux + n + 1;    // 8
  const int tid = threadIdx.x;
  const long long grain = a.row_vecs * 16;

  const unsigned long long epoch = p2p::effective_epoch(a.epoch, a.epoch_counter);
  const bool tracer = a.trace != nullptr && blockIdx.x == 0 && tid == 0;
  if (tracer) {
    a.trace[0] = p2p::global_timer_ns();
    a.trace[4] = ~0ull;
    a.trace[5] = 0ull;
  }
  bool go = p2p::wait_for_flags(a.ready_flags, W, -1, epoch, a.limit_ns);
  if (tracer) a.trace[1] = p2p::global_timer_ns();
  if (!go && tid == 0) {
    p2p::report_timeout(a.status);
    atomicExch(a.abort_word, 1u);
  }
  bool fits = true;
  if (go) {
    const int* S = a.sizes;
    for (int e = tid; e < n; e += kThreads) {
      int column = 0, below = 0;
      for (int s = 0; s < W; s++) {
        const int raw = __ldcg(S + s * n + e);
        const int v = raw > 0 ? raw : 0;
        column += v;
        if (s < me) below += v;
        if (a.keep != nullptr && blockIdx.x == 0) a.keep[s * n + e] = raw;
      }
      const int mine = __ldcg(S + me * n + e);
      s_aux[e] = column;
      s_below[e] = below;
      s_loads[e] = mine > 0 ? mine : 0;
      s_zero[e] = 0;
    }
    p2p::block_exclusive_scan(s_aux, n, s_warp);
    bool ok = true;
    if (tid < W) {
      const long long landed = a.stride_rows ? (long long)n * a.stride_rows
                                             : (long long)(s_aux[(tid + 1) * G] - s_aux[tid * G]);
      ok = landed * grain <= a.half_bytes;
    }
    fits = __syncthreads_and(ok) != 0;
    for (int e = tid; e < n; e += kThreads) {
      const int i = e / G, j = e - i * G;
      const long long row0 = a.stride_rows ? (long long)(j * W + me) * a.stride_rows
                                           : (long long)(s_aux[e] - s_aux[i * G] + s_below[e]);
      s_ptr[e] = a.land[i] + row0 * grain;
    }
    __syncthreads();
    // rows of a bucket beyond the cells it gets (s_fill / s_written; the slot is the load)
    rows::setup_fill(a.dense_counts, n, 0, s_loads, s_written, s_fill);
  }
  const bool move = go && fits;
  if (go && !fits && a.strict && blockIdx.x == 0 && tid == 0)
    p2p::report_status(a.status, BRT_ERR_UNSUPPORTED);

  if (tracer) a.trace[3] = p2p::global_timer_ns();
  if (move) {
    const int lane = tid & 31;
    const int warp_in_cta = tid >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + warp_in_cta;
    const int64_t warps = (int64_t)gridDim.x * kWarps;
    const int64_t items = a.cell_num * a.pieces_per_row;
    const V* __restrict__ src = static_cast<const V*>(a.src);
    CopyStage* my = s_stage + warp_in_cta * kStages;
    const unsigned long long evict_first = l2_evict_first_policy();
    rows::MoveArgs m;  // what the shared index-row scan looks at
    m.indices = a.indices;
    m.gates = nullptr;
    m.path_num = n;
    rows::FillPacer pace(items, (int64_t)s_fill[n] * a.pieces_per_row, warp, warps);

    // zero one (empty row of a bucket, 2 KB piece) at its destination
    auto fill_one = [&](int64_t item) {
      const int64_t nth = item / a.pieces_per_row;
      const int piece = (int)(item - nth * a.pieces_per_row);
      int lo = 0, hi = n - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int64_t)s_fill[mid] <= nth) lo = mid; else hi = mid - 1;
      }
      const int64_t row = (int64_t)s_written[lo] + (nth - s_fill[lo]);
      V* dp = reinterpret_cast<V*>(s_ptr[lo] + row * grain);
      const int64_t v0 = (int64_t)piece * kPieceVecs + lane;
#pragma unroll
      for (int u = 0; u < kCopyUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) dp[v] = make_uint4(0u, 0u, 0u, 0u);
      }
    };

    int seat[IV];
    float gate[IV];
    auto fetch = [&](const ItemCursor& c) {
#pragma unroll
      for (int j = 0; j < IV; j++) { seat[j] = 0; gate[j] = 1.f; }
      if (c.cell < a.cell_num) rows::load_index_chunk<IV>(a.indices, c.cell, n, 0, lane, seat);
    };
    auto issue = [&](CopyStage& st, const ItemCursor& c) {
      if (c.cell < a.cell_num) {
        // routes: row = seat - 1 inside the bucket, the path id rides in the gate field
        const int count = rows::build_routes<IV, 0, BRT_BF16, true>(m, c.cell, seat, gate, s_loads,
                                                                    s_zero, st.route, lane,
                                                                    kCopyRoutes);
        if (lane == 0) st.count = count;
        if (count > 0) {
          const int64_t first = (int64_t)c.piece * kPieceVecs;
          const V* sp = src + c.cell * a.row_vecs + first;
#pragma unroll
          for (int u = 0; u < kCopyUnroll; u++) {
            const int v = u * 32 + lane;
            if (first + v < a.row_vecs) cp_async_16_hint(&st.row[v], sp + v, evict_first);
          }
        }
      }
      cp_async_commit();
    };

    // The warp's items: a fixed share (every warps-th item), or, with a work counter, runs of
    // kClaim consecutive items claimed from it, so that a warp whose rows went to a busy link
    // takes fewer and the CTAs finish together.
    constexpr int kClaim = 4;
    int64_t next_static = warp;
    int64_t claimed = 0;
    int claimed_left = 0;
    auto next_item = [&]() -> ItemCursor {
      int64_t item;
      if (a.work_counter == nullptr) {
        item = next_static;
        next_static += warps;
      } else {
        if (claimed_left == 0) {
          unsigned long long base = 0;
          if (lane == 0) base = atomicAdd(a.work_counter, (unsigned long long)kClaim);
          claimed = (int64_t)__shfl_sync(0xffffffffu, base, 0);
          claimed_left = kClaim;
        }
        item = claimed++;
        claimed_left--;
      }
      ItemCursor c;
      if (item < items) {
        c = rows::cursor_at(item, a.pieces_per_row);
      } else {
        c.cell = a.cell_num;
        c.piece = 0;
      }
      return c;
    };
    ItemCursor at = next_item();
    ItemCursor ahead = next_item();
    ItemCursor ahead2 = next_item();
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
          const int e = __float_as_int(slot.gate);
          V* dp = reinterpret_cast<V*>(s_ptr[e] + (int64_t)slot.row * grain) + first + lane;
#pragma unroll
          for (int u = 0; u < kCopyUnroll; u++) {
            if (!full && first + u * 32 + lane >= a.row_vecs) continue;
            dp[u * 32] = regs[u];
          }
        }
        if (count > kCopyRoutes) {
          // more routes than the table holds: walk the index row for the rest (warp-uniform)
          int seen = 0;
          for (int e = 0; e < n; e++) {
            const int s = a.indices[cell * n + e];
            if (s <= 0 || s > s_loads[e]) continue;
            if (seen++ < kCopyRoutes) continue;
            V* dp = reinterpret_cast<V*>(s_ptr[e] + (int64_t)(s - 1) * grain) + first + lane;
#pragma unroll
            for (int u = 0; u < kCopyUnroll; u++) {
              if (!full && first + u * 32 + lane >= a.row_vecs) continue;
              dp[u * 32] = regs[u];
            }
          }
        }
      }
      for (int k = pace.due(); k > 0 && pace.next < pace.end; k--, pace.next += pace.stride)
        fill_one(pace.next);
      __syncwarp();
      at = ahead;
      ahead = ahead2;
      ahead2 = next_item();
      stage ^= 1;
    }
    cp_async_wait<0>();
    for (; pace.next < pace.end; pace.next += pace.stride) fill_one(pace.next);
  }

  // arrive: the last CTA to finish raises my flag at every rank, unless a wait ran out
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
      if (a.work_counter != nullptr) *a.work_counter = 0ull;
      const unsigned int aborted = atomicExch(a.abort_word, 0u);
      __threadfence_system();
      if (aborted == 0u)
        for (int r = 0; r < W; r++) p2p::store_release_sys(a.arrive_flags[r] + me, epoch);
      if (a.trace != nullptr) a.trace[2] = p2p::global_timer_ns();
    }
  }
}

template <int IV>
int launch(const DispatchLandArgs& a, cudaStream_t st) {
  const int n = a.world_size * a.group_size;
  const size_t smem = sizeof(CopyStage) * kWarps * kStages + plan_bytes(n);
  static thread_local int configured_device = -1;
  int dev = 0;
  BRT_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    BRT_CUDA_TRY(cudaFuncSetAttribute(
        dispatch_land_kernel<IV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
        (int)(sizeof(CopyStage) * kWarps * kStages + plan_bytes(p2p::kMaxBuckets))));
    configured_device = dev;
  }
  const KernelTimer timer("dispatch_land_kernel", st);
  dispatch_land_kernel<IV><<<(unsigned)(sm_count() * 3), kThreads, smem, st>>>(a), note_launch();
  BRT_LAUNCH_CHECK("dispatch_land_kernel");
  return BRT_OK;
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API int brt_p2p_dispatch_land(
    const void* src_data, const int32_t* route_indices, const int32_t* dense_counts,
    int64_t cell_num, int64_t row_bytes, const int32_t* size_matrix, int32_t* keep_matrix,
    int world_size, int group_size, int my_rank, int64_t stride_rows, int64_t half_bytes,
    void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
    void* const* peer_arrive_flag_arrays, void* my_done_counter, void* my_abort_word,
    void* status_word, void* host_status_word, uint64_t wait_limit_ns, void* stream) {
  clear_error();
  return p2p_dispatch_land_launch(src_data, route_indices, dense_counts, cell_num, row_bytes,
                                  size_matrix, keep_matrix, world_size, group_size, my_rank,
                                  stride_rows, half_bytes, landing_ptrs, epoch, my_ready_flags,
                                  peer_arrive_flag_arrays, my_done_counter, my_abort_word,
                                  status_word, host_status_word, wait_limit_ns, P2pReplay{},
                                  stream);
}

}  // extern "C"

namespace brt_b200 {
int p2p_dispatch_land_launch(const void* src_data, const int32_t* route_indices,
                             const int32_t* dense_counts, int64_t cell_num, int64_t row_bytes,
                             const int32_t* size_matrix, int32_t* keep_matrix, int world_size,
                             int group_size, int my_rank, int64_t stride_rows,
                             int64_t half_bytes, void* const* landing_ptrs, uint64_t epoch,
                             const void* my_ready_flags, void* const* peer_arrive_flag_arrays,
                             void* my_done_counter, void* my_abort_word, void* status_word,
                             void* host_status_word, uint64_t wait_limit_ns,
                             const P2pReplay& replay, void* stream) {
  BRT_REQUIRE(route_indices != nullptr && dense_counts != nullptr && size_matrix != nullptr &&
                  landing_ptrs != nullptr && my_ready_flags != nullptr &&
                  peer_arrive_flag_arrays != nullptr && my_done_counter != nullptr &&
                  my_abort_word != nullptr && status_word != nullptr,
              "null pointers");
  BRT_REQUIRE(cell_num >= 0 && (cell_num == 0 || src_data != nullptr), "src_data is null");
  BRT_REQUIRE(world_size >= 1 && world_size <= p2p::kMaxRanks && my_rank >= 0 &&
                  my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(group_size >= 1 && (long long)world_size * group_size <= p2p::kMaxBuckets,
              "at most %d buckets per exchange", p2p::kMaxBuckets);
  BRT_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && aligned_to(src_data, 16),
              "rows must be 16-byte multiples and the source 16-byte aligned");
  BRT_REQUIRE(stride_rows >= 0 && half_bytes >= 0, "negative stride or half size");
  DispatchLandArgs a;
  a.src = src_data;
  a.indices = route_indices;
  a.dense_counts = dense_counts;
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / 16;
  a.pieces_per_row = (a.row_vecs + kPieceVecs - 1) / kPieceVecs;
  a.world_size = world_size;
  a.my_rank = my_rank;
  a.group_size = group_size;
  a.stride_rows = stride_rows;
  a.half_bytes = half_bytes;
  a.epoch = epoch;
  a.epoch_counter = static_cast<const unsigned long long*>(replay.epoch_counter);
  a.strict = replay.strict;
  a.trace = static_cast<unsigned long long*>(replay.trace);
  a.work_counter = static_cast<unsigned long long*>(replay.work_counter);
  a.limit_ns = wait_limit_ns;
  a.sizes = size_matrix;
  a.keep = keep_matrix;
  a.ready_flags = static_cast<const unsigned long long*>(my_ready_flags);
  for (int r = 0; r < world_size; r++) {
    BRT_REQUIRE(landing_ptrs[r] != nullptr && aligned_to(landing_ptrs[r], 16),
                "landing half %d is null or not 16-byte aligned", r);
    a.land[r] = static_cast<char*>(landing_ptrs[r]);
    a.arrive_flags[r] = static_cast<unsigned long long*>(peer_arrive_flag_arrays[r]);
  }
  a.done_counter = static_cast<unsigned int*>(my_done_counter);
  a.abort_word = static_cast<unsigned int*>(my_abort_word);
  a.status.device_word = static_cast<int*>(status_word);
  a.status.host_word = static_cast<int*>(host_status_word);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = world_size * group_size;
  if (n % 4 == 0 && aligned_to(route_indices, 16)) return launch<4>(a, st);
  return launch<1>(a, st);
}
}  // namespace brt_b200
