// Host side of the peer-memory sparse exchange: one context per rank that owns the
// bookkeeping of its arena (the exchange counter, which landing half is current, the size
// matrices kept for the inverse exchanges, a pinned landing buffer for the sizes and the
// host-visible status word) and enqueues the kernels of exchange_p2p.cu.
//
// Arena layout (byte offsets):
//   0        32 x uint64  arrival flags                (slot r: raised by rank r)
//   256      32 x uint64  ready flags                  (slot r: last exchange rank r entered)
//   512      uint32       completion counter of this rank's landing kernel
//   516      uint32       abort word of this rank's landing kernel
//   520      uint64       epoch counter: exchanges this rank has opened (device-side count)
//   528      uint64       work counter of this rank's landing kernel (zero between launches)
//   1024     int32        status word of the bounded waits
//   1088     2 x 8 uint64 timing trace of the last forward / inverse landing kernel
//   2048     two size boards of kBoardInts int32 each, used alternately
//   65536    kKept + kKeptReplay size matrices (kBoardInts int32 each) kept for the inverse
//            exchanges; the last kKeptReplay belong to exchanges issued for replay
//   ...      two more size boards, for the exchanges issued for replay
//   kControlBytes ..      two landing halves of half_bytes each
//
// All ranks call the exchanges in the same order, so the exchange counter advances in step
// on every rank.  The host's count selects the landing half and the size board (count & 1)
// and is the identifier under which a forward exchange's size matrix is kept; the epoch of
// the flags is a second count kept on the device, advanced by the kernel that opens an
// exchange, so that it keeps growing when the same kernels run again from a CUDA graph.
//
// Replays.  Between brt_p2p_ctx_replay_begin and _end the caller issues exchanges whose sizes
// stay on the device (brt_p2p_forward_device_sizes instead of brt_p2p_sparse_forward_sizes),
// normally while a CUDA graph is being captured.  Such exchanges use size boards and kept
// matrices of their own, so that replaying them between ordinary exchanges never touches a
// board or a matrix an ordinary exchange still needs; their landing halves are the ones the
// host's count named when they were issued, on every replay.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "exchange_p2p.cuh"

namespace brt_b200 {
namespace {

constexpr int kMaxRanks = 32;
constexpr size_t kFlagsOffset = 0;
constexpr size_t kReadyOffset = 256;
constexpr size_t kCounterOffset = 512;
constexpr size_t kAbortOffset = 516;
constexpr size_t kEpochCounter = 520;
constexpr size_t kWorkCounter = 528;
constexpr size_t kStatusOffset = 1024;
constexpr size_t kTraceOffset = 1088;
constexpr size_t kBoardOffset = 2048;
constexpr size_t kBoardInts = (65536 - kBoardOffset) / 8;
constexpr size_t kKeptOffset = 65536;
constexpr int kKept = 32;
constexpr int kKeptReplay = 16;
constexpr size_t kControlBytes = 2u << 20;
constexpr size_t kReplayBoardOffset = kKeptOffset + (kKept + kKeptReplay) * kBoardInts * 4;
static_assert(kReplayBoardOffset + 2 * kBoardInts * 4 <= kControlBytes,
              "control block too small");
constexpr uint64_t kDefaultWaitNs = 2000000000ull;  // 2 s: a bound on the skew between ranks

struct KeptMatrix {
  uint64_t id = 0;  // 0: empty
  int group = 0;
  int slot = 0;                // which device copy (see kKeptOffset) holds it
  bool device_only = false;    // the host never saw the sizes
  std::vector<int32_t> sizes;  // [world][world * group]
};

}  // namespace
}  // namespace brt_b200

struct brt_p2p_ctx {
  int world = 0, rank = 0;
  char* base = nullptr;
  char* peer[brt_b200::kMaxRanks] = {};
  size_t half_bytes = 0;
  uint64_t exchanges = 0;
  uint64_t wait_ns = brt_b200::kDefaultWaitNs;
  int32_t* pinned = nullptr;       // [0] status word, [1 ..] the gathered size matrix
  int32_t* host_status = nullptr;  // written by kernels whose wait ran out (host view)
  int32_t* host_status_dev = nullptr;  // the same word as the device addresses it
  cudaEvent_t fork = nullptr;
  void* arrive_flags[brt_b200::kMaxRanks] = {};
  void* ready_flags[brt_b200::kMaxRanks] = {};
  brt_b200::KeptMatrix kept[brt_b200::kKept];
  // forward exchange whose sizes have not been read yet
  uint64_t pending = 0;
  int pending_slot = 0;
  size_t pending_board = 0;  // byte offset of its size board in every arena
  bool pending_sizes_on_host = false;  // its SIZES stage was issued
  bool replaying = false;
  uint64_t replay_slots = 0;
  int group = 0, layout = 0;
  int64_t grain = 0, stride = 0;
};

namespace brt_b200 {
namespace {

char* half_of(const brt_p2p_ctx* c, int r, uint64_t exchange) {
  return c->peer[r] + kControlBytes + (exchange & 1) * c->half_bytes;
}

int check_alive(const brt_p2p_ctx* c) {
  if (c->host_status[0] == BRT_ERR_UNSUPPORTED)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "an earlier peer exchange with device-resident sizes carried rows that "
                     "do not fit a landing half (brt_p2p_ctx_reset_status clears this)");
  if (c->host_status[0] != 0)
    return set_error(BRT_ERR_TIMEOUT,
                     "an earlier peer exchange timed out waiting for another rank "
                     "(brt_p2p_ctx_reset_status clears this)");
  return BRT_OK;
}

P2pReplay replay_of(const brt_p2p_ctx* c, bool strict, int trace_slot = -1) {
  P2pReplay r;
  r.epoch_counter = c->base + kEpochCounter;
  r.strict = strict ? 1 : 0;
  if (trace_slot >= 0) r.trace = c->base + kTraceOffset + 64 * trace_slot;
  r.work_counter = c->base + kWorkCounter;
  return r;
}

int32_t* kept_slot(const brt_p2p_ctx* c, int slot) {
  return reinterpret_cast<int32_t*>(c->base + kKeptOffset) + (size_t)slot * kBoardInts;
}

int land(brt_p2p_ctx* c, const void* rows, const int32_t* matrix, int32_t* keep, int group,
         int layout, int zero_tails, int64_t grain, int64_t stride, uint64_t exchange,
         bool strict, void* stream) {
  void* halves[kMaxRanks];
  for (int r = 0; r < c->world; r++) halves[r] = half_of(c, r, exchange);
  return p2p_land_launch(rows, matrix, keep, c->world, group, c->rank, layout, zero_tails, grain,
                         stride, (int64_t)c->half_bytes, halves, exchange,
                         c->base + kReadyOffset, c->arrive_flags, c->base + kCounterOffset,
                         c->base + kAbortOffset, c->base + kStatusOffset, c->host_status_dev,
                         c->wait_ns,
                         replay_of(c, strict,
                                   layout == BRT_P2P_SPARSE_INVERSE || layout == BRT_P2P_SLOTS_BACK),
                         stream);
}

int wait_arrivals(brt_p2p_ctx* c, uint64_t exchange, void* stream) {
  return p2p_wait_launch(c->base + kFlagsOffset, c->world, c->rank, exchange,
                         c->base + kStatusOffset, c->host_status_dev, c->wait_ns,
                         replay_of(c, false), stream);
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API size_t brt_p2p_control_bytes(void) { return kControlBytes; }

BRT_API int brt_p2p_ctx_create(int world_size, int my_rank, void* my_arena,
                               void* const* arenas, size_t half_bytes, brt_p2p_ctx** out) {
  clear_error();
  BRT_REQUIRE(out != nullptr && my_arena != nullptr && arenas != nullptr, "null pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(half_bytes % 256 == 0, "half_bytes must be a multiple of 256");
  brt_p2p_ctx* c = new brt_p2p_ctx();
  c->world = world_size;
  c->rank = my_rank;
  c->base = static_cast<char*>(my_arena);
  c->half_bytes = half_bytes;
  for (int r = 0; r < world_size; r++) {
    c->peer[r] = static_cast<char*>(arenas[r]);
    c->arrive_flags[r] = c->peer[r] + kFlagsOffset;
    c->ready_flags[r] = c->peer[r] + kReadyOffset;
  }
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->pinned), (1 + kBoardInts) * 4,
                                cudaHostAllocDefault);
  if (e == cudaSuccess)
    e = cudaHostAlloc(reinterpret_cast<void**>(&c->host_status), 64, cudaHostAllocMapped);
  if (e == cudaSuccess) {
    memset(c->host_status, 0, 64);
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->host_status_dev), c->host_status, 0);
  }
  if (e == cudaSuccess) {
    e = cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    brt_p2p_ctx_destroy(c);
    return set_error(BRT_ERR_CUDA, "exchange context: %s", cudaGetErrorString(e));
  }
  *out = c;
  return BRT_OK;
}

BRT_API void brt_p2p_ctx_destroy(brt_p2p_ctx* c) {
  if (c == nullptr) return;
  if (c->pinned) cudaFreeHost(c->pinned);
  if (c->host_status) cudaFreeHost(c->host_status);
  if (c->fork) cudaEventDestroy(c->fork);
  delete c;
}

BRT_API int brt_p2p_ctx_set_wait_limit(brt_p2p_ctx* c, uint64_t nanoseconds) {
  clear_error();
  BRT_REQUIRE(c != nullptr && nanoseconds > 0, "bad arguments");
  c->wait_ns = nanoseconds;
  return BRT_OK;
}

BRT_API int brt_p2p_ctx_status(const brt_p2p_ctx* c) {
  return c == nullptr ? BRT_ERR_INVALID_ARGUMENT : c->host_status[0];
}

BRT_API int brt_p2p_ctx_reset_status(brt_p2p_ctx* c) {
  clear_error();
  BRT_REQUIRE(c != nullptr, "null context");
  // Back to the state of a fresh context: after a wait ran out the ranks may have counted
  // different numbers of exchanges, so the flags, both exchange counts and the kept matrices
  // start over.  The flags in this arena are raised by the OTHER ranks: the caller makes sure
  // (a host barrier on either side of this call) that no rank enters an exchange before every
  // rank has reset.
  BRT_CUDA_TRY(cudaDeviceSynchronize());
  BRT_CUDA_TRY(cudaMemset(c->base, 0, kBoardOffset));
  c->host_status[0] = 0;
  c->pending = 0;
  c->exchanges = 0;
  c->replaying = false;
  c->replay_slots = 0;
  for (auto& k : c->kept) k = KeptMatrix();
  return BRT_OK;
}

BRT_API uint64_t brt_p2p_ctx_exchanges(const brt_p2p_ctx* c) { return c ? c->exchanges : 0; }

BRT_API int brt_p2p_ctx_trace(brt_p2p_ctx* c, uint64_t* nanoseconds) {
  clear_error();
  BRT_REQUIRE(c != nullptr && nanoseconds != nullptr, "null pointers");
  BRT_CUDA_TRY(cudaDeviceSynchronize());
  uint64_t t[16];
  BRT_CUDA_TRY(cudaMemcpy(t, c->base + kTraceOffset, sizeof(t), cudaMemcpyDeviceToHost));
  for (int k = 0; k < 2; k++) {
    const uint64_t* s = t + 8 * k;
    uint64_t* o = nanoseconds + 5 * k;
    o[0] = s[1] - s[0];                        // waiting for the other ranks
    o[1] = s[2] - s[1];                        // moving, up to the raised flags
    o[2] = s[3] - s[1];                        // of which: planning (CTA 0)
    o[3] = s[4] > s[1] ? s[4] - s[1] : 0;      // the first CTA leaves its copy loop
    o[4] = s[5] > s[1] ? s[5] - s[1] : 0;      // the last CTA leaves its copy loop
  }
  return BRT_OK;
}

namespace {
// What the PUSH stage of a forward exchange launches: the landing kernel over rows that are
// already laid out by destination, or the dispatch that lands its rows itself.
struct FusedDispatch {
  const void* src;
  const int32_t* indices;
  const int32_t* dense_counts;
  int64_t cell_num;
};

int forward_begin(brt_p2p_ctx* c, const void* rows, const FusedDispatch* fused,
                  const int32_t* sizes, int group_size, int64_t grain_bytes, int64_t stride_rows,
                  int layout, void* main_stream, void* side_stream, int stages) {
  BRT_REQUIRE(c != nullptr && sizes != nullptr, "null context or sizes");
  BRT_REQUIRE(layout == BRT_P2P_SPARSE_FORWARD || (layout == BRT_P2P_SLOTS && stride_rows > 0),
              "layout must be the sparse forward one or slots with a slot size");
  const int n = c->world * group_size;
  BRT_REQUIRE(group_size >= 1 && grain_bytes > 0 && grain_bytes % 16 == 0 && stride_rows >= 0,
              "bad bucket geometry");
  if (n > 1024 || (size_t)c->world * n > kBoardInts)
    return set_error(BRT_ERR_UNSUPPORTED, "%d buckets are too many for the peer exchange", n);
  if (stages == 0) stages = BRT_P2P_STAGE_ALL;
  if (int rc = check_alive(c)) return rc;
  BRT_REQUIRE(!c->replaying || !(stages & BRT_P2P_STAGE_SIZES),
              "exchanges issued for replay keep their sizes on the device "
              "(brt_p2p_forward_device_sizes); the SIZES stage brings them to the host");
  if (stages & BRT_P2P_STAGE_POST) {
    BRT_REQUIRE(c->pending == 0, "the sizes of the previous forward exchange were never read");
    c->exchanges++;
    c->pending = c->exchanges;
    c->pending_slot = c->replaying ? kKept + (int)(c->replay_slots++ % kKeptReplay)
                                   : (int)(c->exchanges % kKept);
    c->pending_sizes_on_host = false;
    c->pending_board = (c->replaying ? kReplayBoardOffset : kBoardOffset) +
                       4 * (c->exchanges & 1) * kBoardInts;
    c->group = group_size;
    c->layout = layout;
    c->grain = grain_bytes;
    c->stride = stride_rows;
    const size_t board = c->pending_board;
    void* boards[kMaxRanks];
    for (int r = 0; r < c->world; r++) boards[r] = c->peer[r] + board;
    if (int rc = p2p_post_launch(sizes, n, c->world, c->rank, c->exchanges, boards,
                                 c->ready_flags, replay_of(c, false), main_stream))
      return rc;
    if (main_stream != side_stream) {
      BRT_CUDA_TRY(cudaEventRecord(c->fork, static_cast<cudaStream_t>(main_stream)));
      BRT_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(side_stream), c->fork, 0));
    }
  }
  BRT_REQUIRE(c->pending != 0 && c->group == group_size && c->grain == grain_bytes &&
                  c->stride == stride_rows && c->layout == layout,
              "stages of one exchange must be issued with the same geometry");
  const uint64_t x = c->pending;
  const size_t board = c->pending_board;
  if (stages & BRT_P2P_STAGE_SIZES) {
    // the sizes reach the host beside the data: a wait on the ready flags (raised by kernels
    // of OTHER GPUs and by my post above), then the board and the status word come down
    cudaStream_t side = static_cast<cudaStream_t>(side_stream);
    if (int rc = p2p_wait_launch(c->base + kReadyOffset, c->world, -1, x,
                                 c->base + kStatusOffset, c->host_status_dev, c->wait_ns,
                                 replay_of(c, false), side_stream))
      return rc;
    BRT_CUDA_TRY(cudaMemcpyAsync(c->pinned, c->base + kStatusOffset, 4, cudaMemcpyDeviceToHost,
                                 side));
    BRT_CUDA_TRY(cudaMemcpyAsync(c->pinned + 1, c->base + board, (size_t)c->world * n * 4,
                                 cudaMemcpyDeviceToHost, side));
    c->pending_sizes_on_host = true;
  }
  if (stages & BRT_P2P_STAGE_PUSH) {
    int32_t* keep = kept_slot(c, c->pending_slot);
    const int32_t* matrix = reinterpret_cast<const int32_t*>(c->base + board);
    const bool strict = (stages & BRT_P2P_STAGE_STRICT) != 0;
    if (fused == nullptr) {
      if (int rc = land(c, rows, matrix, keep, group_size, layout, 0, grain_bytes, stride_rows, x,
                        strict, main_stream))
        return rc;
    } else {
      void* halves[kMaxRanks];
      for (int r = 0; r < c->world; r++) halves[r] = half_of(c, r, x);
      if (int rc = p2p_dispatch_land_launch(
              fused->src, fused->indices, fused->dense_counts, fused->cell_num, grain_bytes,
              matrix, keep, c->world, group_size, c->rank, stride_rows, (int64_t)c->half_bytes,
              halves, x, c->base + kReadyOffset, c->arrive_flags, c->base + kCounterOffset,
              c->base + kAbortOffset, c->base + kStatusOffset, c->host_status_dev, c->wait_ns,
              replay_of(c, strict, 0), main_stream))
        return rc;
    }
  }
  if (stages & BRT_P2P_STAGE_WAIT)
    if (int rc = wait_arrivals(c, x, main_stream)) return rc;
  return BRT_OK;
}
}  // namespace

BRT_API int brt_p2p_sparse_forward_begin(brt_p2p_ctx* c, const void* rows, const int32_t* sizes,
                                         int group_size, int64_t grain_bytes,
                                         int64_t stride_rows, int layout, void* main_stream,
                                         void* side_stream, int stages) {
  clear_error();
  return forward_begin(c, rows, nullptr, sizes, group_size, grain_bytes, stride_rows, layout,
                       main_stream, side_stream, stages);
}

BRT_API int brt_p2p_dispatch_forward_begin(brt_p2p_ctx* c, const void* src_data,
                                           const int32_t* route_indices, const int32_t* loads,
                                           const int32_t* dense_counts, int64_t cell_num,
                                           int64_t row_bytes, int group_size,
                                           int64_t stride_rows, void* main_stream,
                                           void* side_stream, int stages) {
  clear_error();
  BRT_REQUIRE(route_indices != nullptr && dense_counts != nullptr && cell_num >= 0,
              "null indices or counts");
  const FusedDispatch fused{src_data, route_indices, dense_counts, cell_num};
  return forward_begin(c, nullptr, &fused, loads, group_size, row_bytes, stride_rows,
                       BRT_P2P_SPARSE_FORWARD, main_stream, side_stream, stages);
}

BRT_API int brt_p2p_sparse_forward_sizes(brt_p2p_ctx* c, void* side_stream,
                                         const int32_t** size_matrix, int64_t* out_rows,
                                         int* fits, void** out_data, uint64_t* exchange_id) {
  clear_error();
  BRT_REQUIRE(c != nullptr && size_matrix != nullptr && out_rows != nullptr && fits != nullptr &&
                  out_data != nullptr && exchange_id != nullptr,
              "null pointers");
  BRT_REQUIRE(c->pending != 0, "no forward exchange in flight");
  BRT_REQUIRE(c->pending_sizes_on_host,
              "this exchange was issued without BRT_P2P_STAGE_SIZES: its sizes are on the "
              "device only (brt_p2p_forward_device_sizes)");
  BRT_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(side_stream)));
  const uint64_t x = c->pending;
  c->pending = 0;
  if (c->pinned[0] != 0 || c->host_status[0] != 0)
    return set_error(BRT_ERR_TIMEOUT, "peer exchange timed out waiting for another rank");
  const int W = c->world, G = c->group, n = W * G;
  const int32_t* S = c->pinned + 1;  // [sender][destination * G + expert]
  int64_t rows = 0;
  int ok = 1;
  for (int d = 0; d < W; d++) {
    int64_t landed = 0;
    for (int s = 0; s < W; s++)
      for (int j = 0; j < G; j++) landed += S[s * n + d * G + j] > 0 ? S[s * n + d * G + j] : 0;
    if (c->stride) landed = c->stride * n;
    if (d == c->rank) rows = landed;
    if (landed * c->grain > (int64_t)c->half_bytes) ok = 0;
  }
  KeptMatrix& k = c->kept[x % kKept];
  k.id = x;
  k.group = G;
  k.slot = c->pending_slot;
  k.device_only = false;
  k.sizes.assign(S, S + (size_t)W * n);
  *size_matrix = S;
  *out_rows = rows;
  *fits = ok;
  *out_data = half_of(c, c->rank, x);
  *exchange_id = x;
  return BRT_OK;
}

BRT_API int brt_p2p_forward_device_sizes(brt_p2p_ctx* c, int32_t* received_sizes,
                                         void* stream, void** out_data,
                                         int64_t* capacity_rows, uint64_t* exchange_id) {
  clear_error();
  BRT_REQUIRE(c != nullptr && received_sizes != nullptr && out_data != nullptr &&
                  capacity_rows != nullptr && exchange_id != nullptr,
              "null pointers");
  BRT_REQUIRE(c->pending != 0, "no forward exchange in flight");
  const uint64_t x = c->pending;
  const int W = c->world, G = c->group, n = W * G;
  const size_t board = c->pending_board;
  if (int rc = p2p_received_sizes_launch(
          reinterpret_cast<const int32_t*>(c->base + board), W, G, c->rank, x,
          c->base + kReadyOffset, received_sizes, c->base + kStatusOffset, c->host_status_dev,
          c->wait_ns, replay_of(c, false), stream))
    return rc;
  c->pending = 0;
  KeptMatrix& k = c->kept[x % kKept];
  k.id = x;
  k.group = G;
  k.slot = c->pending_slot;
  k.device_only = true;
  k.sizes.clear();
  *out_data = half_of(c, c->rank, x);
  *capacity_rows = c->stride ? c->stride * n : (int64_t)c->half_bytes / c->grain;
  *exchange_id = x;
  return BRT_OK;
}

BRT_API int brt_p2p_ctx_replay_begin(brt_p2p_ctx* c) {
  clear_error();
  BRT_REQUIRE(c != nullptr, "null context");
  BRT_REQUIRE(!c->replaying, "a replay section is already open");
  BRT_REQUIRE(c->pending == 0, "the sizes of the previous forward exchange were never read");
  if (int rc = check_alive(c)) return rc;
  c->replaying = true;
  return BRT_OK;
}

BRT_API int brt_p2p_ctx_replay_end(brt_p2p_ctx* c) {
  clear_error();
  BRT_REQUIRE(c != nullptr && c->replaying, "no replay section is open");
  c->replaying = false;
  BRT_REQUIRE(c->pending == 0, "the sizes of the last forward exchange were never taken");
  return BRT_OK;
}

BRT_API int brt_p2p_sparse_backward(brt_p2p_ctx* c, uint64_t exchange_id, int group_size,
                                    int64_t grain_bytes, int64_t stride_rows, int layout,
                                    int zero_tails, const void* rows, void* main_stream,
                                    int stages, void** out_data, int64_t* out_rows) {
  clear_error();
  BRT_REQUIRE(c != nullptr && out_data != nullptr && out_rows != nullptr, "null pointers");
  BRT_REQUIRE(layout == BRT_P2P_SPARSE_INVERSE || (layout == BRT_P2P_SLOTS_BACK && stride_rows > 0),
              "layout must be the sparse inverse one or slots-back with a slot size");
  BRT_REQUIRE(group_size >= 1 && grain_bytes > 0 && grain_bytes % 16 == 0 && stride_rows >= 0,
              "bad bucket geometry");
  if (stages == 0) stages = BRT_P2P_STAGE_ALL;
  const KeptMatrix& k = c->kept[exchange_id % kKept];
  if (exchange_id == 0 || k.id != exchange_id || k.group != group_size)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "the size matrix of forward exchange %llu is no longer kept",
                     (unsigned long long)exchange_id);
  const int W = c->world, G = group_size, n = W * G;
  const int32_t* S = k.sizes.data();
  // sizes that never reached the host: the output is the landing half as far as rows of
  // this size go, and the landing kernel itself reports rows that do not fit
  int64_t mine = stride_rows ? stride_rows * n : (int64_t)c->half_bytes / grain_bytes;
  for (int i = 0; i < W && !k.device_only; i++) {
    int64_t total = 0;
    for (int b = 0; b < n; b++) total += S[i * n + b] > 0 ? S[i * n + b] : 0;
    if (stride_rows) total = stride_rows * n;
    if (i == c->rank) mine = total;
    if (total * grain_bytes > (int64_t)c->half_bytes)
      return set_error(BRT_ERR_UNSUPPORTED, "the returned rows do not fit a landing half");
  }
  if (int rc = check_alive(c)) return rc;
  if (stages & BRT_P2P_STAGE_POST) {
    BRT_REQUIRE(c->pending == 0, "the sizes of the previous forward exchange were never read");
    c->exchanges++;
    if (int rc = p2p_post_launch(nullptr, 0, c->world, c->rank, c->exchanges, nullptr,
                                 c->ready_flags, replay_of(c, false), main_stream))
      return rc;
  }
  const uint64_t x = c->exchanges;
  if (stages & BRT_P2P_STAGE_PUSH) {
    if (int rc = land(c, rows, kept_slot(c, k.slot), nullptr, G, layout, zero_tails,
                      grain_bytes, stride_rows, x, k.device_only, main_stream))
      return rc;
  }
  if (stages & BRT_P2P_STAGE_WAIT)
    if (int rc = wait_arrivals(c, x, main_stream)) return rc;
  *out_data = half_of(c, c->rank, x);
  *out_rows = mine;
  return BRT_OK;
}

BRT_API int brt_p2p_combine_backward(brt_p2p_ctx* c, uint64_t exchange_id, int group_size,
                                     int64_t row_bytes, int64_t stride_rows,
                                     int64_t expert_rows_offset, const int32_t* route_indices,
                                     const void* gates, int gates_dtype, int dtype,
                                     int64_t cell_num, void* dst_data, void* main_stream,
                                     int stages) {
  clear_error();
  BRT_REQUIRE(c != nullptr, "null context");
  BRT_REQUIRE(group_size >= 1 && row_bytes > 0 && row_bytes % 16 == 0 && stride_rows >= 0,
              "bad bucket geometry");
  BRT_REQUIRE(expert_rows_offset >= (int64_t)kControlBytes && expert_rows_offset % 16 == 0 &&
                  (size_t)expert_rows_offset < kControlBytes + 2 * c->half_bytes,
              "the expert outputs must lie in the landing halves of the arena, at a 16-byte "
              "aligned offset that is the same on every rank");
  if (stages == 0) stages = BRT_P2P_STAGE_POST | BRT_P2P_STAGE_PUSH | BRT_P2P_STAGE_WAIT;
  const KeptMatrix& k = c->kept[exchange_id % kKept];
  if (exchange_id == 0 || k.id != exchange_id || k.group != group_size)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "the size matrix of forward exchange %llu is no longer kept",
                     (unsigned long long)exchange_id);
  if (int rc = check_alive(c)) return rc;
  if (stages & BRT_P2P_STAGE_POST) {
    BRT_REQUIRE(c->pending == 0, "the sizes of the previous forward exchange were never read");
    c->exchanges++;
    // "my expert outputs are complete": everything enqueued before is ordered by the stream
    if (int rc = p2p_post_launch(nullptr, 0, c->world, c->rank, c->exchanges, nullptr,
                                 c->ready_flags, replay_of(c, false), main_stream))
      return rc;
  }
  const uint64_t x = c->exchanges;
  if (stages & BRT_P2P_STAGE_PUSH) {
    const void* rows_at[kMaxRanks];
    for (int r = 0; r < c->world; r++) rows_at[r] = c->peer[r] + expert_rows_offset;
    if (int rc = p2p_combine_land_launch(
            dst_data, gates, gates_dtype, dtype, route_indices, cell_num, row_bytes,
            kept_slot(c, k.slot), c->world, group_size, c->rank, stride_rows, rows_at, x,
            c->base + kReadyOffset, c->arrive_flags, c->base + kCounterOffset,
            c->base + kAbortOffset, c->base + kStatusOffset, c->host_status_dev, c->wait_ns,
            replay_of(c, false, 1), main_stream))
      return rc;
  }
  if (stages & BRT_P2P_STAGE_WAIT)
    if (int rc = wait_arrivals(c, x, main_stream)) return rc;
  return BRT_OK;
}

}  // extern "C"
