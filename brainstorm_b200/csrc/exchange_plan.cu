// Host-side planning of the peer-memory sparse exchange: one context per process that owns
// the bookkeeping of its arena (epochs, halves, slots, the pinned landing buffer of the size
// exchange) and turns a size matrix into the copy lists of exchange_p2p.cu.  Everything a
// forward or an inverse exchange enqueues is issued from here in a handful of calls, so the
// host path of an exchange is microseconds, not the sum of dozens of interpreter round trips.
//
// Arena layout (byte offsets inside the control block at the start of an arena):
//   0     32 x uint64  data arrival flags            (slot r: raised by rank r)
//   256   32 x uint64  size-board arrival flags
//   512   uint32       completion counter of this rank's pushes
//   1024  int32        status word of the bounded waits
//   2048  two size boards of BOARD_INTS int32 each, used alternately
// followed at 65536 by two data halves of half_bytes each.
#include <cstdlib>
#include <vector>

#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kMaxRanks = 32;
constexpr int kMaxPhases = 4;
constexpr int kDefaultPhases = 1;
constexpr size_t kControlBytes = 65536;
constexpr size_t kFlagsOffset = 0;
constexpr size_t kSizeFlagsOffset = 256;
constexpr size_t kCounterOffset = 512;
constexpr size_t kStatusOffset = 1024;
constexpr size_t kBoardOffset = 2048;
constexpr size_t kBoardInts = (kControlBytes - kBoardOffset) / 8;
constexpr int kMaxListed = 96;  // ranges per brt_p2p_push call

}  // namespace
}  // namespace brt_b200

struct brt_p2p_ctx {
  int world = 0, rank = 0;
  char* base = nullptr;
  char* peer[brt_b200::kMaxRanks] = {};
  size_t half_bytes = 0, slot_bytes = 0;
  uint64_t epoch = 0, exchanges = 0, size_epoch = 0;
  int32_t* pinned = nullptr;  // [0] status word, [1 ..] the gathered size matrix
  cudaEvent_t fork = nullptr, join = nullptr;
  void* flag_arrays[brt_b200::kMaxRanks] = {};
  void* size_flag_arrays[brt_b200::kMaxRanks] = {};
  // forward exchange in flight
  int group = 0, phases = 0;
  int64_t grain = 0, stride = 0;
  size_t half = 0;
  uint64_t phase_epoch[brt_b200::kMaxPhases] = {};
  int phase_lo[brt_b200::kMaxPhases] = {}, phase_hi[brt_b200::kMaxPhases] = {};
};

namespace brt_b200 {
namespace {

// Pushes per exchange.  With more than one, the copy-out of a range overlaps the transfer of
// the next, but every extra push costs a drain, a flag round and a launch: measured at 2 GPUs
// (268 MB per direction) one push of 418 us becomes four of 535 us in total, more than the
// overlapped copy-out saves, so the default is a single push.
// BRT_P2P_PHASES (1..4) overrides the default for experiments.
int split_phases(int group, int* lo, int* hi) {
  int want = kDefaultPhases;
  if (const char* v = getenv("BRT_P2P_PHASES")) {
    const int n = atoi(v);
    if (n >= 1 && n <= kMaxPhases) want = n;
  }
  const int k = group < want ? group : want;
  int n = 0;
  for (int p = 0; p < k; p++) {
    const int a = (int)((long long)group * p / k), b = (int)((long long)group * (p + 1) / k);
    if (b > a) {
      lo[n] = a;
      hi[n] = b;
      n++;
    }
  }
  return n;
}

struct RangeList {
  std::vector<int64_t> src, bytes;
  std::vector<void*> dst;
  void add(const char* base, const char* from, char* to, int64_t n) {
    if (n <= 0) return;
    src.push_back(from - base);
    dst.push_back(to);
    bytes.push_back(n);
  }
};

// Enqueue `list` (offsets relative to `base`) as flag-less or flagged pushes.
int enqueue(const brt_p2p_ctx* c, const char* base, const RangeList& list, bool raise_flag,
            uint64_t epoch, void* stream) {
  const int n = (int)list.bytes.size();
  if (raise_flag) {
    if (n > kMaxListed) return set_error(BRT_ERR_UNSUPPORTED, "too many buckets for one push");
    return brt_p2p_push(base, n, list.src.data(), list.dst.data(), list.bytes.data(), c->world,
                        c->rank, epoch, const_cast<void* const*>(c->flag_arrays),
                        c->base + kCounterOffset, stream);
  }
  for (int at = 0; at < n; at += kMaxListed) {
    const int m = n - at < kMaxListed ? n - at : kMaxListed;
    if (int rc = brt_p2p_push(base, m, list.src.data() + at, list.dst.data() + at,
                              list.bytes.data() + at, 0, 0, 0, nullptr, nullptr, stream))
      return rc;
  }
  return BRT_OK;
}

int fork_side(brt_p2p_ctx* c, void* main_stream, void* side_stream) {
  BRT_CUDA_TRY(cudaEventRecord(c->fork, static_cast<cudaStream_t>(main_stream)));
  BRT_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(side_stream), c->fork, 0));
  return BRT_OK;
}

int join_side(brt_p2p_ctx* c, void* main_stream, void* side_stream) {
  BRT_CUDA_TRY(cudaEventRecord(c->join, static_cast<cudaStream_t>(side_stream)));
  BRT_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(main_stream), c->join, 0));
  return BRT_OK;
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API int brt_p2p_ctx_create(int world_size, int my_rank, void* my_arena,
                               void* const* arenas, size_t half_bytes, brt_p2p_ctx** out) {
  clear_error();
  BRT_REQUIRE(out != nullptr && my_arena != nullptr && arenas != nullptr, "null pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  brt_p2p_ctx* c = new brt_p2p_ctx();
  c->world = world_size;
  c->rank = my_rank;
  c->base = static_cast<char*>(my_arena);
  c->half_bytes = half_bytes;
  c->slot_bytes = (half_bytes / world_size) & ~(size_t)255;
  for (int r = 0; r < world_size; r++) {
    c->peer[r] = static_cast<char*>(arenas[r]);
    c->flag_arrays[r] = c->peer[r] + kFlagsOffset;
    c->size_flag_arrays[r] = c->peer[r] + kSizeFlagsOffset;
  }
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->pinned), (1 + kBoardInts) * 4,
                                cudaHostAllocDefault);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->join, cudaEventDisableTiming);
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
  if (c->fork) cudaEventDestroy(c->fork);
  if (c->join) cudaEventDestroy(c->join);
  delete c;
}

BRT_API size_t brt_p2p_ctx_slot_bytes(const brt_p2p_ctx* c) { return c ? c->slot_bytes : 0; }

BRT_API int brt_p2p_forward_begin(brt_p2p_ctx* c, const void* rows, const int32_t* sizes,
                                  int group_size, int64_t grain_bytes, int64_t stride_rows,
                                  void* main_stream, void* side_stream) {
  clear_error();
  BRT_REQUIRE(c != nullptr && sizes != nullptr, "null context or sizes");
  const int n = c->world * group_size;
  BRT_REQUIRE(group_size >= 1 && grain_bytes > 0 && grain_bytes % 16 == 0 && stride_rows >= 0,
              "bad bucket geometry");
  if (n > 1024 || (size_t)c->world * n > kBoardInts)
    return set_error(BRT_ERR_UNSUPPORTED, "%d buckets are too many for the peer exchange", n);
  if (int rc = fork_side(c, main_stream, side_stream)) return rc;
  c->exchanges++;
  c->half = kControlBytes + (c->exchanges & 1) * c->half_bytes;
  c->group = group_size;
  c->grain = grain_bytes;
  c->stride = stride_rows;
  c->phases = split_phases(group_size, c->phase_lo, c->phase_hi);
  void* slots[kMaxRanks];
  for (int r = 0; r < c->world; r++)
    slots[r] = r == c->rank ? nullptr : c->peer[r] + c->half + (size_t)c->rank * c->slot_bytes;
  for (int p = 0; p < c->phases; p++) {
    c->phase_epoch[p] = ++c->epoch;
    if (int rc = brt_p2p_push_buckets(rows, sizes, c->world, group_size, c->rank, grain_bytes,
                                      stride_rows, slots, (int64_t)c->slot_bytes, c->phase_lo[p],
                                      c->phase_hi[p], c->phase_epoch[p], c->flag_arrays,
                                      c->base + kCounterOffset, main_stream))
      return rc;
  }
  c->size_epoch++;
  const size_t board = kBoardOffset + 4 * (c->size_epoch & 1) * kBoardInts;
  void* boards[kMaxRanks];
  for (int r = 0; r < c->world; r++) boards[r] = c->peer[r] + board;
  return brt_p2p_exchange_sizes(sizes, n, c->world, c->rank, c->size_epoch, boards,
                                c->size_flag_arrays, c->base + kSizeFlagsOffset,
                                c->base + board, c->base + kStatusOffset, c->pinned, side_stream);
}

BRT_API int brt_p2p_forward_sizes(brt_p2p_ctx* c, void* side_stream, const int32_t** size_matrix,
                                  int64_t* out_rows, int* fits) {
  clear_error();
  BRT_REQUIRE(c != nullptr && size_matrix != nullptr && out_rows != nullptr && fits != nullptr,
              "null pointers");
  BRT_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(side_stream)));
  if (c->pinned[0] != 0)
    return set_error(BRT_ERR_TIMEOUT, "peer exchange timed out waiting for another rank");
  const int W = c->world, G = c->group, n = W * G;
  const int32_t* S = c->pinned + 1;  // [sender][destination * G + expert]
  int64_t rows = 0;
  int ok = 1;
  for (int s = 0; s < W; s++) {
    for (int d = 0; d < W; d++) {
      int64_t pair = 0;
      for (int j = 0; j < G; j++) pair += S[s * n + d * G + j] > 0 ? S[s * n + d * G + j] : 0;
      if (d == c->rank) rows += pair;
      if (s != d && pair * c->grain > (int64_t)c->slot_bytes) ok = 0;
    }
  }
  *size_matrix = S;
  *out_rows = c->stride ? c->stride * n : rows;
  *fits = ok;
  return BRT_OK;
}

BRT_API int brt_p2p_forward_finish(brt_p2p_ctx* c, const void* rows, void* out, void* main_stream,
                                   void* side_stream) {
  clear_error();
  BRT_REQUIRE(c != nullptr && c->phases > 0, "no forward exchange in flight");
  const int W = c->world, G = c->group, n = W * G, me = c->rank;
  const int32_t* S = c->pinned + 1;
  const int64_t grain = c->grain;
  auto count = [&](int s, int d, int j) -> int64_t {
    const int32_t v = S[s * n + d * G + j];
    return v > 0 ? v : 0;
  };
  // where bucket (expert j, source s) starts in my expert-major output
  std::vector<int64_t> start((size_t)n);
  {
    int64_t run = 0;
    for (int j = 0; j < G; j++)
      for (int s = 0; s < W; s++) {
        start[(size_t)j * W + s] = c->stride ? (int64_t)(j * W + s) * c->stride : run;
        run += count(s, me, j);
      }
  }
  const char* x = static_cast<const char*>(rows);
  char* o = static_cast<char*>(out);
  // my own buckets: from the rows I hold to their place, while the pushes are running
  {
    RangeList local;
    int64_t run = 0;
    for (int b = 0; b < n; b++) {
      const int64_t mine = count(me, b / G, b % G);
      if (b / G == me)
        local.add(x, x + (c->stride ? (int64_t)b * c->stride : run) * grain,
                  o + start[(size_t)(b % G) * W + me] * grain, mine * grain);
      run += mine;
    }
    if (int rc = enqueue(c, x, local, false, 0, side_stream)) return rc;
  }
  // what the peers pushed: packed per source in that source's slot of my half
  std::vector<int64_t> in_slot((size_t)n);  // [source][expert] row offset inside the slot
  for (int s = 0; s < W; s++) {
    int64_t run = 0;
    for (int j = 0; j < G; j++) {
      in_slot[(size_t)s * G + j] = run;
      run += count(s, me, j);
    }
  }
  for (int p = 0; p < c->phases; p++) {
    if (int rc = brt_p2p_wait(c->base + kFlagsOffset, W, me, c->phase_epoch[p],
                              c->base + kStatusOffset, side_stream))
      return rc;
    RangeList got;
    for (int j = c->phase_lo[p]; j < c->phase_hi[p]; j++)
      for (int s = 0; s < W; s++) {
        if (s == me) continue;
        got.add(c->base,
                c->base + c->half + (size_t)s * c->slot_bytes + in_slot[(size_t)s * G + j] * grain,
                o + start[(size_t)j * W + s] * grain, count(s, me, j) * grain);
      }
    if (int rc = enqueue(c, c->base, got, false, 0, side_stream)) return rc;
  }
  c->phases = 0;
  return join_side(c, main_stream, side_stream);
}

BRT_API int brt_p2p_backward(brt_p2p_ctx* c, const int32_t* size_matrix, int group_size,
                             int64_t grain_bytes, int64_t stride_rows, const void* rows,
                             void* out, void* main_stream, void* side_stream) {
  clear_error();
  BRT_REQUIRE(c != nullptr && size_matrix != nullptr, "null context or size matrix");
  BRT_REQUIRE(group_size >= 1 && grain_bytes > 0 && grain_bytes % 16 == 0 && stride_rows >= 0,
              "bad bucket geometry");
  const int W = c->world, G = group_size, n = W * G, me = c->rank;
  const int32_t* S = size_matrix;  // [sender of the forward exchange][destination * G + expert]
  auto count = [&](int s, int d, int j) -> int64_t {
    const int32_t v = S[s * n + d * G + j];
    return v > 0 ? v : 0;
  };
  // every rank gets back its own rank-major layout: starts[i][b] of bucket b at rank i
  std::vector<int64_t> starts((size_t)W * n);
  int64_t max_rows = 0;
  for (int i = 0; i < W; i++) {
    int64_t run = 0;
    for (int b = 0; b < n; b++) {
      starts[(size_t)i * n + b] = stride_rows ? (int64_t)b * stride_rows : run;
      run += count(i, b / G, b % G);
    }
    const int64_t total = stride_rows ? stride_rows * n : run;
    if (total > max_rows) max_rows = total;
  }
  if (max_rows * grain_bytes > (int64_t)c->half_bytes)
    return set_error(BRT_ERR_UNSUPPORTED, "the returned rows do not fit an arena half");
  if (int rc = fork_side(c, main_stream, side_stream)) return rc;
  c->exchanges++;
  const size_t half = kControlBytes + (c->exchanges & 1) * c->half_bytes;
  const char* x = static_cast<const char*>(rows);
  char* o = static_cast<char*>(out);
  int lo[kMaxPhases], hi[kMaxPhases];
  const int phases = split_phases(G, lo, hi);
  uint64_t epochs[kMaxPhases];
  // what I hold is expert-major: bucket (j, i) came from rank i for my expert j
  int64_t held_at = 0;
  for (int p = 0; p < phases; p++) {
    RangeList send;
    for (int j = lo[p]; j < hi[p]; j++)
      for (int i = 0; i < W; i++) {
        const int64_t rows_ji = count(i, me, j);
        const int64_t src_row = stride_rows ? (int64_t)(j * W + i) * stride_rows : held_at;
        const int64_t dst_row = starts[(size_t)i * n + me * G + j];
        char* to = i == me ? o + dst_row * grain_bytes
                           : c->peer[i] + half + dst_row * grain_bytes;
        send.add(x, x + src_row * grain_bytes, to, rows_ji * grain_bytes);
        held_at += rows_ji;
      }
    epochs[p] = ++c->epoch;
    if (int rc = enqueue(c, x, send, true, epochs[p], main_stream)) return rc;
  }
  for (int p = 0; p < phases; p++) {
    if (int rc = brt_p2p_wait(c->base + kFlagsOffset, W, me, epochs[p], c->base + kStatusOffset,
                              side_stream))
      return rc;
    RangeList got;
    for (int i = 0; i < W; i++) {
      if (i == me) continue;
      for (int j = lo[p]; j < hi[p]; j++) {
        const int64_t at = starts[(size_t)me * n + i * G + j] * grain_bytes;
        got.add(c->base, c->base + half + at, o + at, count(me, i, j) * grain_bytes);
      }
    }
    if (int rc = enqueue(c, c->base, got, false, 0, side_stream)) return rc;
  }
  return join_side(c, main_stream, side_stream);
}

}  // extern "C"
