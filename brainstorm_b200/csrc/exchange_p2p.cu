// Expert-parallel exchange over NVLink peer memory.
//
// Every rank owns one "arena": device memory it allocates here and exports to the other
// ranks of the box through CUDA IPC.  The arena holds a control block (flags, size boards,
// saved size matrices) and two landing halves.  A variable-size all-to-all is then
//
//   post   : a one-CTA kernel writes my bucket sizes into every rank's size board and raises
//            my "ready" flag there.  The flag also tells the peers that everything I enqueued
//            before this exchange has finished, i.e. that the landing half of this exchange
//            may be overwritten;
//   land   : one kernel waits (bounded) for the ready flags, derives from the size matrix
//            where each of my buckets lands in its destination's OUTPUT layout and copies it
//            there with 16-byte stores (plain peer stores; no TMA, no multicast), my own
//            buckets included.  The last CTA to finish raises my arrival flag at every rank;
//   wait   : a tiny kernel waits (bounded) until all peers have raised theirs.
//
// Rows therefore cross each HBM once on the way out and once on the way in: the receiver reads
// its output straight from the landing half, nothing is packed, staged or copied out.  The
// halves alternate from one exchange to the next, so the output of an exchange stays valid
// until its owner enters the second exchange after it.
//
// Every wait is bounded by a wall-clock limit: when it runs out the kernel records
// BRT_ERR_TIMEOUT in the arena's status word and in a host-mapped word, skips its copies
// and returns; it never blocks the GPU.
#include <cstdlib>

#include "exchange_p2p.cuh"

namespace brt_b200 {
namespace {

using namespace p2p;


struct CopyList {
  int count;
  long long src_offset[kMaxCopies];  // bytes from `src`
  char* dst[kMaxCopies];             // absolute destination address (peer or local arena)
  long long bytes[kMaxCopies];       // multiple of 16
  long long first_chunk[kMaxCopies + 1];
};

struct SignalList {
  int world_size;
  int my_rank;
  unsigned long long epoch;
  unsigned long long* peer_flags[kMaxRanks];  // flag array of every rank (index: who raised it)
  unsigned int* done_counter;                 // in my control block
};



// One 32 KB chunk: the whole chunk is in flight (8 loads per thread) before the first store.
__device__ __forceinline__ void copy_chunk(const char* s_bytes, char* d_bytes, long long n) {
  const uint4* s = reinterpret_cast<const uint4*>(s_bytes);
  uint4* d = reinterpret_cast<uint4*>(d_bytes);
  const int vecs = (int)(n >> 4);
  constexpr int kPer = (int)(kChunkBytes / 16 / kThreads);
  uint4 r[kPer];
#pragma unroll
  for (int i = 0; i < kPer; i++)
    if (threadIdx.x + i * kThreads < vecs) r[i] = __ldcs(s + threadIdx.x + i * kThreads);
#pragma unroll
  for (int i = 0; i < kPer; i++)
    if (threadIdx.x + i * kThreads < vecs) d[threadIdx.x + i * kThreads] = r[i];
}

__global__ void __launch_bounds__(kThreads)
p2p_push_kernel(const char* __restrict__ src, const __grid_constant__ CopyList list,
                const __grid_constant__ SignalList sig) {
  // Chunks are visited in kWays interleaved runs of the list, so that at any moment the grid
  // is writing to every destination of the list at once (all links and the local copy busy)
  // rather than finishing one destination before it starts the next.
  const long long total_chunks = list.first_chunk[list.count];
  const long long run = (total_chunks + kWays - 1) / kWays;
  for (long long k = blockIdx.x; k < run * kWays; k += gridDim.x) {
    const long long chunk = (k % kWays) * run + k / kWays;
    if (chunk >= total_chunks) continue;
    int lo = 0, hi = list.count - 1;  // last copy whose first chunk is <= chunk
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (list.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    const int c = lo;
    const long long at = (chunk - list.first_chunk[c]) * kChunkBytes;
    long long n = list.bytes[c] - at;
    if (n > kChunkBytes) n = kChunkBytes;
    copy_chunk(src + list.src_offset[c] + at, list.dst[c] + at, n);
  }
  if (sig.world_size == 0) return;  // plain multi-range copy, nobody to tell
  // arrive: the last CTA to finish raises my flag at every rank
  // (device-scope fence per CTA, one system-scope fence in the last CTA: see p2p_land_kernel)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(sig.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *sig.done_counter = 0;  // ready for the next exchange (stream-ordered)
      __threadfence_system();
      for (int r = 0; r < sig.world_size; r++)
        store_release_sys(sig.peer_flags[r] + sig.my_rank, sig.epoch);
    }
  }
}

// ------------------------------------------------------------------------------- landing
// The size matrix S[s][b] holds the rows rank s sends to global bucket b = i * G + j
// (destination rank i, its local expert j).  Two layouts of rows exist:
//   rank-major   (what a sender holds before the forward exchange and gets back from the
//                 inverse one): bucket b of rank s starts at row sum_{b' < b} S[s][b'];
//   expert-major (what a receiver holds after the forward exchange): at rank i, the rows of
//                 (expert j, source s) start at sum_{j' < j} sum_{s'} S[s'][i*G+j'] +
//                 sum_{s' < s} S[s'][i*G+j].
// With stride_rows != 0 buckets are stride_rows apart instead of back to back.
// layout 1 (sparse forward): my rows are rank-major and land expert-major at their destinations;
// layout 0 (sparse inverse): my rows are expert-major and land rank-major at their owners;
// layout 2 (slots): the padded-slot exchange, an involution: my slot (i, j) lands in rank i's
//          slot (me, j); rows per slot from S[me][i*G+j], stride_rows = the slot size;
// layout 3 (slots back): the same move with the sizes this rank RECEIVED in the slot exchange
//          the matrix belongs to, S[i][me*G+j].
// zero_tails (slot layouts): this rank also zeroes, in its own landing half, the rows of every
// slot beyond what the slot receives.
struct LandArgs {
  int world_size;
  int my_rank;
  int group_size;
  int layout;
  int zero_tails;
  long long grain;        // bytes per row, multiple of 16
  long long stride_rows;  // 0: packed
  long long half_bytes;   // capacity of a landing half
  unsigned long long epoch;
  unsigned long long* trace;                // see P2pReplay
  unsigned long long* work_counter;         // see P2pReplay
  const unsigned long long* epoch_counter;  // see effective_epoch()
  int strict;             // a landing that does not fit is an error (reported), not a verdict
  unsigned long long limit_ns;
  const int* sizes;                         // the matrix [world][world * group] (device)
  int* keep;                                // forward: copy of the matrix kept for the inverse
  const unsigned long long* ready_flags;    // my ready flags (slot r: raised by rank r)
  char* land[kMaxRanks];                    // landing half of every rank for this exchange
  unsigned long long* arrive_flags[kMaxRanks];
  unsigned int* done_counter;
  unsigned int* abort_word;  // set by a CTA whose wait ran out; cleared by the last CTA
  StatusSink status;
};


__global__ void __launch_bounds__(kThreads)
p2p_land_kernel(const char* __restrict__ src, const __grid_constant__ LandArgs a) {
  __shared__ int s_rows[kMaxBuckets];       // rows of my bucket p (p: position in my buffer)
  __shared__ int s_src[kMaxBuckets + 1];    // source row of bucket p
  __shared__ int s_dst[kMaxBuckets];        // landing row of bucket p at its destination
  __shared__ int s_aux[kMaxBuckets + 1];
  __shared__ int s_first[kMaxBuckets + 1];  // exclusive prefix of the chunk counts
  __shared__ int s_base[kMaxRanks];
  __shared__ int s_warp[kThreads / 32];
  const int tid = threadIdx.x;
  const int W = a.world_size, G = a.group_size, me = a.my_rank;
  const int n = W * G;
  const unsigned long long epoch = effective_epoch(a.epoch, a.epoch_counter);
  const bool tracer = a.trace != nullptr && blockIdx.x == 0 && tid == 0;
  if (tracer) {
    a.trace[0] = global_timer_ns();
    a.trace[4] = ~0ull;
    a.trace[5] = 0ull;
  }

  // every rank has entered this exchange: the sizes are on my board and the landing halves
  // may be written
  bool go = wait_for_flags(a.ready_flags, W, -1, epoch, a.limit_ns);
  if (tracer) a.trace[1] = global_timer_ns();
  if (!go) {
    if (tid == 0) {
      report_timeout(a.status);
      atomicExch(a.abort_word, 1u);
    }
  }

  const int* S = a.sizes;
  auto rows_of = [&](int s, int b) -> int {
    const int v = __ldcg(S + s * n + b);
    return v > 0 ? v : 0;
  };
  bool fits = true;
  if (go && a.layout >= 2) {
    // slots: position p == global bucket b = i * G + j, fixed slot size
    for (int b = tid; b < n; b += kThreads) {
      const int i = b / G, j = b - i * G;
      if (a.keep != nullptr && blockIdx.x == 0)
        for (int s = 0; s < W; s++) a.keep[s * n + b] = __ldcg(S + s * n + b);
      int v = a.layout == 2 ? rows_of(me, b) : rows_of(i, me * G + j);
      if (v > a.stride_rows) v = (int)a.stride_rows;
      s_rows[b] = v;
      s_src[b] = (int)((long long)b * a.stride_rows);
      s_dst[b] = (int)((long long)(me * G + j) * a.stride_rows);
      // rows slot b of MY half receives (for the tails): from rank i, its slot (me, j)
      int got = a.layout == 2 ? rows_of(i, me * G + j) : rows_of(me, b);
      if (got > a.stride_rows) got = (int)a.stride_rows;
      s_aux[b] = got;
    }
    fits = (long long)n * a.stride_rows * a.grain <= a.half_bytes;
  } else if (go && a.layout == 1) {
    // position p == global bucket b = i * G + j
    for (int b = tid; b < n; b += kThreads) {
      int column = 0, below = 0;
      for (int s = 0; s < W; s++) {
        const int v = rows_of(s, b);
        column += v;
        if (s < me) below += v;
        if (a.keep != nullptr && blockIdx.x == 0) a.keep[s * n + b] = __ldcg(S + s * n + b);
      }
      const int mine = rows_of(me, b);
      s_aux[b] = column;
      s_dst[b] = below;
      s_rows[b] = mine;
      s_src[b] = mine;
    }
    block_exclusive_scan(s_aux, n, s_warp);
    block_exclusive_scan(s_src, n, s_warp);
    bool ok = true;
    if (tid < W) {
      const long long landed = a.stride_rows ? (long long)n * a.stride_rows
                                             : (long long)(s_aux[(tid + 1) * G] - s_aux[tid * G]);
      ok = landed * a.grain <= a.half_bytes;
    }
    fits = __syncthreads_and(ok) != 0;
    for (int b = tid; b < n; b += kThreads) {
      const int i = b / G, j = b - i * G;
      if (a.stride_rows) {
        s_dst[b] = (int)((long long)(j * W + me) * a.stride_rows);
        s_src[b] = (int)((long long)b * a.stride_rows);
      } else {
        s_dst[b] = s_aux[b] - s_aux[i * G] + s_dst[b];
      }
    }
  } else if (go) {
    // position p = j * W + i: the rows of my expert j that came from rank i
    for (int r = tid >> 5; r < W; r += kThreads / 32) {  // rows rank r sent to ranks below me
      int acc = 0;
      for (int b = tid & 31; b < me * G; b += 32) acc += rows_of(r, b);
#pragma unroll
      for (int d = 16; d != 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
      if ((tid & 31) == 0) s_base[r] = acc;
    }
    for (int p = tid; p < n; p += kThreads) {
      const int j = p / W, i = p - j * W;
      const int v = rows_of(i, me * G + j);
      s_rows[p] = v;
      s_src[p] = v;
      s_aux[i * G + j] = v;
    }
    block_exclusive_scan(s_aux, n, s_warp);
    block_exclusive_scan(s_src, n, s_warp);
    for (int p = tid; p < n; p += kThreads) {
      const int j = p / W, i = p - j * W;
      if (a.stride_rows) {
        s_dst[p] = (int)((long long)(me * G + j) * a.stride_rows);
        s_src[p] = (int)((long long)p * a.stride_rows);
      } else {
        s_dst[p] = s_base[i] + s_aux[i * G + j] - s_aux[i * G];
      }
    }
  }
  __syncthreads();
  const bool move = go && fits;
  if (go && !fits && a.strict && blockIdx.x == 0 && tid == 0)
    report_status(a.status, BRT_ERR_UNSUPPORTED);
  for (int p = tid; p < n; p += kThreads) {
    const long long bytes = (long long)s_rows[p] * a.grain;
    s_first[p] = move ? (int)((bytes + kChunkBytes - 1) / kChunkBytes) : 0;
  }
  if (!go) {
    for (int p = tid; p <= n; p += kThreads) s_first[p] = 0;
    __syncthreads();
  } else {
    block_exclusive_scan(s_first, n, s_warp);
  }

  if (tracer) a.trace[3] = global_timer_ns();
  const long long total_chunks = go ? s_first[n] : 0;
  const long long run = (total_chunks + kWays - 1) / kWays;
  // one 32 KB chunk of the list, by position k in the interleaved order
  auto copy_kth = [&](long long k) {
    const long long chunk = (k % kWays) * run + k / kWays;
    if (chunk >= total_chunks) return;
    int lo = 0, hi = n - 1;  // last bucket whose first chunk is <= chunk (empty ones skipped)
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_first[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    const int p = lo;
    const int dest = a.layout == 0 ? p % W : p / G;
    const long long at = (chunk - s_first[p]) * kChunkBytes;
    long long bytes = (long long)s_rows[p] * a.grain - at;
    if (bytes > kChunkBytes) bytes = kChunkBytes;
    copy_chunk(src + (long long)s_src[p] * a.grain + at,
               a.land[dest] + (long long)s_dst[p] * a.grain + at, bytes);
  };
  if (a.work_counter == nullptr) {
    for (long long k = blockIdx.x; k < run * kWays; k += gridDim.x) copy_kth(k);
  } else {
    // Chunks are handed out one at a time from a counter: a CTA whose chunks went to a busy
    // link simply takes fewer.  The claim of the next chunk is in flight during the copy.
    __shared__ unsigned long long s_claim[2];
    if (tid == 0) s_claim[0] = atomicAdd(a.work_counter, 1ull);
    __syncthreads();
    for (int turn = 0;; turn ^= 1) {
      const long long k = (long long)s_claim[turn];
      if (k >= run * kWays) break;
      if (tid == 0) s_claim[turn ^ 1] = atomicAdd(a.work_counter, 1ull);
      copy_kth(k);
      __syncthreads();
    }
  }

  if (move && a.layout >= 2 && a.zero_tails) {
    // the rows of my own slots that nobody writes (the peers only write rows below s_aux[b])
    __syncthreads();
    for (int b = tid; b < n; b += kThreads) {
      const long long bytes = (a.stride_rows - s_aux[b]) * a.grain;
      s_first[b] = (int)((bytes + kChunkBytes - 1) / kChunkBytes);
    }
    block_exclusive_scan(s_first, n, s_warp);
    const long long tail_chunks = s_first[n];
    for (long long chunk = blockIdx.x; chunk < tail_chunks; chunk += gridDim.x) {
      int lo = 0, hi = n - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_first[mid] <= chunk) lo = mid; else hi = mid - 1;
      }
      const int b = lo;
      const long long at = (chunk - s_first[b]) * kChunkBytes;
      long long bytes = (a.stride_rows - s_aux[b]) * a.grain - at;
      if (bytes > kChunkBytes) bytes = kChunkBytes;
      uint4* d = reinterpret_cast<uint4*>(a.land[me] +
                                          ((long long)b * a.stride_rows + s_aux[b]) * a.grain + at);
      const int vecs = (int)(bytes >> 4);
      for (int v = tid; v < vecs; v += kThreads) d[v] = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  // arrive: the last CTA to finish raises my flag at every rank, unless a wait ran out
  if (a.trace != nullptr) {
    __syncthreads();
    if (tid == 0) {
      const unsigned long long now = global_timer_ns();
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
      *a.done_counter = 0;  // ready for the next exchange (stream-ordered)
      if (a.work_counter != nullptr) *a.work_counter = 0ull;
      const unsigned int aborted = atomicExch(a.abort_word, 0u);
      __threadfence_system();
      if (aborted == 0u)
        for (int r = 0; r < W; r++) store_release_sys(a.arrive_flags[r] + me, epoch);
      if (a.trace != nullptr) a.trace[2] = global_timer_ns();
    }
  }
}

// Post `n` int32 values (my bucket sizes; n may be 0) into row `my_rank` of every rank's size
// board and raise my flag there.  One CTA.
struct PostList {
  int world_size;
  int my_rank;
  int n;
  unsigned long long epoch;
  unsigned long long* epoch_counter;  // advanced here: this kernel opens the exchange
  int* peer_board[kMaxRanks];
  unsigned long long* peer_flags[kMaxRanks];
};

__global__ void __launch_bounds__(kThreads)
p2p_post_kernel(const int* __restrict__ values, const __grid_constant__ PostList post) {
  unsigned long long epoch = post.epoch;
  if (post.epoch_counter != nullptr) {  // read by thread 0 only: no other thread needs it
    if (threadIdx.x == 0) {
      epoch = *post.epoch_counter + 1;
      *post.epoch_counter = epoch;
    }
  }
  for (int r = 0; r < post.world_size; r++)
    for (int t = threadIdx.x; t < post.n; t += kThreads)
      post.peer_board[r][post.my_rank * post.n + t] = values[t];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // cumulative over the barrier: the board rows of every thread
    for (int r = 0; r < post.world_size; r++)
      store_release_sys(post.peer_flags[r] + post.my_rank, epoch);
  }
}

__global__ void __launch_bounds__(32)
p2p_wait_kernel(const unsigned long long* __restrict__ my_flags, int world_size, int skip_rank,
                unsigned long long epoch, const unsigned long long* epoch_counter,
                unsigned long long limit_ns, const StatusSink status) {
  if (!wait_for_flags(my_flags, world_size, skip_rank, effective_epoch(epoch, epoch_counter),
                      limit_ns) &&
      threadIdx.x == 0)
    report_timeout(status);
}

// The rows this rank receives, in the order of its landed output: [expert j][source rank s].
__global__ void __launch_bounds__(kThreads)
p2p_received_sizes_kernel(const int* __restrict__ board, int world_size, int group_size,
                          int my_rank, const unsigned long long* __restrict__ ready_flags,
                          unsigned long long epoch, const unsigned long long* epoch_counter,
                          unsigned long long limit_ns, int* __restrict__ out_loads,
                          const StatusSink status) {
  const int n = world_size * group_size;
  const bool go = wait_for_flags(ready_flags, world_size, -1,
                                 effective_epoch(epoch, epoch_counter), limit_ns);
  if (!go && threadIdx.x == 0) report_timeout(status);
  for (int p = threadIdx.x; p < n; p += kThreads) {
    const int j = p / world_size, s = p - j * world_size;
    const int v = go ? __ldcg(board + s * n + my_rank * group_size + j) : 0;
    out_loads[p] = v > 0 ? v : 0;
  }
}


}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

namespace {
// CTAs per SM of the push kernels.  One per SM already saturates an NVLink direction (about
// 655 GB/s measured at 1, 2, 4 and 8); two leave room for kernels that run beside a push on
// another stream.  BRT_P2P_CTAS_PER_SM overrides it (read once).
int push_ctas_per_sm() {
  static const int chosen = [] {
    const char* v = getenv("BRT_P2P_CTAS_PER_SM");
    const int n = v != nullptr ? atoi(v) : 0;
    return n >= 1 && n <= 8 ? n : 2;
  }();
  return chosen;
}
}  // namespace

extern "C" {

BRT_API int brt_p2p_alloc(size_t bytes, void** dev_ptr, void* ipc_handle_out) {
  clear_error();
  BRT_REQUIRE(dev_ptr != nullptr && ipc_handle_out != nullptr && bytes > 0, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == BRT_P2P_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  BRT_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) memcpy(ipc_handle_out, &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    cudaFree(p);
    return set_error(BRT_ERR_CUDA, "exporting the arena failed: %s", cudaGetErrorString(e));
  }
  *dev_ptr = p;
  return BRT_OK;
}

BRT_API int brt_p2p_open(const void* ipc_handle, void** peer_ptr) {
  clear_error();
  BRT_REQUIRE(ipc_handle != nullptr && peer_ptr != nullptr, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  BRT_CUDA_TRY(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return BRT_OK;
}

BRT_API int brt_p2p_close(void* peer_ptr) {
  clear_error();
  BRT_CUDA_TRY(cudaIpcCloseMemHandle(peer_ptr));
  return BRT_OK;
}

BRT_API int brt_p2p_free(void* dev_ptr) {
  clear_error();
  BRT_CUDA_TRY(cudaFree(dev_ptr));
  return BRT_OK;
}

BRT_API int brt_p2p_push(const void* src, int copy_count, const int64_t* src_offsets,
                         void* const* dst_ptrs, const int64_t* bytes, int world_size,
                         int my_rank, uint64_t epoch, void* const* peer_flag_arrays,
                         void* my_done_counter, void* stream) {
  clear_error();
  BRT_REQUIRE(copy_count >= 0 && copy_count <= kMaxCopies, "at most %d copies per push",
              kMaxCopies);
  BRT_REQUIRE(world_size >= 0 && world_size <= kMaxRanks &&
                  (world_size == 0 || (my_rank >= 0 && my_rank < world_size)),
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(world_size == 0 || (peer_flag_arrays != nullptr && my_done_counter != nullptr),
              "null control pointers");
  CopyList list;
  list.count = copy_count;
  long long chunks = 0;
  for (int i = 0; i < copy_count; i++) {
    BRT_REQUIRE(bytes[i] >= 0 && bytes[i] % 16 == 0 && src_offsets[i] % 16 == 0 &&
                    aligned_to(dst_ptrs[i], 16),
                "copy %d is not 16-byte aligned", i);
    list.src_offset[i] = src_offsets[i];
    list.dst[i] = static_cast<char*>(dst_ptrs[i]);
    list.bytes[i] = bytes[i];
    list.first_chunk[i] = chunks;
    chunks += (bytes[i] + kChunkBytes - 1) / kChunkBytes;
  }
  list.first_chunk[copy_count] = chunks;
  BRT_REQUIRE(copy_count == 0 || aligned_to(src, 16), "source is not 16-byte aligned");
  SignalList sig;
  sig.world_size = world_size;
  sig.my_rank = my_rank;
  sig.epoch = epoch;
  for (int r = 0; r < world_size; r++)
    sig.peer_flags[r] = static_cast<unsigned long long*>(peer_flag_arrays[r]);
  sig.done_counter = static_cast<unsigned int*>(my_done_counter);
  long long grid = chunks;
  // a flag-less call is a local copy, bound by HBM rather than by a link; it gets more CTAs
  // than a push, but not the whole SM
  const long long cap = (long long)sm_count() * (world_size == 0 ? 4 : push_ctas_per_sm());
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  const KernelTimer timer(world_size == 0 ? "p2p_copy_kernel" : "p2p_push_kernel",
                          static_cast<cudaStream_t>(stream));
  p2p_push_kernel<<<(unsigned)grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(src), list, sig), note_launch();
  BRT_LAUNCH_CHECK("p2p_push_kernel");
  return BRT_OK;
}

BRT_API int brt_p2p_land(const void* rows, const int32_t* size_matrix, int32_t* keep_matrix,
                         int world_size, int group_size, int my_rank, int layout,
                         int zero_tails, int64_t grain_bytes, int64_t stride_rows,
                         int64_t half_bytes,
                         void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
                         void* const* peer_arrive_flag_arrays, void* my_done_counter,
                         void* my_abort_word, void* status_word, void* host_status_word,
                         uint64_t wait_limit_ns, void* stream) {
  clear_error();
  return p2p_land_launch(rows, size_matrix, keep_matrix, world_size, group_size, my_rank, layout,
                         zero_tails, grain_bytes, stride_rows, half_bytes, landing_ptrs, epoch,
                         my_ready_flags, peer_arrive_flag_arrays, my_done_counter, my_abort_word,
                         status_word, host_status_word, wait_limit_ns, P2pReplay{}, stream);
}

}  // extern "C"

namespace brt_b200 {
int p2p_land_launch(const void* rows, const int32_t* size_matrix, int32_t* keep_matrix,
                    int world_size, int group_size, int my_rank, int layout, int zero_tails,
                    int64_t grain_bytes, int64_t stride_rows, int64_t half_bytes,
                    void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
                    void* const* peer_arrive_flag_arrays, void* my_done_counter,
                    void* my_abort_word, void* status_word, void* host_status_word,
                    uint64_t wait_limit_ns, const P2pReplay& replay, void* stream) {
  // rows may be null for a rank that holds no rows (all its sizes are zero)
  BRT_REQUIRE(size_matrix != nullptr && landing_ptrs != nullptr && my_ready_flags != nullptr &&
                  peer_arrive_flag_arrays != nullptr && my_done_counter != nullptr &&
                  my_abort_word != nullptr && status_word != nullptr,
              "null pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(group_size >= 1 && (long long)world_size * group_size <= kMaxBuckets,
              "at most %d buckets per exchange", kMaxBuckets);
  BRT_REQUIRE(grain_bytes > 0 && grain_bytes % 16 == 0 && aligned_to(rows, 16),
              "rows must be 16-byte multiples and the source 16-byte aligned");
  BRT_REQUIRE(stride_rows >= 0 && half_bytes >= 0, "negative stride or half size");
  BRT_REQUIRE(layout >= BRT_P2P_SPARSE_INVERSE && layout <= BRT_P2P_SLOTS_BACK,
              "unknown layout %d", layout);
  BRT_REQUIRE(layout < BRT_P2P_SLOTS || stride_rows > 0, "the slot layouts need a slot size");
  BRT_REQUIRE(stride_rows * (int64_t)world_size * group_size <= 0x7fffffffLL,
              "more than 2^31-1 rows per rank");
  LandArgs a;
  a.world_size = world_size;
  a.my_rank = my_rank;
  a.group_size = group_size;
  a.layout = layout;
  a.zero_tails = zero_tails != 0;
  a.grain = grain_bytes;
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
  const KernelTimer timer(layout == BRT_P2P_SPARSE_INVERSE ? "p2p_land_backward_kernel"
                          : layout == BRT_P2P_SPARSE_FORWARD ? "p2p_land_forward_kernel"
                                                             : "p2p_land_slots_kernel",
                          static_cast<cudaStream_t>(stream));
  p2p_land_kernel<<<(unsigned)(sm_count() * push_ctas_per_sm()), kThreads, 0,
                    static_cast<cudaStream_t>(stream)>>>(static_cast<const char*>(rows), a),
      note_launch();
  BRT_LAUNCH_CHECK("p2p_land_kernel");
  return BRT_OK;
}

int p2p_post_launch(const int32_t* values, int n, int world_size, int my_rank, uint64_t epoch,
                    void* const* peer_boards, void* const* peer_flag_arrays,
                    const P2pReplay& replay, void* stream) {
  BRT_REQUIRE(n >= 0 && (n == 0 || (values != nullptr && peer_boards != nullptr)) &&
                  peer_flag_arrays != nullptr,
              "bad arguments");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  PostList post;
  post.world_size = world_size;
  post.my_rank = my_rank;
  post.n = n;
  post.epoch = epoch;
  post.epoch_counter = static_cast<unsigned long long*>(replay.epoch_counter);
  for (int r = 0; r < world_size; r++) {
    post.peer_board[r] = n > 0 ? static_cast<int*>(peer_boards[r]) : nullptr;
    post.peer_flags[r] = static_cast<unsigned long long*>(peer_flag_arrays[r]);
  }
  const KernelTimer timer("p2p_post_kernel", static_cast<cudaStream_t>(stream));
  p2p_post_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(values, post), note_launch();
  BRT_LAUNCH_CHECK("p2p_post_kernel");
  return BRT_OK;
}

int p2p_wait_launch(const void* my_flag_array, int world_size, int skip_rank, uint64_t epoch,
                    void* status_word, void* host_status_word, uint64_t wait_limit_ns,
                    const P2pReplay& replay, void* stream) {
  BRT_REQUIRE(my_flag_array != nullptr && status_word != nullptr, "null control pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks, "bad world size %d", world_size);
  StatusSink sink;
  sink.device_word = static_cast<int*>(status_word);
  sink.host_word = static_cast<int*>(host_status_word);
  const KernelTimer timer("p2p_wait_kernel", static_cast<cudaStream_t>(stream));
  p2p_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(my_flag_array), world_size, skip_rank, epoch,
      static_cast<const unsigned long long*>(replay.epoch_counter), wait_limit_ns, sink),
      note_launch();
  BRT_LAUNCH_CHECK("p2p_wait_kernel");
  return BRT_OK;
}

int p2p_received_sizes_launch(const int32_t* board, int world_size, int group_size, int my_rank,
                              uint64_t epoch, const void* my_ready_flags, int32_t* out_loads,
                              void* status_word, void* host_status_word, uint64_t wait_limit_ns,
                              const P2pReplay& replay, void* stream) {
  BRT_REQUIRE(board != nullptr && my_ready_flags != nullptr && out_loads != nullptr &&
                  status_word != nullptr,
              "null pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size &&
                  group_size >= 1 && (long long)world_size * group_size <= kMaxBuckets,
              "bad geometry");
  StatusSink sink;
  sink.device_word = static_cast<int*>(status_word);
  sink.host_word = static_cast<int*>(host_status_word);
  const KernelTimer timer("p2p_received_sizes_kernel", static_cast<cudaStream_t>(stream));
  p2p_received_sizes_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      board, world_size, group_size, my_rank,
      static_cast<const unsigned long long*>(my_ready_flags), epoch,
      static_cast<const unsigned long long*>(replay.epoch_counter), wait_limit_ns, out_loads,
      sink), note_launch();
  BRT_LAUNCH_CHECK("p2p_received_sizes_kernel");
  return BRT_OK;
}
}  // namespace brt_b200

extern "C" {

BRT_API int brt_p2p_post(const int32_t* values, int n, int world_size, int my_rank,
                         uint64_t epoch, void* const* peer_boards, void* const* peer_flag_arrays,
                         void* stream) {
  clear_error();
  return p2p_post_launch(values, n, world_size, my_rank, epoch, peer_boards, peer_flag_arrays,
                         P2pReplay{}, stream);
}

BRT_API int brt_p2p_wait(const void* my_flag_array, int world_size, int skip_rank,
                         uint64_t epoch, void* status_word, void* host_status_word,
                         uint64_t wait_limit_ns, void* stream) {
  clear_error();
  return p2p_wait_launch(my_flag_array, world_size, skip_rank, epoch, status_word,
                         host_status_word, wait_limit_ns, P2pReplay{}, stream);
}

}  // extern "C"
