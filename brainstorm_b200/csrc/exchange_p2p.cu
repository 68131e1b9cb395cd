// Expert-parallel exchange over NVLink peer memory.
//
// Every rank owns one "arena": device memory it allocates here and exports to the other
// ranks of the box through CUDA IPC.  A variable-size all-to-all is then
//
//   push    : one kernel copies each of my buckets with 16-byte stores straight to its final
//             row offset inside the destination rank's arena (plain peer stores; no TMA, no
//             multicast), my own bucket included;
//   arrive  : when the last CTA of the push has finished, the kernel raises my flag in every
//             peer's arena (system-scope release);
//   wait    : a second, tiny kernel waits until all peers have raised theirs.  The wait is
//             bounded: after the limit it records a timeout in a status word and returns,
//             it never hangs the GPU.
//
// The arena is used in two halves that alternate from one exchange to the next, which is
// what makes a single arrive/wait per exchange sufficient: a peer can only start writing a
// half again after I have signalled the exchange in between, and that signal is enqueued on
// my stream behind my copy out of that half.
#include <cstdlib>

#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kMaxRanks = 32;
constexpr int kMaxCopies = 96;
constexpr int kThreads = 256;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

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

constexpr long long kChunkBytes = 32768;
constexpr int kWays = 32;  // interleaved runs of the copy list (>= any world size)

__device__ __forceinline__ void store_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
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
    const uint4* s = reinterpret_cast<const uint4*>(src + list.src_offset[c] + at);
    uint4* d = reinterpret_cast<uint4*>(list.dst[c] + at);
    const int vecs = (int)(n >> 4);
    constexpr int kPer = (int)(kChunkBytes / 16 / kThreads);  // 8: the whole chunk in flight
    uint4 r[kPer];
#pragma unroll
    for (int i = 0; i < kPer; i++)
      if (threadIdx.x + i * kThreads < vecs) r[i] = __ldcs(s + threadIdx.x + i * kThreads);
#pragma unroll
    for (int i = 0; i < kPer; i++)
      if (threadIdx.x + i * kThreads < vecs) d[threadIdx.x + i * kThreads] = r[i];
  }
  if (sig.world_size == 0) return;  // plain multi-range copy, nobody to tell
  // arrive: the last CTA to finish raises my flag at every rank
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(sig.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *sig.done_counter = 0;  // ready for the next exchange (stream-ordered)
      __threadfence_system();
      for (int r = 0; r < sig.world_size; r++)
        store_release_sys(sig.peer_flags[r] + sig.my_rank, sig.epoch);
    }
  }
}

// Device-planned push: the bucket sizes are still on the device (the host has not seen them
// yet), so every CTA derives the copy list itself.  Bucket b = (destination rank i, local
// expert j), b = i * group + j, holds sizes[b] rows of `grain` bytes.  The buckets bound for
// rank i are packed back to back at plan.slot[i], the region of rank i's arena that belongs
// to this rank, so no rank needs anybody else's sizes to place its data.  A destination whose
// buckets would not fit its slot, or whose slot pointer is null (this rank itself), is left
// out; the host takes the same decision from the gathered size matrix.
constexpr int kMaxBuckets = 1024;

struct BucketPlan {
  int world_size;
  int group_size;
  long long grain;        // bytes per row, multiple of 16
  long long stride_rows;  // source layout: 0 = packed, else bucket b starts at row b * stride
  long long slot_bytes;
  int expert_begin;  // only buckets whose local expert j is in [expert_begin, expert_end) move
  int expert_end;
  char* slot[kMaxRanks];
};

__global__ void __launch_bounds__(kThreads)
p2p_push_buckets_kernel(const char* __restrict__ src, const int* __restrict__ sizes,
                        const __grid_constant__ BucketPlan plan,
                        const __grid_constant__ SignalList sig) {
  __shared__ long long s_rows[kMaxBuckets + 1];   // exclusive prefix of the bucket rows
  __shared__ long long s_first[kMaxBuckets + 1];  // exclusive prefix of the bucket chunks
  __shared__ long long s_warp[kThreads / 32];
  const int n = plan.world_size * plan.group_size;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  // two block-wide exclusive scans over strips of kThreads buckets
  for (int pass = 0; pass < 2; pass++) {
    long long carry = 0;
    for (int b0 = 0; b0 < n; b0 += kThreads) {
      const int b = b0 + threadIdx.x;
      long long v = 0;
      if (b < n) {
        if (pass == 0) {
          v = sizes[b] > 0 ? sizes[b] : 0;
        } else {
          const int i = b / plan.group_size;
          const long long dest_rows = s_rows[(i + 1) * plan.group_size] - s_rows[i * plan.group_size];
          const int j = b - i * plan.group_size;
          const bool send = plan.slot[i] != nullptr && dest_rows * plan.grain <= plan.slot_bytes &&
                            j >= plan.expert_begin && j < plan.expert_end;
          const long long bytes = (s_rows[b + 1] - s_rows[b]) * plan.grain;
          v = send ? (bytes + kChunkBytes - 1) / kChunkBytes : 0;
        }
      }
      long long incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const long long up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (lane == 31) s_warp[warp] = incl;
      __syncthreads();
      long long before = carry;
      for (int w = 0; w < warp; w++) before += s_warp[w];
      long long strip = 0;
      for (int w = 0; w < kThreads / 32; w++) strip += s_warp[w];
      long long* out = pass == 0 ? s_rows : s_first;
      if (b < n) out[b] = before + incl - v;
      carry += strip;
      __syncthreads();
    }
    if (threadIdx.x == 0) (pass == 0 ? s_rows : s_first)[n] = carry;
    __syncthreads();
  }

  const long long total_chunks = s_first[n];
  const long long run = (total_chunks + kWays - 1) / kWays;
  for (long long k = blockIdx.x; k < run * kWays; k += gridDim.x) {
    const long long chunk = (k % kWays) * run + k / kWays;
    if (chunk >= total_chunks) continue;
    int lo = 0, hi = n - 1;  // last bucket whose first chunk is <= chunk (empty ones skipped)
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_first[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    const int b = lo;
    const int i = b / plan.group_size;
    const long long at = (chunk - s_first[b]) * kChunkBytes;
    long long bytes = (s_rows[b + 1] - s_rows[b]) * plan.grain - at;
    if (bytes > kChunkBytes) bytes = kChunkBytes;
    const long long src_row = plan.stride_rows ? (long long)b * plan.stride_rows : s_rows[b];
    const long long dst_row = s_rows[b] - s_rows[i * plan.group_size];
    const uint4* s = reinterpret_cast<const uint4*>(src + src_row * plan.grain + at);
    uint4* d = reinterpret_cast<uint4*>(plan.slot[i] + dst_row * plan.grain + at);
    const int vecs = (int)(bytes >> 4);
    constexpr int kPer = (int)(kChunkBytes / 16 / kThreads);
    uint4 r[kPer];
#pragma unroll
    for (int u = 0; u < kPer; u++)
      if (threadIdx.x + u * kThreads < vecs) r[u] = __ldcs(s + threadIdx.x + u * kThreads);
#pragma unroll
    for (int u = 0; u < kPer; u++)
      if (threadIdx.x + u * kThreads < vecs) d[threadIdx.x + u * kThreads] = r[u];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(sig.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *sig.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < sig.world_size; r++)
        store_release_sys(sig.peer_flags[r] + sig.my_rank, sig.epoch);
    }
  }
}

// Post `n` int32 values (my bucket sizes) into row `my_rank` of every rank's size board and
// raise my flag there.  One CTA.
struct PostList {
  int world_size;
  int my_rank;
  int n;
  unsigned long long epoch;
  int* peer_board[kMaxRanks];
  unsigned long long* peer_flags[kMaxRanks];
};

__global__ void __launch_bounds__(kThreads)
p2p_post_kernel(const int* __restrict__ values, const __grid_constant__ PostList post) {
  for (int r = 0; r < post.world_size; r++)
    for (int t = threadIdx.x; t < post.n; t += kThreads)
      post.peer_board[r][post.my_rank * post.n + t] = values[t];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0)
    for (int r = 0; r < post.world_size; r++)
      store_release_sys(post.peer_flags[r] + post.my_rank, post.epoch);
}

__global__ void p2p_wait_kernel(const unsigned long long* __restrict__ my_flags, int world_size,
                                int skip_rank, unsigned long long epoch,
                                int* __restrict__ status) {
  const int r = threadIdx.x;
  if (r >= world_size || r == skip_rank) return;
  unsigned long long start = 0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  unsigned int spins = 0;
  while (load_acquire_sys(my_flags + r) < epoch) {
    __nanosleep(200);
    if ((++spins & 255u) == 0) {
      unsigned long long now = 0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - start > kWaitLimitNs) {
        atomicExch(status, BRT_ERR_TIMEOUT);
        return;
      }
    }
  }
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

namespace {
// CTAs per SM of the push kernels.  One per SM already saturates an NVLink direction (about
// 655 GB/s measured at 1, 2, 4 and 8); two leave room for the copy-out kernels that run beside
// a push on the side stream.  BRT_P2P_CTAS_PER_SM overrides it.
int push_ctas_per_sm() {
  const char* v = getenv("BRT_P2P_CTAS_PER_SM");
  const int n = v != nullptr ? atoi(v) : 0;
  return n >= 1 && n <= 8 ? n : 2;
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
  // than a push, but not the whole SM: the next push has to find room beside it
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

BRT_API int brt_p2p_push_buckets(const void* src, const int32_t* sizes, int world_size,
                                 int group_size, int my_rank, int64_t grain_bytes,
                                 int64_t stride_rows, void* const* slot_ptrs, int64_t slot_bytes,
                                 int expert_begin, int expert_end, uint64_t epoch,
                                 void* const* peer_flag_arrays, void* my_done_counter,
                                 void* stream) {
  clear_error();
  // src may be null for a rank that holds no rows (all its sizes are zero)
  BRT_REQUIRE(sizes != nullptr && slot_ptrs != nullptr && peer_flag_arrays != nullptr &&
                  my_done_counter != nullptr,
              "null pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  BRT_REQUIRE(group_size >= 1 && (long long)world_size * group_size <= kMaxBuckets,
              "at most %d buckets per device-planned push", kMaxBuckets);
  BRT_REQUIRE(grain_bytes > 0 && grain_bytes % 16 == 0 && aligned_to(src, 16),
              "rows must be 16-byte multiples and the source 16-byte aligned");
  BRT_REQUIRE(stride_rows >= 0 && slot_bytes >= 0, "negative stride or slot size");
  BucketPlan plan;
  plan.world_size = world_size;
  plan.group_size = group_size;
  plan.grain = grain_bytes;
  plan.stride_rows = stride_rows;
  plan.slot_bytes = slot_bytes;
  plan.expert_begin = expert_begin;
  plan.expert_end = expert_end;
  SignalList sig;
  sig.world_size = world_size;
  sig.my_rank = my_rank;
  sig.epoch = epoch;
  for (int r = 0; r < world_size; r++) {
    BRT_REQUIRE(aligned_to(slot_ptrs[r], 16), "slot %d is not 16-byte aligned", r);
    plan.slot[r] = static_cast<char*>(slot_ptrs[r]);
    sig.peer_flags[r] = static_cast<unsigned long long*>(peer_flag_arrays[r]);
  }
  sig.done_counter = static_cast<unsigned int*>(my_done_counter);
  const KernelTimer timer("p2p_push_buckets_kernel", static_cast<cudaStream_t>(stream));
  p2p_push_buckets_kernel<<<(unsigned)(sm_count() * push_ctas_per_sm()), kThreads, 0,
                            static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(src), sizes, plan, sig), note_launch();
  BRT_LAUNCH_CHECK("p2p_push_buckets_kernel");
  return BRT_OK;
}

BRT_API int brt_p2p_post(const int32_t* values, int n, int world_size, int my_rank,
                         uint64_t epoch, void* const* peer_boards, void* const* peer_flag_arrays,
                         void* stream) {
  clear_error();
  BRT_REQUIRE(values != nullptr && n > 0 && peer_boards != nullptr && peer_flag_arrays != nullptr,
              "bad arguments");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks && my_rank >= 0 && my_rank < world_size,
              "bad rank %d of %d", my_rank, world_size);
  PostList post;
  post.world_size = world_size;
  post.my_rank = my_rank;
  post.n = n;
  post.epoch = epoch;
  for (int r = 0; r < world_size; r++) {
    post.peer_board[r] = static_cast<int*>(peer_boards[r]);
    post.peer_flags[r] = static_cast<unsigned long long*>(peer_flag_arrays[r]);
  }
  p2p_post_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(values, post), note_launch();
  BRT_LAUNCH_CHECK("p2p_post_kernel");
  return BRT_OK;
}

BRT_API int brt_p2p_exchange_sizes(const int32_t* values, int n, int world_size, int my_rank,
                                   uint64_t epoch, void* const* peer_boards,
                                   void* const* peer_flag_arrays, const void* my_flag_array,
                                   const void* my_board, void* status_word, int32_t* host_out,
                                   void* stream) {
  if (int rc = brt_p2p_post(values, n, world_size, my_rank, epoch, peer_boards, peer_flag_arrays,
                            stream))
    return rc;
  if (int rc = brt_p2p_wait(my_flag_array, world_size, -1, epoch, status_word, stream)) return rc;
  BRT_REQUIRE(my_board != nullptr && host_out != nullptr, "null board or host buffer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BRT_CUDA_TRY(cudaMemcpyAsync(host_out, status_word, 4, cudaMemcpyDeviceToHost, st));
  BRT_CUDA_TRY(cudaMemcpyAsync(host_out + 1, my_board, (size_t)world_size * n * 4,
                               cudaMemcpyDeviceToHost, st));
  return BRT_OK;
}

BRT_API int brt_p2p_wait(const void* my_flag_array, int world_size, int skip_rank,
                         uint64_t epoch, void* status_word, void* stream) {
  clear_error();
  BRT_REQUIRE(my_flag_array != nullptr && status_word != nullptr, "null control pointers");
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxRanks, "bad world size %d", world_size);
  const KernelTimer timer("p2p_wait_kernel", static_cast<cudaStream_t>(stream));
  p2p_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(my_flag_array), world_size, skip_rank, epoch,
      static_cast<int*>(status_word)), note_launch();
  BRT_LAUNCH_CHECK("p2p_wait_kernel");
  return BRT_OK;
}

}  // extern "C"
