// Device-side building blocks of the peer-memory exchange kernels: system-scope flag
// accesses, bounded waits that report to the host, and a block-wide scan.
#pragma once

#include "common.cuh"

namespace brt_b200 {
namespace p2p {

constexpr int kMaxRanks = 32;
constexpr int kMaxCopies = 96;
constexpr int kMaxBuckets = 1024;
constexpr int kThreads = 256;
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
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The epoch of an exchange: the `epoch` argument for callers that count exchanges themselves,
// else the value of a counter in the rank's own arena that the post kernel (the first kernel
// of every exchange) advances.  A device-side count keeps growing when kernels with fixed
// arguments run again, i.e. when exchanges are replayed from a CUDA graph.
__device__ __forceinline__ unsigned long long effective_epoch(unsigned long long epoch,
                                                              const unsigned long long* counter) {
  return counter != nullptr ? __ldcg(counter) : epoch;
}

// Where a bounded wait reports that it ran out: the arena's status word and a word of
// host-mapped memory that the host can read without synchronising with the device.
struct StatusSink {
  int* device_word;
  int* host_word;
};
__device__ __forceinline__ void report_status(const StatusSink& s, int code) {
  if (s.device_word != nullptr) atomicExch(s.device_word, code);
  if (s.host_word != nullptr) {
    *reinterpret_cast<volatile int*>(s.host_word) = code;
    __threadfence_system();
  }
}
__device__ __forceinline__ void report_timeout(const StatusSink& s) {
  report_status(s, BRT_ERR_TIMEOUT);
}

// Thread r of the CTA (r < world_size, r != skip) polls flags[r] until it holds a value
// >= epoch or `limit_ns` has passed.  Returns true (to every thread) when all flags came.
__device__ __forceinline__ bool wait_for_flags(const unsigned long long* flags, int world_size,
                                               int skip, unsigned long long epoch,
                                               unsigned long long limit_ns) {
  bool ok = true;
  const int r = threadIdx.x;
  if (r < world_size && r != skip) {
    const unsigned long long start = global_timer_ns();
    unsigned int spins = 0;
    while (load_acquire_sys(flags + r) < epoch) {
      __nanosleep(100);
      if ((++spins & 63u) == 0 && global_timer_ns() - start > limit_ns) {
        ok = false;
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// In-place exclusive prefix sum of a[0 .. n) in shared memory (n <= kMaxBuckets), total at
// a[n].  All threads of the CTA call it; it opens and closes with a barrier.
__device__ __forceinline__ void block_exclusive_scan(int* a, int n, int* s_warp) {
  __syncthreads();
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int per = (n + kThreads - 1) / kThreads;
  const int begin = tid * per < n ? tid * per : n;
  const int end = begin + per < n ? begin + per : n;
  int local = 0;
  for (int i = begin; i < end; i++) local += a[i];
  int incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int before = 0, total = 0;
  for (int w = 0; w < kThreads / 32; w++) {
    if (w < warp) before += s_warp[w];
    total += s_warp[w];
  }
  int run = before + incl - local;
  for (int i = begin; i < end; i++) {
    const int v = a[i];
    a[i] = run;
    run += v;
  }
  if (tid == 0) a[n] = total;
  __syncthreads();
}

}  // namespace p2p

// What the exchange context adds to the public low-level entry points: the arena's epoch
// counter (see effective_epoch), and `strict` (a landing that does not fit its half reports
// BRT_ERR_UNSUPPORTED through the status words instead of leaving the verdict to the host).
struct P2pReplay {
  void* epoch_counter = nullptr;
  int strict = 0;
  // six uint64 of %globaltimer (ns) the landing kernel leaves behind: CTA 0 entered, CTA 0
  // saw every rank ready, the last CTA finished (flags raised), CTA 0 had its plan, the
  // first and the last CTA left their copy loops.  Null: no trace.
  void* trace = nullptr;
  // a uint64 in the rank's own arena, zero between launches: the landing kernels hand out
  // their work items from it (warps and CTAs that finish early take more) instead of
  // giving every warp a fixed share.  Null: fixed shares.
  void* work_counter = nullptr;
};
int p2p_land_launch(const void* rows, const int32_t* size_matrix, int32_t* keep_matrix,
                    int world_size, int group_size, int my_rank, int layout, int zero_tails,
                    int64_t grain_bytes, int64_t stride_rows, int64_t half_bytes,
                    void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
                    void* const* peer_arrive_flag_arrays, void* my_done_counter,
                    void* my_abort_word, void* status_word, void* host_status_word,
                    uint64_t wait_limit_ns, const P2pReplay& replay, void* stream);
int p2p_post_launch(const int32_t* values, int n, int world_size, int my_rank, uint64_t epoch,
                    void* const* peer_boards, void* const* peer_flag_arrays,
                    const P2pReplay& replay, void* stream);
int p2p_wait_launch(const void* my_flag_array, int world_size, int skip_rank, uint64_t epoch,
                    void* status_word, void* host_status_word, uint64_t wait_limit_ns,
                    const P2pReplay& replay, void* stream);
int p2p_dispatch_land_launch(const void* src_data, const int32_t* route_indices,
                             const int32_t* dense_counts, int64_t cell_num, int64_t row_bytes,
                             const int32_t* size_matrix, int32_t* keep_matrix, int world_size,
                             int group_size, int my_rank, int64_t stride_rows,
                             int64_t half_bytes, void* const* landing_ptrs, uint64_t epoch,
                             const void* my_ready_flags, void* const* peer_arrive_flag_arrays,
                             void* my_done_counter, void* my_abort_word, void* status_word,
                             void* host_status_word, uint64_t wait_limit_ns,
                             const P2pReplay& replay, void* stream);
// Combine that pulls its rows from the arenas of the ranks hosting the experts (the inverse
// exchange and the combine in one kernel); `expert_rows[i]` is where rank i's expert output
// starts, laid out as the forward exchange landed it, `size_matrix` is that exchange's.
int p2p_combine_land_launch(void* dst_data, const void* gates, int gates_dtype, int dtype,
                            const int32_t* route_indices, int64_t cell_num, int64_t row_bytes,
                            const int32_t* size_matrix, int world_size, int group_size,
                            int my_rank, int64_t stride_rows, const void* const* expert_rows,
                            uint64_t epoch, const void* my_ready_flags,
                            void* const* peer_arrive_flag_arrays, void* my_done_counter,
                            void* my_abort_word, void* status_word, void* host_status_word,
                            uint64_t wait_limit_ns, const P2pReplay& replay, void* stream);
// out_loads[j * world + s] = rows rank s sends to my expert j in the exchange whose sizes are
// on `board`, once every rank's ready flag shows the exchange (bounded wait).
int p2p_received_sizes_launch(const int32_t* board, int world_size, int group_size, int my_rank,
                              uint64_t epoch, const void* my_ready_flags, int32_t* out_loads,
                              void* status_word, void* host_status_word, uint64_t wait_limit_ns,
                              const P2pReplay& replay, void* stream);

}  // namespace brt_b200
