// Locality-aware rank reorder: greedy maximum matching on the [receiver, source] load
// matrix of an expert-parallel all-to-all, so that each rank adopts the shard it already
// holds most of.
//
// One CTA.  Thread i owns entry (c, o) = (i / W, i % W); for the grouped form the entry is
// the sum of its G per-expert loads (any G, summed serially - no power-of-two tree).  Each
// of the W rounds is one block-wide arg-max by warp shuffles: larger value wins, equal
// values go to the smaller flat index (the tie rule of the reference's CUB ArgMax).  The
// winner's row and column are retired, reorder[c] = o, and column c of the output becomes
// column o of the input.
#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kMaxWorld = 32;
constexpr int kThreads = 1024;

struct Best {
  int value;
  int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__global__ void __launch_bounds__(kThreads)
rank_match_kernel(const int* __restrict__ loads, int group_size, int world_size,
                  int* __restrict__ reorder_indices, int* __restrict__ reordered_loads) {
  __shared__ Best s_warp[32];
  __shared__ int s_pick;
  __shared__ int s_reorder[kMaxWorld];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int W = world_size;
  const int n = W * W;
  const bool live = tid < n;
  const int my_row = live ? tid / W : -1;
  const int my_col = live ? tid % W : -1;

  int value = -1;
  if (live) {
    int acc = 0;
    for (int g = 0; g < group_size; g++) acc += loads[(int64_t)tid * group_size + g];
    value = acc;
  }
  for (int round = 0; round < W; round++) {
    Best b{live ? value : -2, live ? tid : 0x7fffffff};
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      Best o;
      o.value = __shfl_xor_sync(0xffffffffu, b.value, d);
      o.index = __shfl_xor_sync(0xffffffffu, b.index, d);
      b = better(b, o);
    }
    if (lane == 0) s_warp[warp] = b;
    __syncthreads();
    if (warp == 0) {
      Best c = s_warp[lane];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        Best o;
        o.value = __shfl_xor_sync(0xffffffffu, c.value, d);
        o.index = __shfl_xor_sync(0xffffffffu, c.index, d);
        c = better(c, o);
      }
      if (lane == 0) s_pick = c.index;
    }
    __syncthreads();
    const int pick = s_pick;
    const int c = pick / W;
    const int o = pick % W;
    if (live && (my_row == c || my_col == o)) value = -1;
    if (tid == 0) s_reorder[c] = o;
    __syncthreads();
  }
  // out[r, c, g] = in[r, reorder[c], g]
  const int64_t total = (int64_t)n * group_size;
  for (int64_t i = tid; i < total; i += kThreads) {
    const int g = (int)(i % group_size);
    const int64_t rc = i / group_size;
    const int c = (int)(rc % W);
    const int r = (int)(rc / W);
    reordered_loads[i] = loads[((int64_t)r * W + s_reorder[c]) * group_size + g];
  }
  if (tid < W) reorder_indices[tid] = s_reorder[tid];
}

int launch_match(const int32_t* loads, int group_size, int world_size, int32_t* reorder_indices,
                 int32_t* reordered_loads, void* stream) {
  clear_error();
  BRT_REQUIRE(world_size >= 1 && world_size <= kMaxWorld, "world_size %d outside [1, %d]",
              world_size, kMaxWorld);
  BRT_REQUIRE(group_size >= 1, "group_size must be positive");
  BRT_REQUIRE(loads != nullptr && reorder_indices != nullptr && reordered_loads != nullptr,
              "null pointer argument");
  BRT_REQUIRE(loads != reordered_loads, "reordered_loads must not alias loads");
  rank_match_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      loads, group_size, world_size, reorder_indices, reordered_loads), note_launch();
  BRT_LAUNCH_CHECK("rank_match_kernel");
  return BRT_OK;
}

}  // namespace
}  // namespace brt_b200

extern "C" {

BRT_API int brt_locality_reorder(const int32_t* loads, int world_size, int32_t* reorder_indices,
                                 int32_t* reordered_loads, void* stream) {
  return brt_b200::launch_match(loads, 1, world_size, reorder_indices, reordered_loads, stream);
}

BRT_API int brt_group_locality_reorder(const int32_t* loads, int group_size, int world_size,
                                       int32_t* reorder_indices, int32_t* reordered_loads,
                                       void* stream) {
  return brt_b200::launch_match(loads, group_size, world_size, reorder_indices, reordered_loads,
                                stream);
}

}  // extern "C"
