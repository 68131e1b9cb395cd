// Route-mask -> seat/tag indices, per-path loads, hot-mask throttling and index-format
// conversion for sm_100a.
//
// The reference runs one CTA per path that walks its column of the [cell, path] mask
// 1024 cells at a time.  Here the mask is streamed exactly once, tile by tile, by as
// many CTAs as there are tiles:
//
//   pack   : each thread owns 32 consecutive cells of V adjacent paths.  It reads them
//            with V*4-byte loads (a warp covers whole rows, so the stream is coalesced),
//            sums them and squeezes them into one 32-bit word per path (bit r = cell r
//            is routed).  Words go to a scratch array that is 1/32 of the mask and stays
//            in L2; per-tile column sums go to a second, tiny array.
//   scan   : one small launch turns the per-tile sums into exclusive prefixes and applies
//            the capacity rules to the column totals (loads / throttle prefix).
//   expand : each thread re-reads its word from L2, finds its offset inside the tile with
//            one block-level scan of the popcounts, and writes 32 rows of V indices.
//
// HBM traffic is one read of the mask and one write of the indices; nothing spins or
// waits on another CTA.  Masks holding values other than 0/1 are detected during `pack`
// and make `expand` re-read the mask instead of the bit words, so the integer semantics
// of the reference (index = running sum * mask value) hold for any int32 mask.
#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kGroupRows = 32;  // cells per bit word

enum class Mode { kSeat, kTag, kThrottle };

// How a [cell, path] int32 matrix is cut into CTA tiles.
struct Tiling {
  int vec;            // paths per thread (1, 2 or 4)
  int col_groups;     // path_num / vec
  int cgb;            // column groups handled by one CTA
  int col_chunks;     // CTAs along the path axis
  int slices;         // 32-cell groups per CTA
  int64_t num_groups; // ceil(cell_num / 32)
  int64_t num_tiles;  // ceil(num_groups / slices)
};

Tiling make_tiling(int64_t cell_num, int path_num, bool aligned16, bool aligned8) {
  Tiling t;
  t.vec = 1;
  if (path_num % 4 == 0 && aligned16)
    t.vec = 4;
  else if (path_num % 2 == 0 && aligned8)
    t.vec = 2;
  t.col_groups = path_num / t.vec;
  t.cgb = t.col_groups < kThreads ? t.col_groups : kThreads;
  t.col_chunks = (t.col_groups + t.cgb - 1) / t.cgb;
  t.slices = kThreads / t.cgb;
  t.num_groups = (cell_num + kGroupRows - 1) / kGroupRows;
  t.num_tiles = (t.num_groups + t.slices - 1) / t.slices;
  return t;
}

// Scratch layout: [flags: 64 ints][tile sums: num_tiles*path_num ints][bits: num_groups*path_num]
struct Scratch {
  int* flags;
  int* tile_sums;
  uint32_t* bits;
};

size_t scratch_bytes_for(int64_t cell_num, int path_num) {
  // Sized for the smallest tile (vec = 1 gives the same group count; slices is smallest when
  // cgb is largest), so any alignment of the caller's pointers fits.
  const int64_t groups = (cell_num + kGroupRows - 1) / kGroupRows;
  int cgb_max = path_num < kThreads ? path_num : kThreads;
  int slices_min = kThreads / (cgb_max > 0 ? cgb_max : 1);
  if (slices_min < 1) slices_min = 1;
  // vec > 1 only makes slices larger (fewer tiles); bound with vec = 4 as well
  int64_t tiles_max = (groups + slices_min - 1) / slices_min + 1;
  size_t bytes = 256;
  bytes += round_up((size_t)tiles_max * (size_t)path_num * 4, 256);
  bytes += round_up((size_t)(groups + 1) * (size_t)path_num * 4, 256);
  return bytes;
}

Scratch carve(void* base, const Tiling& t, int path_num) {
  Scratch s;
  char* p = static_cast<char*>(base);
  s.flags = reinterpret_cast<int*>(p);
  p += 256;
  s.tile_sums = reinterpret_cast<int*>(p);
  p += round_up((size_t)t.num_tiles * (size_t)path_num * 4, 256);
  s.bits = reinterpret_cast<uint32_t*>(p);
  return s;
}

template <int V>
__device__ __forceinline__ void load_vec(const int* p, int (&out)[V]) {
  if constexpr (V == 4) {
    const int4 v = __ldcs(reinterpret_cast<const int4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else if constexpr (V == 2) {
    const int2 v = __ldcs(reinterpret_cast<const int2*>(p));
    out[0] = v.x; out[1] = v.y;
  } else {
    out[0] = __ldcs(p);
  }
}

// Same, through the normal cache path (for small arrays expected to sit in L2).
template <int V>
__device__ __forceinline__ void load_vec_cached(const int* p, int (&out)[V]) {
  if constexpr (V == 4) {
    const int4 v = *reinterpret_cast<const int4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else if constexpr (V == 2) {
    const int2 v = *reinterpret_cast<const int2*>(p);
    out[0] = v.x; out[1] = v.y;
  } else {
    out[0] = *p;
  }
}

template <int V>
__device__ __forceinline__ void store_vec(int* p, const int (&v)[V]) {
  if constexpr (V == 4) {
    __stcs(reinterpret_cast<int4*>(p), make_int4(v[0], v[1], v[2], v[3]));
  } else if constexpr (V == 2) {
    __stcs(reinterpret_cast<int2*>(p), make_int2(v[0], v[1]));
  } else {
    __stcs(p, v[0]);
  }
}

template <int V>
__device__ __forceinline__ void store_vec_cached(int* p, const int (&v)[V]) {
  if constexpr (V == 4) {
    *reinterpret_cast<int4*>(p) = make_int4(v[0], v[1], v[2], v[3]);
  } else if constexpr (V == 2) {
    *reinterpret_cast<int2*>(p) = make_int2(v[0], v[1]);
  } else {
    *p = v[0];
  }
}

// ---------------------------------------------------------------------------------- pack
template <int V>
__global__ void __launch_bounds__(kThreads)
mask_pack_kernel(const int* __restrict__ mask, uint32_t* __restrict__ bits,
                 int* __restrict__ tile_sums, int* __restrict__ flags, int64_t cell_num,
                 int path_num, int cgb, int slices) {
  __shared__ int s_sum[kThreads * V];
  const int tid = threadIdx.x;
  const int g_local = tid % cgb;
  const int s = tid / cgb;
  const int col_groups = path_num / V;
  const int g = blockIdx.y * cgb + g_local;
  const bool active = (s < slices) && (g < col_groups);
  for (int i = tid; i < cgb * V; i += kThreads) s_sum[i] = 0;
  __syncthreads();

  const int64_t tile = blockIdx.x;
  const int64_t group = tile * slices + s;
  const int64_t row0 = group * kGroupRows;
  if (active && row0 < cell_num) {
    uint32_t w[V];
    int sum[V];
    bool nonbinary = false;
#pragma unroll
    for (int j = 0; j < V; j++) { w[j] = 0u; sum[j] = 0; }
    const int* p = mask + row0 * path_num + (int64_t)g * V;
    const int64_t left = cell_num - row0;
    const int nrows = left < kGroupRows ? (int)left : kGroupRows;
    if (nrows == kGroupRows) {
#pragma unroll 8
      for (int r = 0; r < kGroupRows; r++) {
        int m[V];
        load_vec<V>(p + (int64_t)r * path_num, m);
#pragma unroll
        for (int j = 0; j < V; j++) {
          sum[j] += m[j];
          w[j] |= (m[j] != 0 ? 1u : 0u) << r;
          nonbinary |= (static_cast<unsigned>(m[j]) > 1u);
        }
      }
    } else {
      for (int r = 0; r < nrows; r++) {
        int m[V];
        load_vec<V>(p + (int64_t)r * path_num, m);
#pragma unroll
        for (int j = 0; j < V; j++) {
          sum[j] += m[j];
          w[j] |= (m[j] != 0 ? 1u : 0u) << r;
          nonbinary |= (static_cast<unsigned>(m[j]) > 1u);
        }
      }
    }
    int wi[V];
#pragma unroll
    for (int j = 0; j < V; j++) wi[j] = static_cast<int>(w[j]);
    store_vec_cached<V>(reinterpret_cast<int*>(bits) + group * path_num + (int64_t)g * V, wi);
#pragma unroll
    for (int j = 0; j < V; j++)
      if (sum[j] != 0) atomicAdd(&s_sum[g_local * V + j], sum[j]);
    if (nonbinary) atomicOr(flags, 1);
  }
  __syncthreads();
  for (int i = tid; i < cgb * V; i += kThreads) {
    const int col = blockIdx.y * cgb * V + i;
    if (col < path_num) tile_sums[tile * path_num + col] = s_sum[i];
  }
}

// ---------------------------------------------------------------------------------- scan
// Capacity rules of the reference's generate_indices_and_loads kernel.
__device__ __forceinline__ int map_load(int real, int col, const int* __restrict__ caps,
                                        int ncap, bool capacity_padding, bool path_wise) {
  if (capacity_padding && path_wise) return caps[col];
  if (real == 0) return 0;
  if (capacity_padding) {
    for (int i = 0; i < ncap; i++)
      if (real <= caps[i]) return caps[i];
    return caps[ncap - 1];
  }
  if (ncap == 0) return real;
  for (int i = 0; i < ncap; i++)
    if (real <= caps[i]) return real;
  return caps[ncap - 1];
}

// One CTA of 32 warps per 32 paths; lane = path, warp = a contiguous range of tiles.
// tile_sums is rewritten in place with the exclusive prefix of each tile (plus the
// throttle prefix in throttle mode).
template <bool THROTTLE>
__global__ void __launch_bounds__(1024)
tile_scan_kernel(int* __restrict__ tile_sums, int64_t num_tiles, int path_num,
                 int* __restrict__ loads, const int* __restrict__ caps, int ncap,
                 int capacity_padding, int path_wise, int* __restrict__ prefix,
                 const int* __restrict__ threshold) {
  __shared__ int s_part[32][33];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  const bool valid = col < path_num;
  const int64_t chunk = (num_tiles + 31) / 32;
  const int64_t t0 = warp * chunk;
  const int64_t t1 = (t0 + chunk) < num_tiles ? (t0 + chunk) : num_tiles;
  int acc = 0;
  if (valid)
    for (int64_t t = t0; t < t1; t++) acc += tile_sums[t * path_num + col];
  s_part[warp][lane] = acc;
  // read before the barrier: the last warp overwrites prefix[col] at the end
  int start = 0;
  if (THROTTLE && valid) start = prefix[col];
  __syncthreads();
  int run = 0;
  for (int w = 0; w < warp; w++) run += s_part[w][lane];
  if (valid) {
    for (int64_t t = t0; t < t1; t++) {
      const int v = tile_sums[t * path_num + col];
      tile_sums[t * path_num + col] = run + start;
      run += v;
    }
  }
  if (warp == 31 && valid) {
    // run now holds the column total (warps past the last tile own an empty range)
    if (THROTTLE) {
      const int thr = threshold[col];
      const int p = start + run;
      prefix[col] = p >= thr ? thr : p;
    } else {
      loads[col] = map_load(run, col, caps, ncap, capacity_padding != 0, path_wise != 0);
    }
  }
}

// ---------------------------------------------------------------------------------- expand
// Exclusive prefix of `cnt` over the slices of one CTA (same column group), in shared memory.
template <int V>
__device__ __forceinline__ void slice_exclusive_scan(int (&cnt)[V], int (&excl)[V], int cgb,
                                                     int slices, int s, bool active,
                                                     int* buf /*[2][kThreads*V]*/) {
  const int tid = threadIdx.x;
  int* in = buf;
  int* out = buf + kThreads * V;
#pragma unroll
  for (int j = 0; j < V; j++) in[tid * V + j] = active ? cnt[j] : 0;
  for (int d = 1; d < slices; d <<= 1) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < V; j++) {
      int x = in[tid * V + j];
      if (s >= d && s < slices) x += in[(tid - d * cgb) * V + j];
      out[tid * V + j] = x;
    }
    int* tmp = in; in = out; out = tmp;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < V; j++) excl[j] = in[tid * V + j] - (active ? cnt[j] : 0);
  __syncthreads();
}

template <int V, Mode MODE>
__global__ void __launch_bounds__(kThreads)
index_expand_kernel(const int* __restrict__ mask, const uint32_t* __restrict__ bits,
                    const int* __restrict__ tile_prefix, const int* __restrict__ flags,
                    int* __restrict__ out, const int* __restrict__ threshold, int64_t cell_num,
                    int path_num, int cgb, int slices) {
  __shared__ int s_buf[2 * kThreads * V];
  const int tid = threadIdx.x;
  const int g_local = tid % cgb;
  const int s = tid / cgb;
  const int col_groups = path_num / V;
  const int g = blockIdx.y * cgb + g_local;
  const int64_t tile = blockIdx.x;
  const int64_t group = tile * slices + s;
  const int64_t row0 = group * kGroupRows;
  const bool active = (s < slices) && (g < col_groups) && (row0 < cell_num);
  const bool general = (flags[0] & 1) != 0;  // mask holds values other than 0/1
  const int64_t col0 = (int64_t)g * V;
  const int64_t left = cell_num - row0;
  const int nrows = !active ? 0 : (left < kGroupRows ? (int)left : kGroupRows);

  uint32_t w[V];
  int cnt[V];
#pragma unroll
  for (int j = 0; j < V; j++) { w[j] = 0u; cnt[j] = 0; }
  if (active) {
    if (!general) {
      int wi[V];
      load_vec_cached<V>(reinterpret_cast<const int*>(bits) + group * path_num + col0, wi);
#pragma unroll
      for (int j = 0; j < V; j++) { w[j] = static_cast<uint32_t>(wi[j]); cnt[j] = __popc(w[j]); }
    } else {
      const int* p = mask + row0 * path_num + col0;
      for (int r = 0; r < nrows; r++) {
        int m[V];
        load_vec_cached<V>(p + (int64_t)r * path_num, m);
#pragma unroll
        for (int j = 0; j < V; j++) cnt[j] += m[j];
      }
    }
  }
  int run[V];
  slice_exclusive_scan<V>(cnt, run, cgb, slices, s, active, s_buf);
  if (!active) return;
  {
    int base[V];
    load_vec_cached<V>(tile_prefix + tile * path_num + col0, base);
#pragma unroll
    for (int j = 0; j < V; j++) run[j] += base[j];
  }
  int thr[V];
  if constexpr (MODE == Mode::kThrottle) load_vec_cached<V>(threshold + col0, thr);

  const int* mp = mask + row0 * path_num + col0;
  int* op = out + row0 * path_num + col0;
#pragma unroll 4
  for (int r = 0; r < kGroupRows; r++) {
    if (r >= nrows) break;
    int m[V];
    if (!general) {
#pragma unroll
      for (int j = 0; j < V; j++) m[j] = (w[j] >> r) & 1u;
    } else {
      load_vec_cached<V>(mp + (int64_t)r * path_num, m);
    }
    int v[V];
#pragma unroll
    for (int j = 0; j < V; j++) {
      run[j] += m[j];
      if constexpr (MODE == Mode::kThrottle) {
        v[j] = (m[j] == 1 && run[j] <= thr[j]) ? 1 : 0;
      } else {
        v[j] = run[j] * m[j];
      }
    }
    if constexpr (MODE == Mode::kTag) {
#pragma unroll
      for (int j = 0; j < V; j++) {
        if (v[j] != 0) {
          const int64_t dst_row = (int64_t)v[j] - 1;
          if (dst_row >= 0 && dst_row < cell_num)
            out[dst_row * path_num + col0 + j] = (int)(row0 + r + 1);
        }
      }
    } else {
      store_vec<V>(op + (int64_t)r * path_num, v);
    }
  }
}

// ---------------------------------------------------------------------------------- convert
__global__ void __launch_bounds__(kThreads)
seat_to_tag_kernel(const int* __restrict__ seat, int* __restrict__ tag, int64_t cell_num,
                   int path_num) {
  const int64_t n = cell_num * path_num;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int sidx = seat[i];
    if (sidx != 0) {
      const int64_t cell = i / path_num;
      const int e = (int)(i - cell * path_num);
      const int64_t r = (int64_t)sidx - 1;
      if (r >= 0 && r < cell_num) tag[r * path_num + e] = (int)(cell + 1);
    }
  }
}

// The reference's tag->seat kernel runs 1024 threads per path; a thread walks rows
// lane, lane+1024, ... below the path's load and stops at its first zero tag.  To keep
// that visible behaviour, a row r is converted only if no row r-1024, r-2048, ... of the
// same path holds a zero tag.
__global__ void __launch_bounds__(kThreads)
tag_to_seat_kernel(const int* __restrict__ tag, int* __restrict__ seat,
                   const int* __restrict__ loads, int64_t cell_num, int path_num) {
  const int64_t lanes = 1024;
  const int64_t n = lanes * path_num;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t lane = i / path_num;
    const int e = (int)(i - lane * path_num);
    const int64_t load = loads[e];
    for (int64_t r = lane; r < load; r += lanes) {
      // rows at or beyond cell_num do not exist in the [cell_num, path_num] array
      if (r >= cell_num) break;
      const int t = tag[r * path_num + e];
      if (t == 0) break;
      const int64_t cell = (int64_t)t - 1;
      if (cell >= 0 && cell < cell_num) seat[cell * path_num + e] = (int)(r + 1);
    }
  }
}

template <int V>
int launch_scan(Mode mode, const Tiling& tl, const Scratch& sc, const int32_t* mask,
                int32_t* out, int32_t* loads, int64_t cell_num, int path_num,
                const int32_t* caps, int ncap, int capacity_padding, int path_wise,
                int32_t* prefix, const int32_t* threshold, cudaStream_t stream) {
  BRT_CUDA_TRY(cudaMemsetAsync(sc.flags, 0, 256, stream));
  const dim3 grid((unsigned)tl.num_tiles, (unsigned)tl.col_chunks);
  mask_pack_kernel<V><<<grid, kThreads, 0, stream>>>(mask, sc.bits, sc.tile_sums, sc.flags,
                                                     cell_num, path_num, tl.cgb, tl.slices);
  BRT_LAUNCH_CHECK("mask_pack_kernel");
  const unsigned scan_grid = (unsigned)((path_num + 31) / 32);
  if (mode == Mode::kThrottle) {
    tile_scan_kernel<true><<<scan_grid, 1024, 0, stream>>>(
        sc.tile_sums, tl.num_tiles, path_num, nullptr, nullptr, 0, 0, 0, prefix, threshold);
  } else {
    tile_scan_kernel<false><<<scan_grid, 1024, 0, stream>>>(
        sc.tile_sums, tl.num_tiles, path_num, loads, caps, ncap, capacity_padding, path_wise,
        nullptr, nullptr);
  }
  BRT_LAUNCH_CHECK("tile_scan_kernel");
  switch (mode) {
    case Mode::kSeat:
      index_expand_kernel<V, Mode::kSeat><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, nullptr, cell_num, path_num, tl.cgb,
          tl.slices);
      break;
    case Mode::kTag:
      BRT_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)cell_num * path_num * 4, stream));
      index_expand_kernel<V, Mode::kTag><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, nullptr, cell_num, path_num, tl.cgb,
          tl.slices);
      break;
    case Mode::kThrottle:
      index_expand_kernel<V, Mode::kThrottle><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, threshold, cell_num, path_num, tl.cgb,
          tl.slices);
      break;
  }
  BRT_LAUNCH_CHECK("index_expand_kernel");
  return BRT_OK;
}

int run_scan(Mode mode, const int32_t* mask, int32_t* out, int32_t* loads, int64_t cell_num,
             int path_num, const int32_t* caps, int ncap, int capacity_padding, int path_wise,
             int32_t* prefix, const int32_t* threshold, void* scratch, size_t scratch_bytes,
             cudaStream_t stream) {
  BRT_REQUIRE(scratch != nullptr && aligned_to(scratch, 256),
              "scratch must be a 256-byte aligned device buffer");
  const size_t need = scratch_bytes_for(cell_num, path_num);
  if (scratch_bytes < need)
    return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                     scratch_bytes, need);
  const bool a16 = aligned_to(mask, 16) && aligned_to(out, 16) &&
                   (threshold == nullptr || aligned_to(threshold, 16));
  const bool a8 = aligned_to(mask, 8) && aligned_to(out, 8) &&
                  (threshold == nullptr || aligned_to(threshold, 8));
  const Tiling tl = make_tiling(cell_num, path_num, a16, a8);
  BRT_REQUIRE(tl.num_tiles <= 0x7fffffffLL && tl.col_chunks <= 65535,
              "mask of %lld x %d cells is too large for one launch", (long long)cell_num,
              path_num);
  const Scratch sc = carve(scratch, tl, path_num);
  switch (tl.vec) {
    case 4:
      return launch_scan<4>(mode, tl, sc, mask, out, loads, cell_num, path_num, caps, ncap,
                            capacity_padding, path_wise, prefix, threshold, stream);
    case 2:
      return launch_scan<2>(mode, tl, sc, mask, out, loads, cell_num, path_num, caps, ncap,
                            capacity_padding, path_wise, prefix, threshold, stream);
    default:
      return launch_scan<1>(mode, tl, sc, mask, out, loads, cell_num, path_num, caps, ncap,
                            capacity_padding, path_wise, prefix, threshold, stream);
  }
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API size_t brt_index_scratch_bytes(int64_t cell_num, int path_num) {
  if (cell_num < 0 || path_num <= 0) return 256;
  return scratch_bytes_for(cell_num, path_num);
}

BRT_API int brt_generate_indices_and_loads(const int32_t* hot_mask, int32_t* indices,
                                           int32_t* loads, int64_t cell_num, int path_num,
                                           const int32_t* supported_capacities,
                                           int supported_capacity_num, int capacity_padding,
                                           int path_wise_padding, int is_tag_index,
                                           void* scratch, size_t scratch_bytes, void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  BRT_REQUIRE(loads != nullptr, "loads is null");
  BRT_REQUIRE(supported_capacity_num >= 0 &&
                  (supported_capacity_num == 0 || supported_capacities != nullptr),
              "supported_capacities is null but supported_capacity_num=%d",
              supported_capacity_num);
  // the reference launcher's CHECK_GE(supported_capacity_num, 1)
  BRT_REQUIRE(!capacity_padding || supported_capacity_num >= 1,
              "capacity_padding needs at least one supported capacity");
  // the launcher only looks at path_wise_padding inside the capacity_padding branch
  const int path_wise = (capacity_padding && path_wise_padding) ? 1 : 0;
  BRT_REQUIRE(!path_wise || supported_capacity_num >= path_num,
              "path_wise_padding needs one capacity per path (%d < %d)", supported_capacity_num,
              path_num);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cell_num == 0) {
    BRT_CUDA_TRY(cudaMemsetAsync(loads, 0, (size_t)path_num * 4, st));
    return BRT_OK;
  }
  BRT_REQUIRE(hot_mask != nullptr && indices != nullptr, "hot_mask or indices is null");
  return run_scan(is_tag_index ? Mode::kTag : Mode::kSeat, hot_mask, indices, loads, cell_num,
                  path_num, supported_capacities, supported_capacity_num, capacity_padding,
                  path_wise, nullptr, nullptr, scratch, scratch_bytes, st);
}

BRT_API int brt_throttle_hotmask(const int32_t* hotmask, int32_t* throttled, int32_t* prefix,
                                 const int32_t* threshold, int64_t cell_num, int path_num,
                                 void* scratch, size_t scratch_bytes, void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  BRT_REQUIRE(prefix != nullptr && threshold != nullptr, "prefix or threshold is null");
  if (cell_num == 0) return BRT_OK;  // the reference kernel leaves prefix untouched
  BRT_REQUIRE(hotmask != nullptr && throttled != nullptr, "hotmask or throttled is null");
  return run_scan(Mode::kThrottle, hotmask, throttled, nullptr, cell_num, path_num, nullptr, 0,
                  0, 0, prefix, threshold, scratch, scratch_bytes,
                  static_cast<cudaStream_t>(stream));
}

BRT_API int brt_convert_index_format(const int32_t* origin_indices, int32_t* new_indices,
                                     const int32_t* loads, int64_t cell_num, int path_num,
                                     int tag_to_seat, void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  if (cell_num == 0) return BRT_OK;
  BRT_REQUIRE(origin_indices != nullptr && new_indices != nullptr, "index array is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BRT_CUDA_TRY(cudaMemsetAsync(new_indices, 0, (size_t)cell_num * path_num * 4, st));
  const int64_t n = tag_to_seat ? (int64_t)1024 * path_num : cell_num * path_num;
  int64_t blocks = (n + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (tag_to_seat) {
    BRT_REQUIRE(loads != nullptr, "loads is null");
    tag_to_seat_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(origin_indices, new_indices, loads,
                                                              cell_num, path_num);
  } else {
    seat_to_tag_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(origin_indices, new_indices,
                                                              cell_num, path_num);
  }
  BRT_LAUNCH_CHECK("convert_index_format");
  return BRT_OK;
}

}  // extern "C"
