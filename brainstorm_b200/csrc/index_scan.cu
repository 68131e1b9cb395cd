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
// HBM traffic is one read of the mask and one write of the indices.  Masks holding values
// other than 0/1 are detected during `pack` and make `expand` re-read the mask instead of
// the bit words, so the integer semantics of the reference (index = running sum * mask
// value) hold for any int32 mask.
//
// Two implementations of pack/expand share that plan:
//   * the tiled path (path_num % 4 == 0, 16-byte aligned arrays): a CTA stages a
//     [32*k cells, <=256 paths] tile in shared memory with fully coalesced 16-byte loads
//     (every load of the tile is in flight at once), each warp turns a 32x32 block into
//     column bit words with a 5-step shuffle transpose, and `expand` is one popcount per
//     output element with coalesced 16-byte stores.  Whenever the bit words of a CTA's
//     share of the mask fit in shared memory the three steps run as ONE launch (the
//     chained path): a CTA packs a run of consecutive tiles, publishes the run's column
//     sums, adds up the sums of the runs before it (a bounded wait on CTAs that started
//     earlier) and expands its tiles from shared memory;
//   * the strip path (any path_num / alignment): a thread walks 32 cells of V paths.

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kGroupRows = 32;  // cells per bit word

// Where the launch under way writes the per-path cell counts of the indices it produces
// (null: nowhere).  Set by the entry points around their call into the launch helpers.
thread_local int32_t* t_counts_out = nullptr;
struct CountsScope {
  explicit CountsScope(int32_t* p) { t_counts_out = p; }
  ~CountsScope() { t_counts_out = nullptr; }
};

// kMask: write the 0/1 mask itself.  kThrottleSeat: seat indices and loads of the throttled
// mask in one pass (the seat of a kept cell is its seat in the unthrottled mask; a cell is
// kept while prefix + seat <= threshold); single-launch path and 0/1 masks only.
enum class Mode { kSeat, kTag, kThrottle, kMask, kThrottleSeat };

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

size_t tiled_scratch_bytes(int64_t cell_num, int path_num);

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
  const size_t tiled = tiled_scratch_bytes(cell_num, path_num);
  return bytes > tiled ? bytes : tiled;
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
                 const int* __restrict__ threshold, int* __restrict__ counts) {
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
      if (counts != nullptr) counts[col] = run;
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

// ================================================================================ tiled path
constexpr int kTileThreads = 256;
constexpr int kTileWarps = kTileThreads / 32;

struct TileGeom {
  int ec;          // paths per CTA (multiple of 4, <= 256)
  int col_chunks;  // CTAs along the path axis
  int rg;          // 32-cell groups per CTA
  int pitch;       // shared-memory row pitch in ints (ec + 4: conflict-free 16-byte rows)
  int64_t num_groups;
  int64_t num_tiles;
};

int max_row_groups(int ec) {
  const int col_blocks = (ec + 31) / 32;
  const int rg = kTileWarps / col_blocks;  // one 32x32 block per warp
  return rg < 1 ? 1 : rg;
}

// rg == 0: pick the tile height that yields at least two CTAs per SM when possible.
TileGeom make_tile_geom(int64_t cell_num, int path_num, int rg = 0) {
  TileGeom g;
  g.ec = path_num < 256 ? path_num : 256;
  g.col_chunks = (path_num + g.ec - 1) / g.ec;
  g.pitch = g.ec + 4;
  g.num_groups = (cell_num + kGroupRows - 1) / kGroupRows;
  if (rg == 0) {
    rg = max_row_groups(g.ec);
    const int64_t want = (int64_t)sm_count() * 2;
    while (rg > 1 && (g.num_groups + rg - 1) / rg * g.col_chunks < want) rg >>= 1;
  }
  g.rg = rg;
  g.num_tiles = (g.num_groups + rg - 1) / rg;
  return g;
}

// Shared-memory carve-up of one CTA (ints): staged tile | column sums | extra sums | flag |
// bit words | base seats | thresholds.  The staged tile is only needed by pack.
struct TileSmem {
  int* tile;
  int* sum;
  int* extra;
  int* flag;
  int* bits;
  int* base;
  int* thr;
};

__host__ __device__ inline size_t tile_smem_ints(int ec, int rg, int pitch, bool with_tile) {
  return (with_tile ? (size_t)rg * kGroupRows * pitch : 0) + 2 * (size_t)ec + 8 +
         2 * (size_t)rg * ec + ec;
}

__device__ __forceinline__ TileSmem carve_tile_smem(int* s, int ec, int rg, int pitch,
                                                    bool with_tile) {
  TileSmem t;
  t.tile = s;
  s += with_tile ? (size_t)rg * kGroupRows * pitch : 0;
  t.sum = s;
  t.extra = s + ec;
  t.flag = s + 2 * ec;
  s += 2 * ec + 8;
  t.bits = s;
  t.base = s + rg * ec;
  t.thr = s + 2 * rg * ec;
  return t;
}

struct TileCtx {
  int64_t cell_num;
  int path_num;
  int ec, rg, pitch;
  int64_t tile;  // tile index along the cell axis
  int chunk;     // chunk index along the path axis
  int chunks;
};

// 32x32 bit transpose across a warp: lane r enters with row word a (bit c = element (r, c))
// and leaves with the column word of column r (bit k = element (k, r)).
__device__ __forceinline__ uint32_t warp_transpose32(uint32_t a, int lane) {
  uint32_t m = 0x0000ffffu;
#pragma unroll
  for (int j = 16; j != 0; j >>= 1) {
    const uint32_t other = __shfl_xor_sync(0xffffffffu, a, j);
    if ((lane & j) == 0)
      a = (a & m) | ((other & m) << j);
    else
      a = ((other >> j) & m) | (a & ~m);
    m ^= (m << (j >> 1));
  }
  return a;
}

// Turn the tile staged at sm.tile into column bit words at sm.bits (zeroed by the caller
// before the barrier that made the staged tile visible; also written to `bits_out` when that
// is not null).  The tile's column sums are ADDED to sm.sum / sm.extra and a value other
// than 0/1 sets sm.flag.  Ends with a CTA barrier.
__device__ __forceinline__ void pack_staged(const TileCtx& x, const TileSmem& sm,
                                            uint32_t* __restrict__ bits_out) {
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;  // multiple of 4
  const int col_blocks = (cols + 31) >> 5;
  const int blocks = x.rg * col_blocks;
  bool nonbinary = false;
  for (int b = warp; b < blocks; b += kTileWarps) {
    const int g = b / col_blocks;
    const int cb = b - g * col_blocks;
    const int64_t group = x.tile * x.rg + g;
    if (group * kGroupRows >= x.cell_num) continue;  // warp-uniform
    const int c_begin = cb * 32;
    const int c_count = (cols - c_begin) < 32 ? (cols - c_begin) : 32;  // multiple of 4
    const int* rowp = sm.tile + (g * kGroupRows + lane) * x.pitch + c_begin;
    uint32_t roww = 0;
#pragma unroll
    for (int q = 0; q < 8; q++) {
      if (4 * q < c_count) {
        const int4 v = *reinterpret_cast<const int4*>(rowp + 4 * q);
        const int e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          roww |= (e[j] != 0 ? 1u : 0u) << (4 * q + j);
          if (static_cast<unsigned>(e[j]) > 1u) {
            nonbinary = true;
            atomicAdd(&sm.extra[c_begin + 4 * q + j], e[j] - 1);
          }
        }
      }
    }
    const uint32_t colw = warp_transpose32(roww, lane);
    if (lane < c_count) {
      sm.bits[g * x.ec + c_begin + lane] = static_cast<int>(colw);
      if (bits_out != nullptr) bits_out[group * x.path_num + col0 + c_begin + lane] = colw;
      const int n = __popc(colw);
      if (n != 0) atomicAdd(&sm.sum[c_begin + lane], n);
    }
  }
  if (nonbinary) atomicOr(sm.flag, 1);
  __syncthreads();
}

// Start the asynchronous copy of one tile of the mask into `stage` (rows beyond the mask
// are zero-filled with plain stores) and zero the tile's bit words.  The caller commits the
// group, waits for it and passes a CTA barrier before pack_staged.
__device__ __forceinline__ void stage_tile_async(const TileCtx& x, int* stage, int* bits,
                                                 const int* __restrict__ mask) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;
  const int64_t row0 = x.tile * x.rg * kGroupRows;
  const int tile_rows = x.rg * kGroupRows;
  const int vec_per_row = cols >> 2;
  const int total_vecs = tile_rows * vec_per_row;
  for (int i = tid; i < x.rg * x.ec; i += kTileThreads) bits[i] = 0;
  const int step_r = kTileThreads / vec_per_row;
  const int step_q = kTileThreads - step_r * vec_per_row;
  int r = tid / vec_per_row;
  int q = tid - r * vec_per_row;
  for (int idx = tid; idx < total_vecs; idx += kTileThreads) {
    int* dst = stage + r * x.pitch + 4 * q;
    if (row0 + r < x.cell_num)
      cp_async_16(dst, mask + (row0 + r) * x.path_num + col0 + 4 * q);
    else
      *reinterpret_cast<int4*>(dst) = make_int4(0, 0, 0, 0);
    r += step_r;
    q += step_q;
    if (q >= vec_per_row) { q -= vec_per_row; r += 1; }
  }
}

// Stage one tile of the mask and turn it into column bit words (kept in shared memory at
// sm.bits, and written to `bits_out` when that is not null).  The tile's column sums are
// ADDED to sm.sum / sm.extra and a value other than 0/1 sets sm.flag: the caller zeroes the
// three before its first tile.  Ends with a CTA barrier.
__device__ __forceinline__ void pack_tile_body(const TileCtx& x, const TileSmem& sm,
                                               const int* __restrict__ mask,
                                               uint32_t* __restrict__ bits_out) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;  // multiple of 4
  const int64_t row0 = x.tile * x.rg * kGroupRows;
  const int tile_rows = x.rg * kGroupRows;
  const int vec_per_row = cols >> 2;
  const int total_vecs = tile_rows * vec_per_row;

  for (int i = tid; i < x.rg * x.ec; i += kTileThreads) sm.bits[i] = 0;

  // Stage the tile: every 16-byte load is issued before the first store.  A tile holds at
  // most 2048 vectors (8 per thread).  (row, vector) of a thread's k-th element advance by a
  // fixed step with one carry, so the loop has no integer division.
  constexpr int kBatch = 8;
  {
    const int step_r = kTileThreads / vec_per_row;
    const int step_q = kTileThreads - step_r * vec_per_row;
    int r = tid / vec_per_row;
    int q = tid - r * vec_per_row;
    int4 v[kBatch];
    int soff[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; k++) {
      v[k] = make_int4(0, 0, 0, 0);
      soff[k] = r * x.pitch + 4 * q;
      if (r < tile_rows && row0 + r < x.cell_num)
        v[k] = __ldcs(reinterpret_cast<const int4*>(mask + (row0 + r) * x.path_num + col0 +
                                                     4 * q));
      r += step_r;
      q += step_q;
      if (q >= vec_per_row) { q -= vec_per_row; r += 1; }
    }
#pragma unroll
    for (int k = 0; k < kBatch; k++)
      if (tid + k * kTileThreads < total_vecs)
        *reinterpret_cast<int4*>(sm.tile + soff[k]) = v[k];
  }
  __syncthreads();

  pack_staged(x, sm, bits_out);
}

// One tile per CTA: pack it and publish its column sums and its "value other than 0/1
// seen" flag to global memory.
__device__ __forceinline__ void pack_tile(const TileCtx& x, const TileSmem& sm,
                                          const int* __restrict__ mask,
                                          uint32_t* __restrict__ bits_out,
                                          int* __restrict__ tile_sums,
                                          int* __restrict__ tile_flags) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;
  // zeroed before the barrier inside the body that precedes its first atomic
  for (int i = tid; i < 2 * x.ec + 1; i += kTileThreads) sm.sum[i] = 0;
  pack_tile_body(x, sm, mask, bits_out);
  for (int c = tid; c < cols; c += kTileThreads)
    tile_sums[x.tile * x.path_num + col0 + c] = sm.sum[c] + sm.extra[c];
  if (tid == 0) tile_flags[x.tile * x.chunks + x.chunk] = *sm.flag;
}

// Exclusive prefix of the per-tile sums along the tile axis, in place, for the 4 paths
// starting at 4 * col_block; THREADS / 4 tile segments are scanned in parallel.  The CTA
// with col_block == 0 also folds the per-tile flags into flags[0].  The thread that owns
// the last segment applies the capacity / throttle rules to the column total.
template <bool THROTTLE, int THREADS>
__device__ __forceinline__ void scan_tiles(int col_block, int* __restrict__ tile_sums,
                                           int64_t num_tiles, int path_num,
                                           const int* __restrict__ tile_flags,
                                           int64_t num_flags, int* __restrict__ flags,
                                           int* __restrict__ loads,
                                           const int* __restrict__ caps, int ncap,
                                           int capacity_padding, int path_wise,
                                           int* __restrict__ prefix,
                                           const int* __restrict__ threshold,
                                           int (*s_warp)[4], int* __restrict__ counts) {
  constexpr int kSegs = THREADS / 4;
  constexpr int kWarpsHere = THREADS / 32;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int cw = tid & 3;
  const int seg = tid >> 2;
  const int col = col_block * 4 + cw;
  const bool valid = col < path_num;
  const int64_t len = (num_tiles + kSegs - 1) / kSegs;
  const int64_t t0 = seg * len;
  const int64_t t1 = (t0 + len) < num_tiles ? (t0 + len) : num_tiles;

  // The segment is read once into registers when it is short enough (the common case),
  // so that the prefix pass needs no second, serialised trip to memory.
  constexpr int kKeep = 16;
  int kept[kKeep];
  const bool short_seg = len <= kKeep;
  int own = 0;
  if (valid) {
    if (short_seg) {
#pragma unroll
      for (int i = 0; i < kKeep; i++) {
        const int64_t t = t0 + i;
        kept[i] = t < t1 ? tile_sums[t * path_num + col] : 0;
      }
#pragma unroll
      for (int i = 0; i < kKeep; i++) own += kept[i];
    } else {
      for (int64_t tb = t0; tb < t1; tb += kKeep) {
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
          const int64_t t = tb + i;
          kept[i] = t < t1 ? tile_sums[t * path_num + col] : 0;
        }
#pragma unroll
        for (int i = 0; i < kKeep; i++) own += kept[i];
      }
    }
  }
  int incl = own;
#pragma unroll
  for (int d = 4; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  if (lane >= 28) s_warp[warp][cw] = incl;
  int start = 0;
  if (THROTTLE && valid) start = prefix[col];  // read before anyone overwrites it below
  int any_flag = 0;
  if (col_block == 0)
    for (int64_t i = tid; i < num_flags; i += THREADS) any_flag |= tile_flags[i];
  any_flag = __syncthreads_or(any_flag);
  if (col_block == 0 && tid == 0) flags[0] = any_flag;

  int run = incl - own;
  for (int w = 0; w < warp && w < kWarpsHere; w++) run += s_warp[w][cw];
  if (valid) {
    int acc = run + start;
    if (short_seg) {
#pragma unroll
      for (int i = 0; i < kKeep; i++) {
        const int64_t t = t0 + i;
        if (t < t1) tile_sums[t * path_num + col] = acc;
        acc += kept[i];
      }
    } else {
      for (int64_t tb = t0; tb < t1; tb += kKeep) {
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
          const int64_t t = tb + i;
          kept[i] = t < t1 ? tile_sums[t * path_num + col] : 0;
        }
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
          const int64_t t = tb + i;
          if (t < t1) tile_sums[t * path_num + col] = acc;
          acc += kept[i];
        }
      }
    }
    if (seg == kSegs - 1) {
      const int total = run + own;
      if (THROTTLE) {
        const int thr = threshold[col];
        const int p = start + total;
        prefix[col] = p >= thr ? thr : p;
      } else {
        loads[col] = map_load(total, col, caps, ncap, capacity_padding != 0, path_wise != 0);
        if (counts != nullptr) counts[col] = total;
      }
    }
  }
}

// Masks with values other than 0/1: thread c walks path c of the tile serially through the
// mask itself (integer semantics: index = running sum * value).  `run` enters as the
// column's sum over all earlier cells and leaves advanced by this tile.
template <Mode MODE>
__device__ __forceinline__ void expand_general(const TileCtx& x, const int* __restrict__ mask,
                                               int& run, int* __restrict__ out,
                                               const int* __restrict__ threshold) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;
  const int64_t row0 = x.tile * x.rg * kGroupRows;
  if (tid >= cols) return;
  const int thr = MODE == Mode::kThrottle ? threshold[col0 + tid] : 0;
  for (int r = 0; r < x.rg * kGroupRows; r++) {
    const int64_t row = row0 + r;
    if (row >= x.cell_num) break;
    const int64_t at = row * x.path_num + col0 + tid;
    const int m = mask[at];
    run += m;
    if constexpr (MODE == Mode::kThrottle) {
      out[at] = (m == 1 && run <= thr) ? 1 : 0;
    } else if constexpr (MODE == Mode::kThrottleSeat) {
      out[at] = 0;  // not defined for masks with values other than 0/1 (reported by the caller)
    } else if constexpr (MODE == Mode::kSeat) {
      out[at] = run * m;
    } else if constexpr (MODE == Mode::kMask) {
      out[at] = m != 0 ? 1 : 0;
    } else {
      const int64_t dst_row = (int64_t)run * m - 1;
      if (run * m != 0 && dst_row >= 0 && dst_row < x.cell_num)
        out[dst_row * x.path_num + col0 + tid] = (int)(row + 1);
    }
  }
}

// 0/1 masks: write one tile from its bit words (sm.bits) and the per-path sums over all
// earlier cells (`run` of thread c for path c, advanced by this tile on return).  Opens with
// a CTA barrier, so sm.bits / sm.thr written just before the call are visible and sm.base
// of an earlier tile is no longer read.
template <Mode MODE>
__device__ __forceinline__ void expand_binary(const TileCtx& x, const TileSmem& sm, int& run,
                                              int* __restrict__ out,
                                              int* __restrict__ mask_out = nullptr) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;
  const int64_t row0 = x.tile * x.rg * kGroupRows;
  __syncthreads();
  if (tid < cols) {  // cols <= 256 = kTileThreads: one path per thread
    for (int g = 0; g < x.rg; g++) {
      sm.base[g * x.ec + tid] = run;
      run += __popc(static_cast<uint32_t>(sm.bits[g * x.ec + tid]));
    }
  }
  __syncthreads();

  const int vec_per_row = cols >> 2;
  const int total_vecs = x.rg * kGroupRows * vec_per_row;
  const int step_r = kTileThreads / vec_per_row;
  const int step_q = kTileThreads - step_r * vec_per_row;
  int r = tid / vec_per_row;
  int q = tid - r * vec_per_row;
  for (int idx = tid; idx < total_vecs; idx += kTileThreads) {
    const int64_t row = row0 + r;
    if (row >= x.cell_num) break;
    const int g = r >> 5;
    const int rr = r & 31;
    const uint32_t low = 0xffffffffu >> (31 - rr);  // bits 0..rr
    const int4 w4 = *reinterpret_cast<const int4*>(sm.bits + g * x.ec + 4 * q);
    const int4 b4 = *reinterpret_cast<const int4*>(sm.base + g * x.ec + 4 * q);
    const uint32_t w[4] = {(uint32_t)w4.x, (uint32_t)w4.y, (uint32_t)w4.z, (uint32_t)w4.w};
    const int b[4] = {b4.x, b4.y, b4.z, b4.w};
    int v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int bit = (w[j] >> rr) & 1u;
      const int seat = b[j] + __popc(w[j] & low);
      if constexpr (MODE == Mode::kThrottle)
        v[j] = (bit && seat <= sm.thr[4 * q + j]) ? 1 : 0;
      else if constexpr (MODE == Mode::kThrottleSeat)
        v[j] = (bit && seat <= sm.thr[4 * q + j]) ? seat : 0;
      else if constexpr (MODE == Mode::kMask)
        v[j] = bit;
      else
        v[j] = bit ? seat : 0;
    }
    if constexpr (MODE == Mode::kTag) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int64_t dst_row = (int64_t)v[j] - 1;
        if (v[j] != 0 && dst_row < x.cell_num)
          out[dst_row * x.path_num + col0 + 4 * q + j] = (int)(row + 1);
      }
    } else {
      __stcs(reinterpret_cast<int4*>(out + row * x.path_num + col0 + 4 * q),
             make_int4(v[0], v[1], v[2], v[3]));
      if constexpr (MODE == Mode::kThrottleSeat || MODE == Mode::kSeat) {
        if (mask_out != nullptr)  // the (throttled) 0/1 mask itself, for callers that want both
          __stcs(reinterpret_cast<int4*>(mask_out + row * x.path_num + col0 + 4 * q),
                 make_int4(v[0] != 0, v[1] != 0, v[2] != 0, v[3] != 0));
      }
    }
    r += step_r;
    q += step_q;
    if (q >= vec_per_row) { q -= vec_per_row; r += 1; }
  }
}

// Write the indices (or the throttled mask) of one tile from its bit words and the tile's
// exclusive prefix in global memory.  `bits_in` != null: the words are first fetched from
// global memory (separate-launch path); null: pack left them in shared memory.
template <Mode MODE>
__device__ __forceinline__ void expand_tile(const TileCtx& x, const TileSmem& sm,
                                            const int* __restrict__ mask,
                                            const uint32_t* __restrict__ bits_in,
                                            const int* __restrict__ tile_prefix,
                                            const int* __restrict__ flags,
                                            int* __restrict__ out,
                                            const int* __restrict__ threshold) {
  const int tid = threadIdx.x;
  const int col0 = x.chunk * x.ec;
  const int cols = (x.path_num - col0) < x.ec ? (x.path_num - col0) : x.ec;
  const int64_t num_groups = (x.cell_num + kGroupRows - 1) / kGroupRows;
  // fetched before any barrier so that the global reads of the prologue overlap
  int run = tid < cols ? tile_prefix[x.tile * x.path_num + col0 + tid] : 0;
  if ((flags[0] & 1) != 0) {
    expand_general<MODE>(x, mask, run, out, threshold);
    return;
  }
  if (bits_in != nullptr) {
    for (int i = tid; i < x.rg * cols; i += kTileThreads) {
      const int g = i / cols;
      const int c = i - g * cols;
      const int64_t group = x.tile * x.rg + g;
      sm.bits[g * x.ec + c] =
          group < num_groups ? static_cast<int>(bits_in[group * x.path_num + col0 + c]) : 0;
    }
  }
  if constexpr (MODE == Mode::kThrottle)
    for (int c = tid; c < cols; c += kTileThreads) sm.thr[c] = threshold[col0 + c];
  expand_binary<MODE>(x, sm, run, out);
}

struct TiledArgs {
  const int* mask;
  int* out;
  int* mask_out;  // seat modes of the gated scan, may be null: the 0/1 mask beside the indices
  uint32_t* bits;
  int* tile_sums;
  int* tile_flags;
  int* flags;
  int* loads;
  int* counts;  // may be null: cells per path that the written indices hold (before the
                // capacity rules turn them into loads)
  const int* caps;
  int ncap;
  int capacity_padding;
  int path_wise;
  int* prefix;
  const int* threshold;
  int64_t cell_num;
  int path_num;
  int ec, rg, pitch;
  int64_t num_tiles;
  int chunks;
};

__device__ __forceinline__ TileCtx ctx_of(const TiledArgs& a) {
  TileCtx x;
  x.cell_num = a.cell_num;
  x.path_num = a.path_num;
  x.ec = a.ec;
  x.rg = a.rg;
  x.pitch = a.pitch;
  x.tile = blockIdx.x;
  x.chunk = blockIdx.y;
  x.chunks = a.chunks;
  return x;
}

__global__ void __launch_bounds__(kTileThreads) mask_pack_tiled_kernel(const TiledArgs a) {
  extern __shared__ __align__(16) int s_dyn[];
  const TileSmem sm = carve_tile_smem(s_dyn, a.ec, a.rg, a.pitch, true);
  pack_tile(ctx_of(a), sm, a.mask, a.bits, a.tile_sums, a.tile_flags);
}

template <bool THROTTLE>
__global__ void __launch_bounds__(1024) tile_scan_wide_kernel(const TiledArgs a) {
  __shared__ int s_warp[32][4];
  scan_tiles<THROTTLE, 1024>(blockIdx.x, a.tile_sums, a.num_tiles, a.path_num, a.tile_flags,
                             a.num_tiles * a.chunks, a.flags, a.loads, a.caps, a.ncap,
                             a.capacity_padding, a.path_wise, a.prefix, a.threshold, s_warp,
                             a.counts);
}

template <Mode MODE>
__global__ void __launch_bounds__(kTileThreads) index_expand_tiled_kernel(const TiledArgs a) {
  extern __shared__ __align__(16) int s_dyn[];
  const TileSmem sm = carve_tile_smem(s_dyn, a.ec, a.rg, a.pitch, false);
  expand_tile<MODE>(ctx_of(a), sm, a.mask, a.bits, a.tile_sums, a.flags, a.out, a.threshold);
}

// ------------------------------------------------------------------------------- gate rows
// Route decision of a staged tile of fp32 scores.  A warp (or a part of it, for narrow rows)
// decides one row at a time and keeps the outcome as bits of the column words of the row's
// 32-cell group; the words of all warps meet in shared memory, so no mask is ever written.
//   kind 1: ones at the top_k largest scores of the row (python/brt/router/protocol/topk.py:
//           26-31); equal scores go to the lower path index;
//   kind 2: ones where score > threshold; a row without any goes to residual_path when that
//           is >= 0 (python/brt/router/protocol/threshold.py:23-39).
// gates_out (optional, [cell, path] fp32): the picked scores divided by their sum clamped at
// FLT_EPSILON, zero elsewhere (python/brt/router/protocol/swin_moe.py:193-204).
struct GateArgs {
  int kind;  // 0: the input is a mask already
  int top_k;
  float threshold;
  int residual_path;
  float* gates_out;
};

// fp32 bits -> unsigned key with the same order (and back); key 0 is below every score
__device__ __forceinline__ unsigned score_key(int bits) {
  const unsigned u = static_cast<unsigned>(bits);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_score(unsigned key) {
  const unsigned u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
  return __uint_as_float(u);
}

// PER scores per lane, L lanes per row (L < 32 only with PER == 1: 32 / L rows per warp).
// A pick costs two warp reductions: the largest key among the row's unpicked scores, then
// the lowest path that holds it.
template <int PER, int L>
__device__ __forceinline__ void gate_rows_as(const TileCtx& x, const int* stage, int* bits,
                                             int* sums, const GateArgs& g) {
  constexpr int kRowsPerWarp = 32 / L;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / L;
  const int l = lane - sub * L;
  const unsigned members = L == 32 ? 0xffffffffu : (((1u << L) - 1u) << (sub * L));
  const int cols = x.path_num;  // a gated tile spans every path
  const int64_t row0 = x.tile * x.rg * kGroupRows;
  const int tile_rows = x.rg * kGroupRows;
  // column bit words of the 32-cell group this lane is in, for the rows it has seen so far;
  // handed to shared memory (where the other warps' rows of the group meet) when the group
  // changes
  unsigned word[PER];
#pragma unroll
  for (int i = 0; i < PER; i++) word[i] = 0;
  int group = 0;
  auto flush = [&]() {
#pragma unroll
    for (int i = 0; i < PER; i++) {
      if (word[i] != 0) {
        const int c = l + L * i;
        atomicOr(reinterpret_cast<unsigned*>(bits) + group * x.ec + c, word[i]);
        atomicAdd(sums + c, __popc(word[i]));
        word[i] = 0;
      }
    }
  };
  for (int r = warp * kRowsPerWarp + sub; r < tile_rows; r += kTileWarps * kRowsPerWarp) {
    const int64_t row = row0 + r;
    if (row >= x.cell_num) break;  // uniform per row group; later rows were staged as zeros
    if ((r >> 5) != group) {
      flush();
      group = r >> 5;
    }
    const int* p = stage + r * x.pitch;
    unsigned key[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
      const int c = l + L * i;
      key[i] = c < cols ? score_key(p[c]) : 0u;
    }
    unsigned picked = 0;
    float denom = 0.f;
    if (g.kind == 1) {
      for (int t = 0; t < g.top_k; t++) {
        unsigned mine = 0;
#pragma unroll
        for (int i = 0; i < PER; i++)
          if (!((picked >> i) & 1u) && key[i] > mine) mine = key[i];
        const unsigned best = __reduce_max_sync(members, mine);
        if (best == 0u) break;  // fewer paths than top_k
        unsigned my_col = 0xffffffffu;
#pragma unroll
        for (int i = PER - 1; i >= 0; i--)
          if (!((picked >> i) & 1u) && key[i] == best) my_col = l + L * i;
        const unsigned col = __reduce_min_sync(members, my_col);
        if (col == my_col) picked |= 1u << (col / L);
        denom = __fadd_rn(denom, key_score(best));
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; i++)
        if (l + L * i < cols && key_score(key[i]) > g.threshold) picked |= 1u << i;
      if (g.residual_path >= 0 && __ballot_sync(members, picked != 0) == 0 &&
          (g.residual_path % L) == l)
        picked |= 1u << (g.residual_path / L);
    }
    const int rr = r & 31;
#pragma unroll
    for (int i = 0; i < PER; i++) word[i] |= ((picked >> i) & 1u) << rr;
    if (g.gates_out != nullptr) {
      denom = fmaxf(denom, 1.1920928955078125e-07f);
#pragma unroll
      for (int i = 0; i < PER; i++) {
        const int c = l + L * i;
        if (c < cols)
          __stcs(g.gates_out + row * x.path_num + c,
                 ((picked >> i) & 1u) ? __fdiv_rn(key_score(key[i]), denom) : 0.f);
      }
    }
  }
  flush();
}

// Decide the routes of a staged tile of scores and leave the result as column bit words in
// `bits` (zeroed beforehand) and per-path counts added to `sums`: what pack_staged produces
// from a staged mask, without a mask in between.  The caller passes a CTA barrier next.
__device__ __forceinline__ void gate_rows(const TileCtx& x, const int* stage, int* bits,
                                          int* sums, const GateArgs& g) {
  const int cols = x.path_num;  // <= 256, warp-uniform
  if (cols <= 8) gate_rows_as<1, 8>(x, stage, bits, sums, g);
  else if (cols <= 16) gate_rows_as<1, 16>(x, stage, bits, sums, g);
  else if (cols <= 32) gate_rows_as<1, 32>(x, stage, bits, sums, g);
  else if (cols <= 64) gate_rows_as<2, 32>(x, stage, bits, sums, g);
  else if (cols <= 128) gate_rows_as<4, 32>(x, stage, bits, sums, g);
  else gate_rows_as<8, 32>(x, stage, bits, sums, g);
}

// ---------------------------------------------------------------------------- chained path
// One launch, no grid-wide barrier.  A CTA takes a ticket; ticket k owns a run of
// consecutive tiles of one path chunk.  It packs them all (the bit words stay in shared
// memory), publishes the run's column sums, adds up the sums published by the tickets before
// it and then writes its tiles.  A ticket only ever waits for SMALLER tickets, whose CTAs
// have started by construction, so the kernel needs no co-residency guarantee.
struct ChainArgs {
  TiledArgs t;
  GateArgs gate;
  unsigned long long* status;  // [ranges][path_num]: (1 << 32) | column sum once published
  int* ticket;
  int* error;       // set to 1 when a wait ran out
  int* host_error;  // host-mapped word that receives BRT_ERR_TIMEOUT then (may be null)
  int spin_limit;   // polls (each followed by a short sleep) before a wait gives up
  int first_ticket; // 0; a test passes 1 so that the first run is never published
  int tiles_per_cta;
  int ranges;
};

constexpr int kChainFly = 16;            // status words a thread keeps in flight
constexpr int kChainSpinLimit = 1 << 20;  // default number of polls

__device__ __forceinline__ void status_publish(unsigned long long* p, int value) {
  const unsigned long long w = (1ull << 32) | static_cast<unsigned>(value);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long status_peek(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}

template <Mode MODE, bool GATED>
__global__ void __launch_bounds__(kTileThreads, 2) index_chain_kernel(const ChainArgs c) {
  extern __shared__ __align__(16) int s_dyn[];
  __shared__ int s_ticket;
  const TiledArgs& a = c.t;
  const int tid = threadIdx.x;
  if (tid == 0) s_ticket = atomicAdd(c.ticket, 1);
  TileSmem sm = carve_tile_smem(s_dyn, a.ec, a.rg, a.pitch, true);
  int* bits_all = s_dyn + tile_smem_ints(a.ec, a.rg, a.pitch, true);
  for (int i = tid; i < 2 * a.ec + 1; i += kTileThreads) sm.sum[i] = 0;
  __syncthreads();
  const int ticket = s_ticket + c.first_ticket;
  const int range = ticket / a.chunks;
  if (range >= c.ranges) return;  // only with first_ticket != 0: nothing left to own
  TileCtx x;
  x.cell_num = a.cell_num;
  x.path_num = a.path_num;
  x.ec = a.ec;
  x.rg = a.rg;
  x.pitch = a.pitch;
  x.chunk = ticket - range * a.chunks;
  x.chunks = a.chunks;
  const int col0 = x.chunk * a.ec;
  const int cols = (a.path_num - col0) < a.ec ? (a.path_num - col0) : a.ec;
  const int64_t tile0 = (int64_t)range * c.tiles_per_cta;
  const int64_t tile1 = (tile0 + c.tiles_per_cta) < a.num_tiles ? (tile0 + c.tiles_per_cta)
                                                                 : a.num_tiles;
  const int words_per_tile = a.rg * a.ec;

  // read before this CTA publishes anything: the last ticket overwrites prefix[] only after
  // it has seen every publication
  // (kThrottleSeat counts seats from 1 within this call, so its limit is what is left of the
  // threshold after the prefix)
  constexpr bool kThrottles = MODE == Mode::kThrottle || MODE == Mode::kThrottleSeat;
  int start = 0;
  if (kThrottles && tid < cols) {
    start = a.prefix[col0 + tid];
    const int thr = a.threshold[col0 + tid];
    sm.thr[tid] = MODE == Mode::kThrottleSeat ? thr - start : thr;
  }

  // two staging buffers: the copy of tile t + 1 is in flight while tile t is packed
  int* const stage[2] = {sm.tile, bits_all + (size_t)c.tiles_per_cta * words_per_tile};
  x.tile = tile0;
  stage_tile_async(x, stage[0], bits_all, a.mask);
  cp_async_commit();
  for (int64_t t = tile0; t < tile1; t++) {
    const int i = (int)(t - tile0);
    if (t + 1 < tile1) {
      x.tile = t + 1;
      stage_tile_async(x, stage[(i + 1) & 1], bits_all + (size_t)(i + 1) * words_per_tile, a.mask);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    x.tile = t;
    TileSmem cur = sm;
    cur.tile = stage[i & 1];
    cur.bits = bits_all + (size_t)i * words_per_tile;
    if constexpr (GATED) {  // the staged tile holds scores: straight to bit words and counts
      gate_rows(x, cur.tile, cur.bits, sm.sum, c.gate);
      __syncthreads();
    } else {
      pack_staged(x, cur, nullptr);
    }
  }
  const int own = tid < cols ? sm.sum[tid] + sm.extra[tid] : 0;
  const bool general = *sm.flag != 0;
  __threadfence();
  if (tid < cols) status_publish(c.status + (int64_t)range * a.path_num + col0 + tid, own);

  // sum of the tickets before this one: thread (part, path) takes every parts-th of them,
  // kChainFly loads in flight at a time
  int* s_before = sm.base;  // free until the first expand
  for (int i = tid; i < a.ec; i += kTileThreads) s_before[i] = 0;
  __syncthreads();
  {
    const int parts = kTileThreads / cols;
    const int part = tid / cols;
    const int path = tid - part * cols;
    if (part < parts && range > 0) {
      const unsigned long long* column = c.status + col0 + path;
      int acc = 0;
      for (int j0 = part; j0 < range; j0 += parts * kChainFly) {
        unsigned long long w[kChainFly];
        int spins = 0;
        for (;;) {
          bool ready = true;
#pragma unroll
          for (int u = 0; u < kChainFly; u++) {
            const int j = j0 + u * parts;
            w[u] = j < range ? status_peek(column + (int64_t)j * a.path_num) : (1ull << 32);
          }
#pragma unroll
          for (int u = 0; u < kChainFly; u++) ready = ready && (w[u] >> 32) != 0;
          if (ready) break;
          if (++spins > c.spin_limit) {  // give up: report it and carry on with what is there
            *c.error = 1;
            if (c.host_error != nullptr) {
              *reinterpret_cast<volatile int*>(c.host_error) = BRT_ERR_TIMEOUT;
              __threadfence_system();
            }
            break;
          }
          __nanosleep(64);
        }
#pragma unroll
        for (int u = 0; u < kChainFly; u++) acc += static_cast<int>(static_cast<unsigned>(w[u]));
      }
      if (acc != 0) atomicAdd(&s_before[path], acc);
    }
  }
  __syncthreads();
  int run = tid < cols ? s_before[tid] + (MODE == Mode::kThrottle ? start : 0) : 0;

  if (range == c.ranges - 1 && tid < cols) {
    const int total = s_before[tid] + own;
    __threadfence();
    if constexpr (kThrottles) {
      const int thr = MODE == Mode::kThrottleSeat ? sm.thr[tid] + start : sm.thr[tid];
      const int p = start + total;
      a.prefix[col0 + tid] = p >= thr ? thr : p;
    }
    if constexpr (MODE == Mode::kThrottleSeat) {
      const int room = sm.thr[tid] > 0 ? sm.thr[tid] : 0;
      const int kept = total < room ? total : room;
      a.loads[col0 + tid] = map_load(kept, col0 + tid, a.caps, a.ncap, a.capacity_padding != 0,
                                     a.path_wise != 0);
      if (a.counts != nullptr) a.counts[col0 + tid] = kept;
    } else if constexpr (!kThrottles) {
      a.loads[col0 + tid] = map_load(total, col0 + tid, a.caps, a.ncap, a.capacity_padding != 0,
                                     a.path_wise != 0);
      if (a.counts != nullptr) a.counts[col0 + tid] = total;
    }
  }
  if (MODE == Mode::kThrottleSeat && general && tid == 0) {
    // the fused pass is only defined for 0/1 masks: say so instead of inventing indices
    *c.error = 2;
    if (c.host_error != nullptr) {
      *reinterpret_cast<volatile int*>(c.host_error) = BRT_ERR_INVALID_ARGUMENT;
      __threadfence_system();
    }
  }

  for (int64_t t = tile0; t < tile1; t++) {
    x.tile = t;
    if (general) {
      expand_general<MODE>(x, a.mask, run, a.out, a.threshold);
    } else {
      TileSmem cur = sm;
      cur.bits = bits_all + (t - tile0) * words_per_tile;
      expand_binary<MODE>(x, cur, run, a.out, a.mask_out);
    }
  }
}

size_t tiled_scratch_bytes(int64_t cell_num, int path_num) {
  // bounded for the smallest tile (one 32-cell group per tile)
  const size_t groups = (size_t)((cell_num + kGroupRows - 1) / kGroupRows);
  const size_t chunks = (size_t)(path_num + 255) / 256;
  return 256 + round_up(groups * chunks * 4 + 4, 256) + 2 * round_up(groups * path_num * 4 + 4, 256);
}

constexpr int kChainCtasPerSm = 2;
constexpr size_t kChainSmemLimit = 110 * 1024;

// A run-out look-back wait is reported through one word of host-mapped memory per process:
// kernels write it, the host reads it without synchronising (brt_index_status).  The word is
// created by the first call that may allocate; the entry point that must not allocate only
// uses it when it exists already.
struct HostStatus {
  std::mutex mu;
  int* host = nullptr;
  int* device = nullptr;
};
HostStatus& index_status() {
  static HostStatus s;
  return s;
}
int* index_status_word(bool may_allocate) {
  HostStatus& s = index_status();
  std::lock_guard<std::mutex> lock(s.mu);
  if (s.host == nullptr && may_allocate) {
    int* h = nullptr;
    void* d = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64,
                      cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      memset(h, 0, 64);
      if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) {
        s.host = h;
        s.device = static_cast<int*>(d);
      } else {
        cudaFreeHost(h);
      }
    }
    cudaGetLastError();
  }
  return s.device;
}

// Test hooks (brt_index_set_test_hooks): a shorter wait and a first run that nobody owns.
std::atomic<int> g_spin_limit{kChainSpinLimit};
std::atomic<int> g_first_ticket{0};
thread_local bool t_may_allocate = true;  // false inside the entry point that must not

template <Mode MODE, bool GATED>
int launch_chain_mode(const ChainArgs& c, unsigned grid, size_t smem, cudaStream_t stream) {
  static thread_local std::map<int, size_t> configured;  // device -> opted-in bytes
  if (smem > 48 * 1024) {
    int dev = 0;
    BRT_CUDA_TRY(cudaGetDevice(&dev));
    if (configured[dev] < smem) {
      BRT_CUDA_TRY(cudaFuncSetAttribute(index_chain_kernel<MODE, GATED>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kChainSmemLimit));
      configured[dev] = kChainSmemLimit;
    }
  }
  const KernelTimer timer(GATED ? "route_scores_kernel"
                                : MODE == Mode::kThrottle ? "throttle_chain_kernel"
                                : MODE == Mode::kThrottleSeat ? "throttle_index_chain_kernel"
                                                              : "index_chain_kernel",
                          stream);
  index_chain_kernel<MODE, GATED><<<grid, kTileThreads, smem, stream>>>(c), note_launch();
  BRT_LAUNCH_CHECK("index_chain_kernel");
  return BRT_OK;
}

int launch_chain(Mode mode, const TileGeom& g, int tiles_per_cta, int ranges, size_t smem,
                 const int32_t* mask, int32_t* out, int32_t* loads, int64_t cell_num,
                 int path_num, const int32_t* caps, int ncap, int capacity_padding,
                 int path_wise, int32_t* prefix, const int32_t* threshold, void* scratch,
                 cudaStream_t stream, const GateArgs* gate = nullptr,
                 int32_t* mask_out = nullptr) {
  ChainArgs c;
  c.gate = gate != nullptr ? *gate : GateArgs{0, 0, 0.f, -1, nullptr};
  char* p = static_cast<char*>(scratch);
  c.t.flags = reinterpret_cast<int*>(p);
  c.error = c.t.flags + 1;
  c.ticket = c.t.flags + 2;
  c.host_error = index_status_word(t_may_allocate);
  c.spin_limit = g_spin_limit.load(std::memory_order_relaxed);
  c.first_ticket = g_first_ticket.load(std::memory_order_relaxed);
  c.status = reinterpret_cast<unsigned long long*>(p + 256);
  c.tiles_per_cta = tiles_per_cta;
  c.ranges = ranges;
  c.t.tile_flags = nullptr;
  c.t.tile_sums = nullptr;
  c.t.bits = nullptr;
  c.t.mask = mask;
  c.t.out = out;
  c.t.mask_out = mask_out;
  c.t.loads = loads;
  c.t.counts = t_counts_out;
  c.t.caps = caps;
  c.t.ncap = ncap;
  c.t.capacity_padding = capacity_padding;
  c.t.path_wise = path_wise;
  c.t.prefix = prefix;
  c.t.threshold = threshold;
  c.t.cell_num = cell_num;
  c.t.path_num = path_num;
  c.t.ec = g.ec;
  c.t.rg = g.rg;
  c.t.pitch = g.pitch;
  c.t.num_tiles = g.num_tiles;
  c.t.chunks = g.col_chunks;
  BRT_CUDA_TRY(cudaMemsetAsync(p, 0, 256 + (size_t)ranges * path_num * 8, stream));
  if (mode == Mode::kTag)
    BRT_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)cell_num * path_num * 4, stream));
  const unsigned grid = (unsigned)ranges * (unsigned)g.col_chunks;
  if (gate != nullptr) {
    switch (mode) {
      case Mode::kSeat: return launch_chain_mode<Mode::kSeat, true>(c, grid, smem, stream);
      case Mode::kMask: return launch_chain_mode<Mode::kMask, true>(c, grid, smem, stream);
      case Mode::kThrottleSeat:
        return launch_chain_mode<Mode::kThrottleSeat, true>(c, grid, smem, stream);
      default: return launch_chain_mode<Mode::kThrottle, true>(c, grid, smem, stream);
    }
  }
  switch (mode) {
    case Mode::kSeat: return launch_chain_mode<Mode::kSeat, false>(c, grid, smem, stream);
    case Mode::kTag: return launch_chain_mode<Mode::kTag, false>(c, grid, smem, stream);
    case Mode::kThrottleSeat:
      return launch_chain_mode<Mode::kThrottleSeat, false>(c, grid, smem, stream);
    default: return launch_chain_mode<Mode::kThrottle, false>(c, grid, smem, stream);
  }
}

int launch_tiled(Mode mode, const int32_t* mask, int32_t* out, int32_t* loads, int64_t cell_num,
                 int path_num, const int32_t* caps, int ncap, int capacity_padding,
                 int path_wise, int32_t* prefix, const int32_t* threshold, void* scratch,
                 cudaStream_t stream, const GateArgs* gate = nullptr,
                 int32_t* mask_out = nullptr) {
  TileGeom g = make_tile_geom(cell_num, path_num);
  BRT_REQUIRE(g.num_tiles <= 0x7fffffffLL && g.col_chunks <= 65535,
              "mask of %lld x %d cells is too large for one launch", (long long)cell_num,
              path_num);
  // One chained launch when the bit words of a CTA's tiles fit in shared memory, else three
  // launches (pack, scan, expand).  BRT_INDEX_PATH=split forces the latter (for tests).
  static const bool forced_split = [] {
    const char* const forced = getenv("BRT_INDEX_PATH");
    return forced != nullptr && strcmp(forced, "split") == 0;
  }();
  if (gate != nullptr || !forced_split || mode == Mode::kThrottleSeat) {
    int64_t target = (int64_t)sm_count() * kChainCtasPerSm / g.col_chunks;
    if (target < 1) target = 1;
    const int64_t ranges0 = g.num_tiles < target ? g.num_tiles : target;
    const int64_t tiles_per_cta = (g.num_tiles + ranges0 - 1) / ranges0;
    const int64_t ranges = (g.num_tiles + tiles_per_cta - 1) / tiles_per_cta;
    const size_t smem = (tile_smem_ints(g.ec, g.rg, g.pitch, true) +
                         (size_t)tiles_per_cta * g.rg * g.ec +
                         (size_t)g.rg * kGroupRows * g.pitch) *
                        sizeof(int);
    if (smem <= kChainSmemLimit)
      return launch_chain(mode, g, (int)tiles_per_cta, (int)ranges, smem, mask, out, loads,
                          cell_num, path_num, caps, ncap, capacity_padding, path_wise, prefix,
                          threshold, scratch, stream, gate, mask_out);
  }
  if (gate != nullptr)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "%lld x %d scores do not fit the single-launch gate; route in two steps",
                     (long long)cell_num, path_num);
  if (mode == Mode::kThrottleSeat)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "a %lld x %d mask does not fit the single-launch scan; throttle and index "
                     "it in two steps", (long long)cell_num, path_num);
  TiledArgs a;
  char* p = static_cast<char*>(scratch);
  a.flags = reinterpret_cast<int*>(p);
  p += 256;
  a.tile_flags = reinterpret_cast<int*>(p);
  p += round_up((size_t)g.num_tiles * g.col_chunks * 4 + 4, 256);
  a.tile_sums = reinterpret_cast<int*>(p);
  p += round_up((size_t)g.num_tiles * path_num * 4 + 4, 256);
  a.bits = reinterpret_cast<uint32_t*>(p);
  a.mask = mask;
  a.out = out;
  a.mask_out = nullptr;
  a.loads = loads;
  a.counts = t_counts_out;
  a.caps = caps;
  a.ncap = ncap;
  a.capacity_padding = capacity_padding;
  a.path_wise = path_wise;
  a.prefix = prefix;
  a.threshold = threshold;
  a.cell_num = cell_num;
  a.path_num = path_num;
  a.ec = g.ec;
  a.rg = g.rg;
  a.pitch = g.pitch;
  a.num_tiles = g.num_tiles;
  a.chunks = g.col_chunks;

  const dim3 grid((unsigned)g.num_tiles, (unsigned)g.col_chunks);
  const size_t smem_full = tile_smem_ints(g.ec, g.rg, g.pitch, true) * sizeof(int);
  const size_t smem_expand = tile_smem_ints(g.ec, g.rg, g.pitch, false) * sizeof(int);
  if (mode == Mode::kTag)
    BRT_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)cell_num * path_num * 4, stream));

  const KernelTimer timer(mode == Mode::kThrottle ? "throttle_split_kernels" : "index_split_kernels",
                          stream);
  mask_pack_tiled_kernel<<<grid, kTileThreads, smem_full, stream>>>(a), note_launch();
  BRT_LAUNCH_CHECK("mask_pack_tiled_kernel");
  const unsigned scan_grid = (unsigned)((path_num + 3) / 4);
  if (mode == Mode::kThrottle)
    tile_scan_wide_kernel<true><<<scan_grid, 1024, 0, stream>>>(a), note_launch();
  else
    tile_scan_wide_kernel<false><<<scan_grid, 1024, 0, stream>>>(a), note_launch();
  BRT_LAUNCH_CHECK("tile_scan_wide_kernel");
  switch (mode) {
    case Mode::kSeat:
      index_expand_tiled_kernel<Mode::kSeat><<<grid, kTileThreads, smem_expand, stream>>>(a), note_launch();
      break;
    case Mode::kTag:
      index_expand_tiled_kernel<Mode::kTag><<<grid, kTileThreads, smem_expand, stream>>>(a), note_launch();
      break;
    case Mode::kThrottle:
      index_expand_tiled_kernel<Mode::kThrottle><<<grid, kTileThreads, smem_expand, stream>>>(a), note_launch();
      break;
  }
  BRT_LAUNCH_CHECK("index_expand_tiled_kernel");
  return BRT_OK;
}

// ================================================================================ strip path
template <int V>
int launch_scan(Mode mode, const Tiling& tl, const Scratch& sc, const int32_t* mask,
                int32_t* out, int32_t* loads, int64_t cell_num, int path_num,
                const int32_t* caps, int ncap, int capacity_padding, int path_wise,
                int32_t* prefix, const int32_t* threshold, cudaStream_t stream) {
  BRT_CUDA_TRY(cudaMemsetAsync(sc.flags, 0, 256, stream));
  const dim3 grid((unsigned)tl.num_tiles, (unsigned)tl.col_chunks);
  mask_pack_kernel<V><<<grid, kThreads, 0, stream>>>(mask, sc.bits, sc.tile_sums, sc.flags,
                                                     cell_num, path_num, tl.cgb, tl.slices), note_launch();
  BRT_LAUNCH_CHECK("mask_pack_kernel");
  const unsigned scan_grid = (unsigned)((path_num + 31) / 32);
  if (mode == Mode::kThrottle) {
    tile_scan_kernel<true><<<scan_grid, 1024, 0, stream>>>(
        sc.tile_sums, tl.num_tiles, path_num, nullptr, nullptr, 0, 0, 0, prefix, threshold,
        nullptr), note_launch();
  } else {
    tile_scan_kernel<false><<<scan_grid, 1024, 0, stream>>>(
        sc.tile_sums, tl.num_tiles, path_num, loads, caps, ncap, capacity_padding, path_wise,
        nullptr, nullptr, t_counts_out), note_launch();
  }
  BRT_LAUNCH_CHECK("tile_scan_kernel");
  switch (mode) {
    case Mode::kSeat:
      index_expand_kernel<V, Mode::kSeat><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, nullptr, cell_num, path_num, tl.cgb,
          tl.slices), note_launch();
      break;
    case Mode::kTag:
      BRT_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)cell_num * path_num * 4, stream));
      index_expand_kernel<V, Mode::kTag><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, nullptr, cell_num, path_num, tl.cgb,
          tl.slices), note_launch();
      break;
    case Mode::kThrottle:
      index_expand_kernel<V, Mode::kThrottle><<<grid, kThreads, 0, stream>>>(
          mask, sc.bits, sc.tile_sums, sc.flags, out, threshold, cell_num, path_num, tl.cgb,
          tl.slices), note_launch();
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
  if (path_num % 4 == 0 && aligned_to(mask, 16) && aligned_to(out, 16))
    return launch_tiled(mode, mask, out, loads, cell_num, path_num, caps, ncap,
                        capacity_padding, path_wise, prefix, threshold, scratch, stream);
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

// ------------------------------------------------------------------------ fixed scratch
// Scratch for the entry point that must not allocate: lives in the library's image on
// every GPU that loads it, until the process exits.
constexpr size_t kStaticScratchBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_index_scratch[kStaticScratchBytes];

// Device address of the array above for the current device.  The name of a __device__
// array is only a host-side handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static void* cached[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  BRT_CUDA_TRY(cudaGetDevice(&dev));
  BRT_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d is not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    BRT_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_index_scratch));
    BRT_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return BRT_OK;
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
                                           int32_t* loads, int32_t* path_counts,
                                           int64_t cell_num, int path_num,
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
    if (path_counts != nullptr)
      BRT_CUDA_TRY(cudaMemsetAsync(path_counts, 0, (size_t)path_num * 4, st));
    return BRT_OK;
  }
  BRT_REQUIRE(hot_mask != nullptr && indices != nullptr, "hot_mask or indices is null");
  const CountsScope counts(path_counts);
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

BRT_API int brt_throttle_and_generate_indices(
    const int32_t* hot_mask, int32_t* indices, int32_t* loads, int32_t* path_counts,
    int32_t* prefix, const int32_t* threshold, int32_t* throttled_mask, int64_t cell_num,
    int path_num,
    const int32_t* supported_capacities, int supported_capacity_num, int capacity_padding,
    int path_wise_padding, void* scratch, size_t scratch_bytes, void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  BRT_REQUIRE(loads != nullptr && prefix != nullptr && threshold != nullptr,
              "loads, prefix or threshold is null");
  BRT_REQUIRE(supported_capacity_num >= 0 &&
                  (supported_capacity_num == 0 || supported_capacities != nullptr),
              "supported_capacities is null but supported_capacity_num=%d",
              supported_capacity_num);
  BRT_REQUIRE(!capacity_padding || supported_capacity_num >= 1,
              "capacity_padding needs at least one supported capacity");
  const int path_wise = (capacity_padding && path_wise_padding) ? 1 : 0;
  BRT_REQUIRE(!path_wise || supported_capacity_num >= path_num,
              "path_wise_padding needs one capacity per path (%d < %d)", supported_capacity_num,
              path_num);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cell_num == 0) {  // as the two ops it stands for: prefix untouched, loads zero
    BRT_CUDA_TRY(cudaMemsetAsync(loads, 0, (size_t)path_num * 4, st));
    if (path_counts != nullptr)
      BRT_CUDA_TRY(cudaMemsetAsync(path_counts, 0, (size_t)path_num * 4, st));
    return BRT_OK;
  }
  BRT_REQUIRE(hot_mask != nullptr && indices != nullptr, "hot_mask or indices is null");
  if (path_num % 4 != 0 || !aligned_to(hot_mask, 16) || !aligned_to(indices, 16) ||
      !aligned_to(throttled_mask, 16))
    return set_error(BRT_ERR_UNSUPPORTED,
                     "the fused scan needs path_num %% 4 == 0 and 16-byte aligned arrays; "
                     "throttle and index in two steps");
  BRT_REQUIRE(scratch != nullptr && aligned_to(scratch, 256),
              "scratch must be a 256-byte aligned device buffer");
  const size_t need = scratch_bytes_for(cell_num, path_num);
  if (scratch_bytes < need)
    return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                     scratch_bytes, need);
  const CountsScope counts(path_counts);
  return launch_tiled(Mode::kThrottleSeat, hot_mask, indices, loads, cell_num, path_num,
                      supported_capacities, supported_capacity_num, capacity_padding, path_wise,
                      prefix, threshold, scratch, st, nullptr, throttled_mask);
}

BRT_API int brt_route_scores(const float* scores, int64_t cell_num, int path_num, int decision,
                             int top_k, float threshold, int residual_path, int output,
                             int32_t* out, int32_t* loads, int32_t* path_counts,
                             const int32_t* capacities,
                             int capacity_num, int capacity_padding, int path_wise_padding,
                             int32_t* prefix, const int32_t* throttle_capacity, float* gates_out,
                             int32_t* mask_out, void* scratch, size_t scratch_bytes,
                             void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  BRT_REQUIRE(decision == BRT_GATE_TOPK || decision == BRT_GATE_THRESHOLD, "unknown decision %d",
              decision);
  BRT_REQUIRE(decision != BRT_GATE_TOPK || (top_k >= 1 && top_k <= path_num),
              "top_k=%d outside [1, %d]", top_k, path_num);
  BRT_REQUIRE(residual_path < path_num, "residual_path=%d outside the %d paths", residual_path,
              path_num);
  BRT_REQUIRE(output == BRT_ROUTE_MASK || output == BRT_ROUTE_THROTTLED_MASK ||
                  output == BRT_ROUTE_SEAT_INDICES || output == BRT_ROUTE_THROTTLED_SEAT_INDICES,
              "unknown output %d", output);
  const bool throttles =
      output == BRT_ROUTE_THROTTLED_MASK || output == BRT_ROUTE_THROTTLED_SEAT_INDICES;
  BRT_REQUIRE(!throttles || (prefix != nullptr && throttle_capacity != nullptr),
              "a throttled output needs prefix and throttle_capacity");
  BRT_REQUIRE(output == BRT_ROUTE_THROTTLED_MASK || loads != nullptr, "loads is null");
  BRT_REQUIRE(capacity_num >= 0 && (capacity_num == 0 || capacities != nullptr),
              "capacities missing");
  // the same rules as brt_generate_indices_and_loads: padding needs a capacity to pad to, and
  // path-wise padding only exists inside capacity padding
  BRT_REQUIRE(!capacity_padding || capacity_num >= 1,
              "capacity_padding needs at least one supported capacity");
  path_wise_padding = (capacity_padding && path_wise_padding) ? 1 : 0;
  BRT_REQUIRE(!path_wise_padding || capacity_num >= path_num,
              "path_wise_padding needs one capacity per path (%d < %d)", capacity_num, path_num);
  BRT_REQUIRE(path_counts == nullptr || output == BRT_ROUTE_SEAT_INDICES ||
                  output == BRT_ROUTE_THROTTLED_SEAT_INDICES,
              "path_counts goes with the seat-index outputs only");
  if (cell_num == 0) {
    if (output != BRT_ROUTE_THROTTLED_MASK)
      BRT_CUDA_TRY(cudaMemsetAsync(loads, 0, (size_t)path_num * 4, static_cast<cudaStream_t>(stream)));
    if (path_counts != nullptr)
      BRT_CUDA_TRY(cudaMemsetAsync(path_counts, 0, (size_t)path_num * 4,
                                   static_cast<cudaStream_t>(stream)));
    return BRT_OK;
  }
  BRT_REQUIRE(scores != nullptr && out != nullptr, "scores or out is null");
  BRT_REQUIRE(mask_out == nullptr || output == BRT_ROUTE_THROTTLED_SEAT_INDICES ||
                  output == BRT_ROUTE_SEAT_INDICES,
              "mask_out goes with the seat-index outputs only");
  if (path_num % 4 != 0 || path_num > 256 || !aligned_to(scores, 16) || !aligned_to(out, 16) ||
      !aligned_to(mask_out, 16) || (gates_out != nullptr && !aligned_to(gates_out, 4)))
    return set_error(BRT_ERR_UNSUPPORTED,
                     "the single-launch gate needs path_num %% 4 == 0, path_num <= 256 and "
                     "16-byte aligned arrays; route in two steps");
  BRT_REQUIRE(scratch != nullptr && aligned_to(scratch, 256),
              "scratch must be a 256-byte aligned device buffer");
  const size_t need = scratch_bytes_for(cell_num, path_num);
  if (scratch_bytes < need)
    return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                     scratch_bytes, need);
  const GateArgs gate{decision == BRT_GATE_TOPK ? 1 : 2, top_k, threshold, residual_path, gates_out};
  const Mode mode = output == BRT_ROUTE_MASK ? Mode::kMask
                    : output == BRT_ROUTE_THROTTLED_MASK ? Mode::kThrottle
                    : output == BRT_ROUTE_THROTTLED_SEAT_INDICES ? Mode::kThrottleSeat
                                                                 : Mode::kSeat;
  const CountsScope counts(path_counts);
  return launch_tiled(mode, reinterpret_cast<const int32_t*>(scores), out, loads, cell_num,
                      path_num, capacities, capacity_num, capacity_padding, path_wise_padding,
                      prefix, throttle_capacity, scratch, static_cast<cudaStream_t>(stream), &gate,
                      mask_out);
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
                                                              cell_num, path_num), note_launch();
  } else {
    seat_to_tag_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(origin_indices, new_indices,
                                                              cell_num, path_num), note_launch();
  }
  BRT_LAUNCH_CHECK("convert_index_format");
  return BRT_OK;
}

BRT_API size_t brt_static_index_scratch_bytes(void) { return kStaticScratchBytes; }

BRT_API int brt_generate_indices_and_loads_static(const int32_t* hot_mask, int32_t* indices,
                                                  int32_t* loads, int64_t cell_num, int path_num,
                                                  const int32_t* supported_capacities,
                                                  int supported_capacity_num,
                                                  int capacity_padding, int path_wise_padding,
                                                  int is_tag_index, void* stream) {
  clear_error();
  BRT_REQUIRE(cell_num >= 0 && path_num > 0, "bad shape: cell_num=%lld path_num=%d",
              (long long)cell_num, path_num);
  const size_t need = scratch_bytes_for(cell_num, path_num);
  if (need > kStaticScratchBytes)
    return set_error(BRT_ERR_SCRATCH_TOO_SMALL,
                     "a %lld x %d mask needs %zu bytes of scratch; the built-in scratch of "
                     "this entry point holds %zu bytes (use brt_generate_indices_and_loads "
                     "with caller-provided scratch for larger masks)",
                     (long long)cell_num, path_num, need, kStaticScratchBytes);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != BRT_OK) return rc;
  t_may_allocate = false;  // the status word of brt_index_status is used only if it exists
  const int out = brt_generate_indices_and_loads(hot_mask, indices, loads, nullptr, cell_num,
                                                 path_num,
                                                 supported_capacities, supported_capacity_num,
                                                 capacity_padding, path_wise_padding,
                                                 is_tag_index, scratch, kStaticScratchBytes,
                                                 stream);
  t_may_allocate = true;
  return out;
}

BRT_API int brt_index_status(void) {
  index_status_word(true);
  HostStatus& s = index_status();
  return s.host != nullptr ? *reinterpret_cast<volatile int*>(s.host) : BRT_OK;
}

BRT_API void brt_index_status_reset(void) {
  HostStatus& s = index_status();
  if (s.host != nullptr) *reinterpret_cast<volatile int*>(s.host) = BRT_OK;
}

BRT_API void brt_index_set_test_hooks(int spin_limit, int skip_first_run) {
  g_spin_limit.store(spin_limit > 0 ? spin_limit : kChainSpinLimit);
  g_first_ticket.store(skip_first_run ? 1 : 0);
}

}  // extern "C"
