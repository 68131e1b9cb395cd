// Token dispatch and weighted combine for sm_100a.
//
// Both are pure data movement, so the design goal is HBM traffic equal to the
// algorithmic minimum:
//
//   dispatch : source-major.  One warp owns (cell, 2 KB piece of the row): it reads the
//              cell's index row once, keeps the piece in registers and stores it to every
//              path that kept the cell, so a source row crosses HBM once however many
//              copies are made.  All accesses are 16 bytes per lane (narrower only when the
//              row size or a pointer is not 16-byte aligned).  Rows of the output that no
//              cell lands on (capacity padding, dropped seats) are found through a byte map
//              that the copy pass marks, and are written as zeros by a second launch: the
//              output is never memset as a whole and no row is written twice.
//   combine  : destination-major.  One warp owns (cell, piece): it walks the cell's kept
//              routes in ascending path order, accumulates in fp32 registers with separate
//              multiply and add roundings (the order and rounding of the reference's
//              atomicAdd sequence, without atomics) and writes the row once.
//
// Per-path base rows (prefix sum of loads, or e * max_path_load) are computed once per
// CTA into shared memory instead of once per thread.
#include "common.cuh"

#include <initializer_list>

namespace brt_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;                 // vectors per lane per piece
constexpr int kPieceVecs = 32 * kUnroll;   // vectors per piece
constexpr int kMaxPaths = 4096;

// s_loads[e], s_base[e] for every path; called by all threads of the CTA.
__device__ __forceinline__ void setup_paths(const int* __restrict__ loads, int path_num,
                                            int max_path_load, int* s_loads, int* s_base) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int p = 0; p < path_num; p += 32) {
      const int e = p + lane;
      const int v = e < path_num ? loads[e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (e < path_num) {
        s_loads[e] = v;
        s_base[e] = max_path_load != 0 ? e * max_path_load : carry + incl - v;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
}

template <int VB, int DT>
struct Lanes {
  using V = typename Chunk<VB>::type;
  using E = typename Elem<DT>::type;
  static constexpr int N = VB / (int)sizeof(E);
};

// x * g element-wise in the storage type: exact product in fp32, one rounding.
template <int VB, int DT>
__device__ __forceinline__ typename Chunk<VB>::type scale_chunk(typename Chunk<VB>::type x,
                                                                float g) {
  using L = Lanes<VB, DT>;
  alignas(VB) typename L::E e[L::N];
  *reinterpret_cast<typename L::V*>(e) = x;
#pragma unroll
  for (int i = 0; i < L::N; i++)
    e[i] = Elem<DT>::from_f32(__fmul_rn(Elem<DT>::to_f32(e[i]), g));
  return *reinterpret_cast<typename L::V*>(e);
}

struct DispatchArgs {
  const void* src;
  void* dst;
  const void* gates;
  const int* indices;
  const int* loads;
  const int* old_tags;
  int* new_tags;
  unsigned char* row_marks;
  int64_t cell_num;
  int64_t row_vecs;       // vectors per row
  int64_t pieces_per_row;
  int path_num;
  int max_path_load;
  int64_t total_rows;
};

// ---------------------------------------------------------------------------------- dispatch
template <int VB, int DT, bool WEIGHTED, bool IS_1D>
__global__ void __launch_bounds__(kThreads) dispatch_seat_kernel(const DispatchArgs a) {
  using V = typename Chunk<VB>::type;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;

  for (int64_t item = warp; item < items; item += warps) {
    const int64_t cell = item / a.pieces_per_row;
    const int64_t piece = item - cell * a.pieces_per_row;
    const int64_t v0 = piece * kPieceVecs + lane;
    V regs[kUnroll];
    bool loaded = false;
    for (int p = 0; p < E; p += 32) {
      const int e_lane = p + lane;
      int seat = 0;
      if (e_lane < E) seat = a.indices[cell * E + e_lane];
      const bool keep = e_lane < E && seat > 0 && seat <= s_loads[e_lane];
      float gate = 0.f;
      if constexpr (WEIGHTED) {
        if (keep)
          gate = Elem<DT>::to_f32(
              static_cast<const typename Elem<DT>::type*>(a.gates)[cell * E + e_lane]);
      }
      unsigned ballot = __ballot_sync(0xffffffffu, keep);
      while (ballot) {
        const int b = __ffs(ballot) - 1;
        ballot &= ballot - 1;
        const int e = p + b;
        const int seat_b = __shfl_sync(0xffffffffu, seat, b);
        const int64_t row = (int64_t)s_base[e] + seat_b - 1;
        if (!IS_1D || !loaded) {
          const int64_t src_row = IS_1D ? cell : cell * E + e;
          const V* sp = src + src_row * a.row_vecs;
#pragma unroll
          for (int u = 0; u < kUnroll; u++) {
            const int64_t v = v0 + u * 32;
            if (v < a.row_vecs) regs[u] = load_stream(sp + v);
          }
          loaded = true;
        }
        V* dp = dst + row * a.row_vecs;
        if constexpr (WEIGHTED) {
          const float g = __shfl_sync(0xffffffffu, gate, b);
#pragma unroll
          for (int u = 0; u < kUnroll; u++) {
            const int64_t v = v0 + u * 32;
            if (v < a.row_vecs) store_stream(dp + v, scale_chunk<VB, DT>(regs[u], g));
          }
        } else {
#pragma unroll
          for (int u = 0; u < kUnroll; u++) {
            const int64_t v = v0 + u * 32;
            if (v < a.row_vecs) store_stream(dp + v, regs[u]);
          }
        }
        if (piece == 0 && lane == 0) {
          a.row_marks[row] = 1;
          if (a.new_tags != nullptr) a.new_tags[row] = a.old_tags[cell];
        }
      }
    }
  }
}

// Writes zeros to every row (and tag) the copy pass did not mark.
template <int VB>
__global__ void __launch_bounds__(kThreads) dispatch_zero_fill_kernel(const DispatchArgs a) {
  using V = typename Chunk<VB>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.total_rows * a.pieces_per_row;
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const V zero = zero_chunk<V>();
  for (int64_t item = warp; item < items; item += warps) {
    const int64_t row = item / a.pieces_per_row;
    const int64_t piece = item - row * a.pieces_per_row;
    if (a.row_marks[row] != 0) continue;
    V* dp = dst + row * a.row_vecs;
    const int64_t v0 = piece * kPieceVecs + lane;
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const int64_t v = v0 + u * 32;
      if (v < a.row_vecs) store_stream(dp + v, zero);
    }
    if (piece == 0 && lane == 0 && a.new_tags != nullptr) a.new_tags[row] = 0;
  }
}

// Tag-index dispatch: output-major.  One warp owns (output row, piece); row i of path e
// pulls cell tag-1 when i < loads[e] and the tag is non-zero, otherwise it is zeroed.
template <int VB, int DT, bool WEIGHTED, bool IS_1D>
__global__ void __launch_bounds__(kThreads) dispatch_tag_kernel(const DispatchArgs a) {
  using V = typename Chunk<VB>::type;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.total_rows * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;
  const V zero = zero_chunk<V>();

  for (int64_t item = warp; item < items; item += warps) {
    const int64_t row = item / a.pieces_per_row;
    const int64_t piece = item - row * a.pieces_per_row;
    // path of this row: last e with s_base[e] <= row (binary search; equal bases of empty
    // paths resolve to the last one, whose slot is the one that contains the row)
    int lo = 0, hi = E - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((int64_t)s_base[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int e = lo;
    const int64_t i = row - s_base[e];
    int tag = 0;
    if (i < s_loads[e] && i < a.cell_num) tag = a.indices[i * E + e];
    const int64_t cell = (int64_t)tag - 1;
    const bool pull = tag != 0 && cell >= 0 && cell < a.cell_num;
    V* dp = dst + row * a.row_vecs;
    const int64_t v0 = piece * kPieceVecs + lane;
    if (pull) {
      const int64_t src_row = IS_1D ? cell : cell * E + e;
      const V* sp = src + src_row * a.row_vecs;
      V regs[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) regs[u] = load_stream(sp + v);
      }
      float g = 1.f;
      if constexpr (WEIGHTED)
        g = Elem<DT>::to_f32(static_cast<const typename Elem<DT>::type*>(a.gates)[cell * E + e]);
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) {
          if constexpr (WEIGHTED)
            store_stream(dp + v, scale_chunk<VB, DT>(regs[u], g));
          else
            store_stream(dp + v, regs[u]);
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) store_stream(dp + v, zero);
      }
    }
    if (piece == 0 && lane == 0 && a.new_tags != nullptr)
      a.new_tags[row] = pull ? a.old_tags[cell] : 0;
  }
}

// ---------------------------------------------------------------------------------- combine
struct CombineArgs {
  const void* src;
  void* dst;
  const void* gates;
  const int* indices;
  const int* loads;
  int64_t cell_num;
  int64_t row_vecs;
  int64_t pieces_per_row;
  int path_num;
  int max_path_load;
  int is_residual;
};

// GMODE: 0 = no gates, 1 = fp32 gates, 2 = gates stored in the data type.
template <int VB, int DT, int GMODE>
__global__ void __launch_bounds__(kThreads) combine_seat_kernel(const CombineArgs a) {
  using L = Lanes<VB, DT>;
  using V = typename L::V;
  extern __shared__ int s_mem[];
  int* s_loads = s_mem;
  int* s_base = s_mem + a.path_num;
  setup_paths(a.loads, a.path_num, a.max_path_load, s_loads, s_base);

  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  const int64_t items = a.cell_num * a.pieces_per_row;
  const V* __restrict__ src = static_cast<const V*>(a.src);
  V* __restrict__ dst = static_cast<V*>(a.dst);
  const int E = a.path_num;

  for (int64_t item = warp; item < items; item += warps) {
    const int64_t cell = item / a.pieces_per_row;
    const int64_t piece = item - cell * a.pieces_per_row;
    const int64_t v0 = piece * kPieceVecs + lane;
    float acc[kUnroll][L::N];
#pragma unroll
    for (int u = 0; u < kUnroll; u++)
#pragma unroll
      for (int i = 0; i < L::N; i++) acc[u][i] = 0.f;
    bool routed = false;
    for (int p = 0; p < E; p += 32) {
      const int e_lane = p + lane;
      int seat = 0;
      if (e_lane < E) seat = a.indices[cell * E + e_lane];
      const bool keep = e_lane < E && seat > 0 && seat <= s_loads[e_lane];
      float gate = 1.f;
      if constexpr (GMODE == 1) {
        if (keep) gate = static_cast<const float*>(a.gates)[cell * E + e_lane];
      } else if constexpr (GMODE == 2) {
        if (keep)
          gate = Elem<DT>::to_f32(
              static_cast<const typename Elem<DT>::type*>(a.gates)[cell * E + e_lane]);
      }
      unsigned ballot = __ballot_sync(0xffffffffu, keep);
      while (ballot) {
        const int b = __ffs(ballot) - 1;
        ballot &= ballot - 1;
        const int e = p + b;
        const int seat_b = __shfl_sync(0xffffffffu, seat, b);
        const float g = __shfl_sync(0xffffffffu, gate, b);
        const int64_t row = (int64_t)s_base[e] + seat_b - 1;
        const V* sp = src + row * a.row_vecs;
        V regs[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
          const int64_t v = v0 + u * 32;
          if (v < a.row_vecs) regs[u] = load_stream(sp + v);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
          const int64_t v = v0 + u * 32;
          if (v < a.row_vecs) {
            alignas(VB) typename L::E el[L::N];
            *reinterpret_cast<V*>(el) = regs[u];
#pragma unroll
            for (int i = 0; i < L::N; i++) {
              float x = Elem<DT>::to_f32(el[i]);
              if constexpr (GMODE != 0) x = __fmul_rn(x, g);
              acc[u][i] = __fadd_rn(acc[u][i], x);
            }
          }
        }
        routed = true;
      }
    }
    if (routed || !a.is_residual) {
      V* dp = dst + cell * a.row_vecs;
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int64_t v = v0 + u * 32;
        if (v < a.row_vecs) {
          alignas(VB) typename L::E el[L::N];
#pragma unroll
          for (int i = 0; i < L::N; i++) el[i] = Elem<DT>::from_f32(acc[u][i]);
          store_stream(dp + v, *reinterpret_cast<V*>(el));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------- launch
int pick_vec_bytes(int64_t row_bytes, std::initializer_list<const void*> ptrs, int min_bytes) {
  for (int vb : {16, 8, 4, 2}) {
    if (vb < min_bytes) break;
    if (row_bytes % vb != 0) continue;
    bool ok = true;
    for (const void* p : ptrs)
      if (p != nullptr && !aligned_to(p, vb)) ok = false;
    if (ok) return vb;
  }
  return 0;
}

unsigned grid_for(int64_t items) {
  int64_t blocks = (items + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

template <int VB, int DT, bool WEIGHTED, bool IS_1D>
void launch_dispatch(const DispatchArgs& a, bool is_tag, cudaStream_t st) {
  const size_t smem = (size_t)a.path_num * 2 * sizeof(int);
  if (is_tag) {
    dispatch_tag_kernel<VB, DT, WEIGHTED, IS_1D>
        <<<grid_for(a.total_rows * a.pieces_per_row), kThreads, smem, st>>>(a);
  } else {
    dispatch_seat_kernel<VB, DT, WEIGHTED, IS_1D>
        <<<grid_for(a.cell_num * a.pieces_per_row), kThreads, smem, st>>>(a);
  }
}

template <int VB>
int dispatch_by_flags(const DispatchArgs& a, int dtype, bool weighted, bool is_1d, bool is_tag,
                      cudaStream_t st) {
  if (!weighted) {
    // an unweighted move is a byte copy: the element type does not matter
    if (is_1d)
      launch_dispatch<VB, BRT_BF16, false, true>(a, is_tag, st);
    else
      launch_dispatch<VB, BRT_BF16, false, false>(a, is_tag, st);
    return BRT_OK;
  }
  if (dtype == BRT_F32) {
    if constexpr (VB >= 4) {
      launch_dispatch<VB, BRT_F32, true, true>(a, is_tag, st);
      return BRT_OK;
    }
    return set_error(BRT_ERR_INVALID_ARGUMENT, "fp32 rows must be 4-byte aligned");
  }
  if (dtype == BRT_F16)
    launch_dispatch<VB, BRT_F16, true, true>(a, is_tag, st);
  else
    launch_dispatch<VB, BRT_BF16, true, true>(a, is_tag, st);
  return BRT_OK;
}

template <int VB>
void launch_zero_fill(const DispatchArgs& a, cudaStream_t st) {
  dispatch_zero_fill_kernel<VB>
      <<<grid_for(a.total_rows * a.pieces_per_row), kThreads, 0, st>>>(a);
}

template <int VB, int DT>
int combine_by_gates(const CombineArgs& a, int gmode, cudaStream_t st) {
  const size_t smem = (size_t)a.path_num * 2 * sizeof(int);
  const unsigned grid = grid_for(a.cell_num * a.pieces_per_row);
  switch (gmode) {
    case 0:
      combine_seat_kernel<VB, DT, 0><<<grid, kThreads, smem, st>>>(a);
      break;
    case 1:
      combine_seat_kernel<VB, DT, 1><<<grid, kThreads, smem, st>>>(a);
      break;
    default:
      if constexpr (DT == BRT_F32)
        combine_seat_kernel<VB, DT, 1><<<grid, kThreads, smem, st>>>(a);
      else
        combine_seat_kernel<VB, DT, 2><<<grid, kThreads, smem, st>>>(a);
      break;
  }
  return BRT_OK;
}

template <int VB>
int combine_by_dtype(const CombineArgs& a, int dtype, int gmode, cudaStream_t st) {
  if (dtype == BRT_F32) {
    if constexpr (VB >= 4) return combine_by_gates<VB, BRT_F32>(a, gmode, st);
    return set_error(BRT_ERR_INVALID_ARGUMENT, "fp32 rows must be 4-byte aligned");
  }
  if (dtype == BRT_F16) return combine_by_gates<VB, BRT_F16>(a, gmode, st);
  return combine_by_gates<VB, BRT_BF16>(a, gmode, st);
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API size_t brt_dispatch_scratch_bytes(int64_t total_rows, int path_num) {
  (void)path_num;
  if (total_rows < 0) total_rows = 0;
  return round_up((size_t)total_rows + 1, 256);
}

BRT_API int brt_dispatch_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, const int32_t* old_tags, int32_t* new_tags, int64_t cell_num,
    int64_t cell_size, int path_num, int32_t max_path_load, int64_t total_rows,
    int is_1d_routing, int is_tag_index, int dtype, void* scratch, size_t scratch_bytes,
    void* stream) {
  clear_error();
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(cell_num >= 0 && cell_size >= 0 && total_rows >= 0, "negative size");
  BRT_REQUIRE(path_num > 0 && path_num <= kMaxPaths, "path_num %d outside [1, %d]", path_num,
              kMaxPaths);
  BRT_REQUIRE(max_path_load >= 0, "negative max_path_load");
  BRT_REQUIRE(total_rows <= 0x7fffffffLL, "more than 2^31-1 output rows");
  BRT_REQUIRE((old_tags == nullptr) == (new_tags == nullptr),
              "old_tags and new_tags must be given together");
  BRT_REQUIRE(gates == nullptr || is_1d_routing, "gates are only supported with 1-D routing");
  if (total_rows == 0 || cell_size == 0) return BRT_OK;
  BRT_REQUIRE(dst_data != nullptr && route_indices != nullptr && loads != nullptr,
              "null pointer argument");
  BRT_REQUIRE(cell_num == 0 || src_data != nullptr, "src_data is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int es = dtype_size(dtype);
  const int64_t row_bytes = cell_size * es;
  const int vb = pick_vec_bytes(row_bytes, {src_data, dst_data}, gates != nullptr ? es : 2);
  BRT_REQUIRE(vb != 0, "rows of %lld bytes cannot be moved: misaligned pointers",
              (long long)row_bytes);

  DispatchArgs a;
  a.src = src_data;
  a.dst = dst_data;
  a.gates = gates;
  a.indices = route_indices;
  a.loads = loads;
  a.old_tags = old_tags;
  a.new_tags = new_tags;
  a.row_marks = static_cast<unsigned char*>(scratch);
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / vb;
  a.pieces_per_row = (a.row_vecs + kPieceVecs - 1) / kPieceVecs;
  a.path_num = path_num;
  a.max_path_load = max_path_load;
  a.total_rows = total_rows;

  const bool is_tag = is_tag_index != 0;
  if (!is_tag) {
    const size_t need = brt_dispatch_scratch_bytes(total_rows, path_num);
    BRT_REQUIRE(scratch != nullptr, "scratch is null");
    if (scratch_bytes < need)
      return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                       scratch_bytes, need);
    BRT_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)total_rows, st));
  }
  int rc = BRT_OK;
  if (cell_num > 0 || is_tag) {
    switch (vb) {
      case 16: rc = dispatch_by_flags<16>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      case 8: rc = dispatch_by_flags<8>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      case 4: rc = dispatch_by_flags<4>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
      default: rc = dispatch_by_flags<2>(a, dtype, gates != nullptr, is_1d_routing != 0, is_tag, st); break;
    }
    if (rc != BRT_OK) return rc;
    BRT_LAUNCH_CHECK("dispatch kernel");
  }
  if (!is_tag) {
    switch (vb) {
      case 16: launch_zero_fill<16>(a, st); break;
      case 8: launch_zero_fill<8>(a, st); break;
      case 4: launch_zero_fill<4>(a, st); break;
      default: launch_zero_fill<2>(a, st); break;
    }
    BRT_LAUNCH_CHECK("dispatch_zero_fill_kernel");
  }
  return BRT_OK;
}

BRT_API int brt_combine_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, int64_t cell_num, int64_t cell_size, int path_num,
    int32_t max_path_load, int is_residual, int dtype, int gates_dtype, void* stream) {
  clear_error();
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(gates == nullptr || gates_dtype == BRT_F32 || gates_dtype == dtype,
              "gates must be fp32 or match the data type");
  BRT_REQUIRE(cell_num >= 0 && cell_size >= 0, "negative size");
  BRT_REQUIRE(path_num > 0 && path_num <= kMaxPaths, "path_num %d outside [1, %d]", path_num,
              kMaxPaths);
  BRT_REQUIRE(max_path_load >= 0, "negative max_path_load");
  if (cell_num == 0 || cell_size == 0) return BRT_OK;
  BRT_REQUIRE(dst_data != nullptr && route_indices != nullptr && loads != nullptr,
              "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype_size(dtype);
  const int64_t row_bytes = cell_size * es;
  const int vb = pick_vec_bytes(row_bytes, {src_data, dst_data}, es);
  BRT_REQUIRE(vb != 0, "rows of %lld bytes cannot be moved: misaligned pointers",
              (long long)row_bytes);
  CombineArgs a;
  a.src = src_data;
  a.dst = dst_data;
  a.gates = gates;
  a.indices = route_indices;
  a.loads = loads;
  a.cell_num = cell_num;
  a.row_vecs = row_bytes / vb;
  a.pieces_per_row = (a.row_vecs + kPieceVecs - 1) / kPieceVecs;
  a.path_num = path_num;
  a.max_path_load = max_path_load;
  a.is_residual = is_residual;
  const int gmode = gates == nullptr ? 0 : (gates_dtype == BRT_F32 ? 1 : 2);
  int rc;
  switch (vb) {
    case 16: rc = combine_by_dtype<16>(a, dtype, gmode, st); break;
    case 8: rc = combine_by_dtype<8>(a, dtype, gmode, st); break;
    case 4: rc = combine_by_dtype<4>(a, dtype, gmode, st); break;
    default: rc = combine_by_dtype<2>(a, dtype, gmode, st); break;
  }
  if (rc != BRT_OK) return rc;
  BRT_LAUNCH_CHECK("combine_seat_kernel");
  return BRT_OK;
}

}  // extern "C"
