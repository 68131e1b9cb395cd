// Sum of rows by destination index: out[o] = sum of in[r] over the rows r with index[r] == o,
// added in ascending r.  This is the tag-index branch of combine (the reference's binding
// does it with torch: scatter_reduce("sum") over the inverse indices of unique(tags),
// src/backend/torch/router.cc:449-459; its launcher refuses tag indices,
// src/router/route.cu:519-521).
//
// Destination-major and deterministic: the rows are first grouped by destination (count,
// scan, fill, per-destination sort of the usually very short lists), then one thread per
// 16-byte piece of a destination row walks that row's list, accumulates in fp32 in ascending
// source order and writes the piece once.  Every input row is read once, every output row is
// written once (rows nobody points at as zeros); no atomics on data, no pre-zeroed output.
#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
index_count_kernel(const int* __restrict__ index, int64_t rows_in, int64_t rows_out,
                   int* __restrict__ seg /* [rows_out + 1], zeroed */) {
  for (int64_t r = (int64_t)blockIdx.x * kThreads + threadIdx.x; r < rows_in;
       r += (int64_t)gridDim.x * kThreads) {
    const int o = index[r];
    if (o >= 0 && o < rows_out) atomicAdd(&seg[o + 1], 1);
  }
}

// In-place inclusive scan of seg[0 .. n] (seg[0] == 0) by one CTA, so that seg[o] becomes the
// first list slot of destination o; cursor[o] starts at the same value.
__global__ void __launch_bounds__(1024)
index_scan_kernel(int* __restrict__ seg, int* __restrict__ cursor, int64_t n) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int64_t base = 0; base <= n; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const int v = i <= n ? seg[i] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = s_carry;
    for (int w = 0; w < warp; w++) before += s_warp[w];
    const int mine = before + incl;
    if (i <= n) {
      seg[i] = mine;
      if (i < n) cursor[i] = mine;
    }
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = mine;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
index_fill_kernel(const int* __restrict__ index, int64_t rows_in, int64_t rows_out,
                  int* __restrict__ cursor, int* __restrict__ list) {
  for (int64_t r = (int64_t)blockIdx.x * kThreads + threadIdx.x; r < rows_in;
       r += (int64_t)gridDim.x * kThreads) {
    const int o = index[r];
    if (o >= 0 && o < rows_out) list[atomicAdd(&cursor[o], 1)] = (int)r;
  }
}

// The fill order inside a destination's list depends on scheduling; sort every list so the
// sums are taken in ascending source order (lists hold one entry per path at most in the
// router's use, so an insertion sort by one thread is the cheapest).
__global__ void __launch_bounds__(kThreads)
index_sort_kernel(const int* __restrict__ seg, int* __restrict__ list, int64_t rows_out) {
  for (int64_t o = (int64_t)blockIdx.x * kThreads + threadIdx.x; o < rows_out;
       o += (int64_t)gridDim.x * kThreads) {
    const int lo = seg[o], hi = seg[o + 1];
    for (int i = lo + 1; i < hi; i++) {
      const int v = list[i];
      int j = i - 1;
      while (j >= lo && list[j] > v) {
        list[j + 1] = list[j];
        j--;
      }
      list[j + 1] = v;
    }
  }
}

// VB-byte pieces: one thread per (destination row, piece).
template <int DT, int VB>
__global__ void __launch_bounds__(kThreads)
row_sum_kernel(const void* __restrict__ in, void* __restrict__ out,
               const int* __restrict__ seg, const int* __restrict__ list, int64_t rows_out,
               int64_t row_vecs) {
  using T = typename Elem<DT>::type;
  using V = typename Chunk<VB>::type;
  constexpr int N = VB / (int)sizeof(T);
  const V* __restrict__ src = static_cast<const V*>(in);
  V* __restrict__ dst = static_cast<V*>(out);
  const int64_t items = rows_out * row_vecs;
  for (int64_t it = (int64_t)blockIdx.x * kThreads + threadIdx.x; it < items;
       it += (int64_t)gridDim.x * kThreads) {
    const int64_t o = it / row_vecs;
    const int64_t v = it - o * row_vecs;
    float acc[N];
#pragma unroll
    for (int i = 0; i < N; i++) acc[i] = 0.f;
    const int lo = seg[o], hi = seg[o + 1];
    for (int k = lo; k < hi; k++) {
      const V piece = load_stream(src + (int64_t)list[k] * row_vecs + v);
      const T* e = reinterpret_cast<const T*>(&piece);
#pragma unroll
      for (int i = 0; i < N; i++) acc[i] = __fadd_rn(acc[i], Elem<DT>::to_f32(e[i]));
    }
    V res;
    T* e = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int i = 0; i < N; i++) e[i] = Elem<DT>::from_f32(acc[i]);
    store_stream(dst + it, res);
  }
}

size_t group_scratch_bytes(int64_t rows_in, int64_t rows_out) {
  return round_up((size_t)(rows_out + 1) * 4, 256) + round_up((size_t)rows_out * 4 + 4, 256) +
         round_up((size_t)rows_in * 4 + 4, 256);
}

template <int DT>
void launch_row_sum(int vb, const void* in, void* out, const int* seg, const int* list,
                    int64_t rows_out, int64_t row_bytes, cudaStream_t st) {
  const int64_t row_vecs = row_bytes / vb;
  int64_t blocks = (rows_out * row_vecs + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const KernelTimer timer("row_sum_kernel", st);
  constexpr int kElem = DT == BRT_F32 ? 4 : 2;
  if (vb == 16)
    row_sum_kernel<DT, 16><<<(unsigned)blocks, kThreads, 0, st>>>(in, out, seg, list, rows_out,
                                                                   row_vecs), note_launch();
  else
    row_sum_kernel<DT, kElem><<<(unsigned)blocks, kThreads, 0, st>>>(in, out, seg, list, rows_out,
                                                                      row_vecs), note_launch();
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

BRT_API size_t brt_sum_rows_scratch_bytes(int64_t rows_in, int64_t rows_out) {
  if (rows_in < 0 || rows_out < 0) return 0;
  return group_scratch_bytes(rows_in, rows_out);
}

BRT_API int brt_sum_rows_by_index(const void* in_rows, const int32_t* row_index, void* out_rows,
                                  int64_t rows_in, int64_t rows_out, int64_t cell_size,
                                  int dtype, void* scratch, size_t scratch_bytes, void* stream) {
  clear_error();
  BRT_REQUIRE(dtype == BRT_F32 || dtype == BRT_F16 || dtype == BRT_BF16, "bad dtype %d", dtype);
  BRT_REQUIRE(rows_in >= 0 && rows_out >= 0 && cell_size >= 0, "negative size");
  BRT_REQUIRE(rows_in <= 0x7fffffffLL && rows_out <= 0x7ffffffeLL, "too many rows");
  if (rows_out == 0 || cell_size == 0) return BRT_OK;
  BRT_REQUIRE(out_rows != nullptr && (rows_in == 0 || (in_rows != nullptr && row_index != nullptr)),
              "null pointer argument");
  BRT_REQUIRE(scratch != nullptr && aligned_to(scratch, 256),
              "scratch must be a 256-byte aligned device buffer");
  const size_t need = group_scratch_bytes(rows_in, rows_out);
  if (scratch_bytes < need)
    return set_error(BRT_ERR_SCRATCH_TOO_SMALL, "scratch holds %zu bytes, %zu needed",
                     scratch_bytes, need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* p = static_cast<char*>(scratch);
  int* seg = reinterpret_cast<int*>(p);
  p += round_up((size_t)(rows_out + 1) * 4, 256);
  int* cursor = reinterpret_cast<int*>(p);
  p += round_up((size_t)rows_out * 4 + 4, 256);
  int* list = reinterpret_cast<int*>(p);
  BRT_CUDA_TRY(cudaMemsetAsync(seg, 0, (size_t)(rows_out + 1) * 4, st));
  int64_t blocks = (rows_in + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  index_count_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(row_index, rows_in, rows_out, seg),
      note_launch();
  index_scan_kernel<<<1, 1024, 0, st>>>(seg, cursor, rows_out), note_launch();
  index_fill_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(row_index, rows_in, rows_out, cursor,
                                                           list),
      note_launch();
  int64_t sort_blocks = (rows_out + kThreads - 1) / kThreads;
  if (sort_blocks > cap) sort_blocks = cap;
  index_sort_kernel<<<(unsigned)sort_blocks, kThreads, 0, st>>>(seg, list, rows_out),
      note_launch();
  BRT_LAUNCH_CHECK("row grouping kernels");
  const int es = dtype_size(dtype);
  const int64_t row_bytes = cell_size * es;
  const int vb = (row_bytes % 16 == 0 && aligned_to(in_rows, 16) && aligned_to(out_rows, 16))
                     ? 16
                     : es;
  BRT_REQUIRE(aligned_to(in_rows, es) && aligned_to(out_rows, es), "misaligned rows");
  switch (dtype) {
    case BRT_F32: launch_row_sum<BRT_F32>(vb, in_rows, out_rows, seg, list, rows_out, row_bytes, st); break;
    case BRT_F16: launch_row_sum<BRT_F16>(vb, in_rows, out_rows, seg, list, rows_out, row_bytes, st); break;
    default: launch_row_sum<BRT_BF16>(vb, in_rows, out_rows, seg, list, rows_out, row_bytes, st); break;
  }
  BRT_LAUNCH_CHECK("row_sum_kernel");
  return BRT_OK;
}

}  // extern "C"
