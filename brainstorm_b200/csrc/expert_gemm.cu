// Grouped expert GEMM on the dispatched layout, for sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
//   out[rows of expert e, :] = act(rows[rows of expert e, :] x weights[e]^T)
//
// rows    [L, K] bf16: the output of dispatch (path e starts at e * max_path_load when padded,
//                      else at sum(loads[0..e)); only the first loads[e] rows of a path count)
// weights [E, N, K] bf16 (every expert's [N, K] matrix, K contiguous)
// out     [L, N] bf16
// loads   [E] int32 ON THE DEVICE: the kernel never needs them on the host.
//
// One persistent CTA per SM walks the list of (expert, 128-row tile, BN-column tile) work
// items that it derives from `loads` itself.  Roles inside a CTA (192 threads):
//   warp 0     one elected lane issues the TMA loads (cp.async.bulk.tensor, 128B swizzle, no
//              multicast) of the A tile [128 x 64] and the B tile [BN x 64] of every k-block
//              into a 4-stage shared-memory ring, completion on mbarriers;
//   warp 1     allocates tensor memory (2 accumulators of 128 lanes x BN fp32 columns), and
//              one elected lane issues tcgen05.mma (M = 128, N = BN, K = 16, bf16 -> fp32)
//              four times per k-block, releasing ring slots and publishing finished
//              accumulators with tcgen05.commit;
//   warps 2-5  epilogue: tcgen05.ld of the accumulator quarter their warp id selects, optional
//              ReLU, fp32 -> bf16, 16-byte stores of the rows that exist (row < loads[e]).
// The second accumulator lets the epilogue of tile i run under the MMAs of tile i + 1.
// Every mbarrier wait is bounded: after the limit the role records an error and leaves its
// loop, the CTA frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace brt_b200 {
namespace {

constexpr int kBM = 128, kBK = 64;  // tile rows; kBK bf16 = one 128-byte swizzle row
// Tile columns BN are 256 when out_features allows it (the A tile is then used by twice as many
// multiply-accumulates, which is what keeps the tensor pipe fed from shared memory), else 128.
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kMaxExperts = 1024;
constexpr uint32_t kTileBytes = kBM * kBK * 2;  // 16 KB: an A tile, or 128 columns of a B tile
constexpr int kSpinLimit = 1 << 22;

struct GemmArgs {
  const int* loads;
  __nv_bfloat16* out;
  int* error;
  int experts;
  int max_path_load;  // 0: packed
  int n_tiles;        // N / BN
  int k_blocks;       // K / kBK
  long long N;
  long long total_rows;
  int relu;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (int spin = 0; spin < kSpinLimit; spin++) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 64) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored with the 128-byte swizzle (rows of
// 128 bytes, groups of 8 rows 1024 bytes apart): start address, leading byte offset 1 (unused
// by swizzled K-major layouts), stride byte offset 1024, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both operands K-major.
template <int BN>
__device__ __forceinline__ uint32_t umma_idesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(kBM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

template <int BN>
struct alignas(1024) GemmSmem {
  unsigned char a[kStages][kTileBytes];
  unsigned char b[kStages][kTileBytes * (BN / 128)];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int first_tile[kMaxExperts + 1];  // exclusive prefix of the tiles per expert
  int row_base[kMaxExperts];
};

struct TileAt {
  int expert, m_tile, n_tile;
};
template <int BN>
__device__ __forceinline__ TileAt tile_at(const GemmSmem<BN>& s, int experts, int n_tiles, int t) {
  int lo = 0, hi = experts - 1;  // last expert whose first tile is <= t (empty ones skipped)
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (s.first_tile[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int local = t - s.first_tile[lo];
  TileAt at;
  at.expert = lo;
  at.m_tile = local / n_tiles;
  at.n_tile = local - at.m_tile * n_tiles;
  return at;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kStageBytes = kTileBytes + kTileBytes * (BN / 128);
  extern __shared__ __align__(1024) unsigned char s_raw[];
  GemmSmem<BN>& s = *reinterpret_cast<GemmSmem<BN>*>(
      (reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // tiles per expert and the first row of every expert (serial scan: E is small)
  if (tid == 0) {
    int tiles = 0, row = 0;
    for (int e = 0; e < g.experts; e++) {
      int load = g.loads[e];
      if (load < 0) load = 0;
      if (g.max_path_load != 0 && load > g.max_path_load) load = g.max_path_load;
      s.first_tile[e] = tiles;
      s.row_base[e] = g.max_path_load != 0 ? e * g.max_path_load : row;
      tiles += (load + kBM - 1) / kBM * g.n_tiles;
      row += load;
    }
    s.first_tile[g.experts] = tiles;
    for (int i = 0; i < kStages; i++) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s.tmem_base;
  const int total_tiles = s.first_tile[g.experts];
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
        const TileAt at = tile_at(s, g.experts, g.n_tiles, t);
        const int row0 = s.row_base[at.expert] + at.m_tile * kBM;
        for (int kb = 0; kb < g.k_blocks; kb++) {
          if (!mbar_wait(&s.empty[slot], phase ^ 1)) { failed = true; break; }
          mbar_expect_tx(&s.full[slot], kStageBytes);
          tma_load_2d(s.a[slot], &map_a, &s.full[slot], kb * kBK, row0);
          tma_load_3d(s.b[slot], &map_b, &s.full[slot], kb * kBK, at.n_tile * BN, at.expert);
          if (++slot == kStages) { slot = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc<BN>();
      int slot = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
        if (!mbar_wait(&s.acc_empty[acc], acc_phase ^ 1)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + (uint32_t)acc * BN;
        for (int kb = 0; kb < g.k_blocks; kb++) {
          if (!mbar_wait(&s.full[slot], phase)) { failed = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = umma_desc(s.a[slot]);
          const uint64_t db = umma_desc(s.b[slot]);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; k++) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(&s.empty[slot]);  // the slot is free once these MMAs have read it
          if (++slot == kStages) { slot = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&s.acc_full[acc]);  // the accumulator is complete once they have finished
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // epilogue: this warp reads the 32 accumulator lanes (tile rows) of quarter warp % 4
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
      const TileAt at = tile_at(s, g.experts, g.n_tiles, t);
      int load = g.loads[at.expert];
      if (g.max_path_load != 0 && load > g.max_path_load) load = g.max_path_load;
      const int row_in_expert = at.m_tile * kBM + quarter * 32 + lane;
      const long long row = (long long)s.row_base[at.expert] + row_in_expert;
      if (!mbar_wait(&s.acc_full[acc], acc_phase)) { failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_load_32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + c0), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row_in_expert < load && row < g.total_rows) {
          uint4* dst = reinterpret_cast<uint4*>(g.out + row * g.N + (long long)at.n_tile * BN + c0);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              float lo = __uint_as_float(v[q * 8 + 2 * i]);
              float hi = __uint_as_float(v[q * 8 + 2 * i + 1]);
              if (g.relu) { lo = fmaxf(lo, 0.f); hi = fmaxf(hi, 0.f); }
              const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
              w[i] = *reinterpret_cast<const uint32_t*>(&p);
            }
            dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }
  if (failed) atomicExch(g.error, BRT_ERR_TIMEOUT);
  __syncwarp();  // the single-lane roles rejoin their warps before the CTA barrier

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(kTmemCols)
                 : "memory");
}

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (no link against libcuda).
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) !=
            cudaSuccess ||
        found != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

extern "C" {

BRT_API int brt_grouped_expert_gemm(const void* rows, const void* weights, void* out,
                                    const int32_t* loads, int path_num, int64_t total_rows,
                                    int32_t max_path_load, int64_t in_features,
                                    int64_t out_features, int relu, void* error_word,
                                    void* stream) {
  clear_error();
  BRT_REQUIRE(path_num > 0 && path_num <= kMaxExperts, "path_num %d outside [1, %d]", path_num,
              kMaxExperts);
  BRT_REQUIRE(total_rows >= 0 && max_path_load >= 0, "negative size");
  BRT_REQUIRE(loads != nullptr && error_word != nullptr, "loads or error_word is null");
  if (in_features <= 0 || out_features <= 0 || in_features % kBK != 0 || out_features % 128 != 0)
    return set_error(BRT_ERR_UNSUPPORTED,
                     "the tensor-core expert GEMM needs in_features %% %d == 0 and "
                     "out_features %% 128 == 0 (got %lld, %lld)",
                     kBK, (long long)in_features, (long long)out_features);
  const int bn = out_features % 256 == 0 ? 256 : 128;
  if (total_rows == 0) return BRT_OK;
  BRT_REQUIRE(rows != nullptr && weights != nullptr && out != nullptr, "null pointer argument");
  BRT_REQUIRE(aligned_to(rows, 16) && aligned_to(weights, 16) && aligned_to(out, 16),
              "rows, weights and out must be 16-byte aligned");
  BRT_REQUIRE(total_rows <= 0x7fffffffLL, "more than 2^31-1 rows");
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr)
    return set_error(BRT_ERR_CUDA, "the driver does not offer cuTensorMapEncodeTiled");

  alignas(64) CUtensorMap map_a, map_b;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)in_features, (cuuint64_t)total_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)in_features * 2};
    const cuuint32_t box[2] = {kBK, kBM};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(rows), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(BRT_ERR_CUDA, "cuTensorMapEncodeTiled(rows) failed with %d", (int)r);
  }
  {
    const cuuint64_t dims[3] = {(cuuint64_t)in_features, (cuuint64_t)out_features,
                                (cuuint64_t)path_num};
    const cuuint64_t strides[2] = {(cuuint64_t)in_features * 2,
                                   (cuuint64_t)in_features * out_features * 2};
    const cuuint32_t box[3] = {kBK, (cuuint32_t)bn, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                              const_cast<void*>(weights), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(BRT_ERR_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
  }
  GemmArgs g;
  g.loads = loads;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.error = static_cast<int*>(error_word);
  g.experts = path_num;
  g.max_path_load = max_path_load;
  g.n_tiles = (int)(out_features / bn);
  g.k_blocks = (int)(in_features / kBK);
  g.N = out_features;
  g.total_rows = total_rows;
  g.relu = relu != 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  BRT_CUDA_TRY(cudaGetDevice(&dev));
  const KernelTimer timer("expert_gemm_kernel", st);
  if (bn == 256) {
    const size_t smem = sizeof(GemmSmem<256>) + 1024;
    static thread_local int configured_device = -1;
    if (configured_device != dev) {
      BRT_CUDA_TRY(cudaFuncSetAttribute(expert_gemm_kernel<256>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured_device = dev;
    }
    expert_gemm_kernel<256><<<(unsigned)sm_count(), kThreads, smem, st>>>(map_a, map_b, g),
        note_launch();
  } else {
    const size_t smem = sizeof(GemmSmem<128>) + 1024;
    static thread_local int configured_device = -1;
    if (configured_device != dev) {
      BRT_CUDA_TRY(cudaFuncSetAttribute(expert_gemm_kernel<128>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured_device = dev;
    }
    expert_gemm_kernel<128><<<(unsigned)sm_count(), kThreads, smem, st>>>(map_a, map_b, g),
        note_launch();
  }
  BRT_LAUNCH_CHECK("expert_gemm_kernel");
  return BRT_OK;
}

}  // extern "C"
