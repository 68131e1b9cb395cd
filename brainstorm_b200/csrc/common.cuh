// Shared helpers for the brt_b200 kernels: error reporting across the C ABI, launch
// checks, vector types for 128-bit row moves and dtype conversion.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/brt_b200.h"

namespace brt_b200 {

// Per-thread message buffer behind brt_last_error().
char* error_buffer();
int set_error(int code, const char* fmt, ...);
void clear_error();

// Counts a kernel launch made by this library (process-wide; read by
// brt_kernel_launch_count()).
void note_launch();

// Optional per-kernel timing (off by default; brt_profile_enable).  While it is on, a
// KernelTimer records a CUDA event on the launching stream before and after the launches it
// brackets; brt_profile_report sums the elapsed times per name.  Never enable it while a
// stream is being captured into a graph.
struct KernelTimer {
  KernelTimer(const char* name, cudaStream_t stream);
  ~KernelTimer();
  cudaStream_t stream_;
  void* slot_;
};

// Number of SMs of the current device (cached per device).
int sm_count();

#define BRT_CUDA_TRY(expr)                                                                    \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::brt_b200::set_error(BRT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,              \
                                   cudaGetErrorString(_e), __FILE__, __LINE__);               \
  } while (0)

#define BRT_LAUNCH_CHECK(name)                                                                \
  do {                                                                                        \
    cudaError_t _e = cudaGetLastError();                                                      \
    if (_e != cudaSuccess)                                                                    \
      return ::brt_b200::set_error(BRT_ERR_CUDA, "launch of %s failed: %s", name,             \
                                   cudaGetErrorString(_e));                                   \
  } while (0)

#define BRT_REQUIRE(cond, ...)                                                                \
  do {                                                                                        \
    if (!(cond)) return ::brt_b200::set_error(BRT_ERR_INVALID_ARGUMENT, __VA_ARGS__);         \
  } while (0)

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline int dtype_size(int dtype) { return dtype == BRT_F32 ? 4 : 2; }

// ---- asynchronous 16-byte copies from global to shared memory (bypassing L1) ----------------
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem_src) : "memory");
}
// The same copy with an L2 eviction policy (createpolicy) attached to the line it reads.
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void cp_async_16_hint(void* smem_dst, const void* gmem_src,
                                                 unsigned long long policy) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(s),
               "l"(gmem_src), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
// Waits until at most N of this thread's committed groups are still in flight.
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- device-side conversion between storage types and fp32 ---------------------------------

template <int DT>
struct Elem;
template <>
struct Elem<BRT_F32> {
  using type = float;
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <>
struct Elem<BRT_F16> {
  using type = __half;
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<BRT_BF16> {
  using type = __nv_bfloat16;
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) {
    return __float2bfloat16_rn(v);
  }
};

// A VB-byte chunk of a row, moved with one load/store instruction.
template <int VB>
struct Chunk;
template <>
struct Chunk<16> {
  using type = uint4;
};
template <>
struct Chunk<8> {
  using type = uint2;
};
template <>
struct Chunk<4> {
  using type = uint32_t;
};
template <>
struct Chunk<2> {
  using type = uint16_t;
};

template <typename T>
__device__ __forceinline__ T zero_chunk() {
  T z;
  unsigned char* p = reinterpret_cast<unsigned char*>(&z);
#pragma unroll
  for (int i = 0; i < (int)sizeof(T); i++) p[i] = 0;
  return z;
}

// Streaming (evict-first) global accesses for data that is touched once.
template <typename T>
__device__ __forceinline__ T load_stream(const T* p) {
  return __ldcs(p);
}
template <typename T>
__device__ __forceinline__ void store_stream(T* p, const T& v) {
  __stcs(p, v);
}
template <>
__device__ __forceinline__ uint16_t load_stream<uint16_t>(const uint16_t* p) {
  return *p;
}
template <>
__device__ __forceinline__ void store_stream<uint16_t>(uint16_t* p, const uint16_t& v) {
  *p = v;
}

}  // namespace brt_b200
