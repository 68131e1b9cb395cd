// Expert-parallel exchange over NCCL point-to-point: one communicator owned by the library
// (bootstrapped from a unique id that the caller moves between ranks), and the grouped
// send/recv patterns of the routing path.  All sizes are 64-bit byte counts; per-bucket row
// counts come from host arrays exactly as in the interfaces these functions replace.
#include <nccl.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace brt_b200 {
namespace {

struct Comm {
  std::mutex mu;
  ncclComm_t comm = nullptr;
  int rank = -1;
  int size = 0;
  int device = -1;
};

Comm& comm_state() {
  static Comm c;
  return c;
}

#define BRT_NCCL_TRY(expr)                                                                    \
  do {                                                                                        \
    ncclResult_t _r = (expr);                                                                 \
    if (_r != ncclSuccess)                                                                    \
      return ::brt_b200::set_error(BRT_ERR_NCCL, "%s failed: %s (%s:%d)", #expr,              \
                                   ncclGetErrorString(_r), __FILE__, __LINE__);               \
  } while (0)

#define BRT_NEED_COMM(c)                                                                      \
  do {                                                                                        \
    if ((c).comm == nullptr)                                                                  \
      return ::brt_b200::set_error(BRT_ERR_NOT_INITIALIZED,                                   \
                                   "brt_nccl_init has not been called in this process");      \
  } while (0)

inline const char* at(const void* p, int64_t bytes) { return static_cast<const char*>(p) + bytes; }
inline char* at(void* p, int64_t bytes) { return static_cast<char*>(p) + bytes; }

}  // namespace
}  // namespace brt_b200

using namespace brt_b200;

extern "C" {

static_assert(sizeof(ncclUniqueId) == BRT_NCCL_UNIQUE_ID_BYTES, "unique id size");

BRT_API int brt_nccl_get_unique_id(void* out_id) {
  clear_error();
  BRT_REQUIRE(out_id != nullptr, "out_id is null");
  ncclUniqueId id;
  BRT_NCCL_TRY(ncclGetUniqueId(&id));
  memcpy(out_id, &id, sizeof(id));
  return BRT_OK;
}

BRT_API int brt_nccl_init(const void* unique_id, int world_rank, int world_size) {
  clear_error();
  BRT_REQUIRE(unique_id != nullptr, "unique_id is null");
  BRT_REQUIRE(world_size >= 1 && world_rank >= 0 && world_rank < world_size,
              "bad rank %d of %d", world_rank, world_size);
  Comm& c = comm_state();
  std::lock_guard<std::mutex> lock(c.mu);
  if (c.comm != nullptr) {
    // same outcome as the reference: a second init is refused, the first communicator stays
    return set_error(BRT_ERR_INVALID_ARGUMENT, "NCCL communicator already initialised (rank %d of %d)",
                     c.rank, c.size);
  }
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  BRT_CUDA_TRY(cudaGetDevice(&c.device));
  ncclComm_t comm = nullptr;
  BRT_NCCL_TRY(ncclCommInitRank(&comm, world_size, id, world_rank));
  c.comm = comm;
  c.rank = world_rank;
  c.size = world_size;
  return BRT_OK;
}

BRT_API int brt_nccl_is_initialized(void) { return comm_state().comm != nullptr ? 1 : 0; }

BRT_API int brt_nccl_world(int* world_rank, int* world_size) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  if (world_rank) *world_rank = c.rank;
  if (world_size) *world_size = c.size;
  return BRT_OK;
}

BRT_API int brt_nccl_destroy(void) {
  clear_error();
  Comm& c = comm_state();
  std::lock_guard<std::mutex> lock(c.mu);
  if (c.comm != nullptr) {
    ncclResult_t r = ncclCommDestroy(c.comm);
    c.comm = nullptr;
    c.rank = -1;
    c.size = 0;
    if (r != ncclSuccess) return set_error(BRT_ERR_NCCL, "ncclCommDestroy: %s", ncclGetErrorString(r));
  }
  return BRT_OK;
}

BRT_API int brt_broadcast(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                          void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(bytes >= 0 && root >= 0 && root < c.size, "bad broadcast arguments");
  BRT_NCCL_TRY(ncclBroadcast(send_buffer, recv_buffer, (size_t)bytes, ncclChar, root, c.comm,
                             static_cast<cudaStream_t>(stream)));
  return BRT_OK;
}

BRT_API int brt_exchange(const void* send_buffer, void* recv_buffer, int64_t bytes, int dest,
                         int source, void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(bytes >= 0 && dest >= 0 && dest < c.size && source >= 0 && source < c.size,
              "bad exchange arguments (dest %d, source %d, world %d)", dest, source, c.size);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BRT_NCCL_TRY(ncclGroupStart());
  ncclResult_t r1 = ncclSend(send_buffer, (size_t)bytes, ncclChar, dest, c.comm, st);
  ncclResult_t r2 = ncclRecv(recv_buffer, (size_t)bytes, ncclChar, source, c.comm, st);
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(r1);
  BRT_NCCL_TRY(r2);
  return BRT_OK;
}

BRT_API int brt_scatter(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                        void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(bytes >= 0 && root >= 0 && root < c.size, "bad scatter arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ncclResult_t bad = ncclSuccess;
  BRT_NCCL_TRY(ncclGroupStart());
  if (c.rank == root)
    for (int i = 0; i < c.size; i++) {
      ncclResult_t r = ncclSend(at(send_buffer, (int64_t)i * bytes), (size_t)bytes, ncclChar, i, c.comm, st);
      if (r != ncclSuccess) bad = r;
    }
  ncclResult_t r = ncclRecv(recv_buffer, (size_t)bytes, ncclChar, root, c.comm, st);
  if (r != ncclSuccess) bad = r;
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(bad);
  return BRT_OK;
}

BRT_API int brt_gather(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                       void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(bytes >= 0 && root >= 0 && root < c.size, "bad gather arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ncclResult_t bad = ncclSuccess;
  BRT_NCCL_TRY(ncclGroupStart());
  if (c.rank == root)
    for (int i = 0; i < c.size; i++) {
      ncclResult_t r = ncclRecv(at(recv_buffer, (int64_t)i * bytes), (size_t)bytes, ncclChar, i, c.comm, st);
      if (r != ncclSuccess) bad = r;
    }
  ncclResult_t r = ncclSend(send_buffer, (size_t)bytes, ncclChar, root, c.comm, st);
  if (r != ncclSuccess) bad = r;
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(bad);
  return BRT_OK;
}

BRT_API int brt_all_to_all(const void* send_buffer, void* recv_buffer, int64_t slice_bytes,
                           void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(slice_bytes >= 0, "negative slice size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ncclResult_t bad = ncclSuccess;
  BRT_NCCL_TRY(ncclGroupStart());
  for (int i = 0; i < c.size; i++) {
    ncclResult_t r = ncclSend(at(send_buffer, i * slice_bytes), (size_t)slice_bytes, ncclChar, i, c.comm, st);
    if (r != ncclSuccess) bad = r;
    r = ncclRecv(at(recv_buffer, i * slice_bytes), (size_t)slice_bytes, ncclChar, i, c.comm, st);
    if (r != ncclSuccess) bad = r;
  }
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(bad);
  return BRT_OK;
}

BRT_API int brt_group_asymmetry_all_to_all(const void* send_buffer, void* recv_buffer,
                                           const int32_t* send_sizes, const int32_t* recv_sizes,
                                           int64_t grain_bytes, int64_t slot_bytes, int group_size,
                                           void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(send_sizes != nullptr && recv_sizes != nullptr, "size arrays are null");
  BRT_REQUIRE(grain_bytes >= 0 && slot_bytes >= 0 && group_size >= 1, "bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int k = 0; k < c.size * group_size; k++)
    BRT_REQUIRE(send_sizes[k] >= 0 && recv_sizes[k] >= 0 &&
                    (int64_t)send_sizes[k] * grain_bytes <= slot_bytes &&
                    (int64_t)recv_sizes[k] * grain_bytes <= slot_bytes,
                "bucket %d does not fit its slot", k);
  ncclResult_t bad = ncclSuccess;
  BRT_NCCL_TRY(ncclGroupStart());
  for (int i = 0; i < c.size; i++)
    for (int j = 0; j < group_size; j++) {
      const int k = i * group_size + j;
      ncclResult_t r = ncclSend(at(send_buffer, k * slot_bytes), (size_t)send_sizes[k] * grain_bytes, ncclChar, i, c.comm, st);
      if (r != ncclSuccess) bad = r;
      r = ncclRecv(at(recv_buffer, k * slot_bytes), (size_t)recv_sizes[k] * grain_bytes, ncclChar, i, c.comm, st);
      if (r != ncclSuccess) bad = r;
    }
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(bad);
  return BRT_OK;
}

// forward != 0: sends walk buckets [rank i][expert j], receives walk [expert j][rank i];
// forward == 0: the inverse walk.  stride_rows != 0 places every bucket stride_rows apart
// (max_path_padding) instead of back to back.
BRT_API int brt_group_sparse_all_to_all(const void* send_buffer, void* recv_buffer,
                                        const int32_t* send_sizes, const int32_t* recv_sizes,
                                        int64_t grain_bytes, int64_t stride_rows, int group_size,
                                        int forward, void* stream) {
  clear_error();
  Comm& c = comm_state();
  BRT_NEED_COMM(c);
  BRT_REQUIRE(send_sizes != nullptr && recv_sizes != nullptr, "size arrays are null");
  BRT_REQUIRE(grain_bytes >= 0 && stride_rows >= 0 && group_size >= 1, "bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int W = c.size, G = group_size;
  for (int k = 0; k < W * G; k++)
    BRT_REQUIRE(send_sizes[k] >= 0 && recv_sizes[k] >= 0 &&
                    (stride_rows == 0 || (send_sizes[k] <= stride_rows && recv_sizes[k] <= stride_rows)),
                "bucket %d has a bad size", k);
  ncclResult_t bad = ncclSuccess;
  BRT_NCCL_TRY(ncclGroupStart());
  int64_t cursor = 0;
  // rank-major side
  auto rank_major = [&](bool sending, const void* sbuf, void* rbuf, const int32_t* sizes) {
    cursor = 0;
    for (int i = 0; i < W; i++)
      for (int j = 0; j < G; j++) {
        const int64_t rows = sizes[i * G + j];
        ncclResult_t r = sending
            ? ncclSend(at(sbuf, cursor * grain_bytes), (size_t)(rows * grain_bytes), ncclChar, i, c.comm, st)
            : ncclRecv(at(rbuf, cursor * grain_bytes), (size_t)(rows * grain_bytes), ncclChar, i, c.comm, st);
        if (r != ncclSuccess) bad = r;
        cursor += stride_rows != 0 ? stride_rows : rows;
      }
  };
  // expert-major side
  auto expert_major = [&](bool sending, const void* sbuf, void* rbuf, const int32_t* sizes) {
    cursor = 0;
    for (int j = 0; j < G; j++)
      for (int i = 0; i < W; i++) {
        const int64_t rows = sizes[j * W + i];
        ncclResult_t r = sending
            ? ncclSend(at(sbuf, cursor * grain_bytes), (size_t)(rows * grain_bytes), ncclChar, i, c.comm, st)
            : ncclRecv(at(rbuf, cursor * grain_bytes), (size_t)(rows * grain_bytes), ncclChar, i, c.comm, st);
        if (r != ncclSuccess) bad = r;
        cursor += stride_rows != 0 ? stride_rows : rows;
      }
  };
  if (forward) {
    rank_major(true, send_buffer, nullptr, send_sizes);
    expert_major(false, nullptr, recv_buffer, recv_sizes);
  } else {
    expert_major(true, send_buffer, nullptr, send_sizes);
    rank_major(false, nullptr, recv_buffer, recv_sizes);
  }
  BRT_NCCL_TRY(ncclGroupEnd());
  BRT_NCCL_TRY(bad);
  return BRT_OK;
}

}  // extern "C"
