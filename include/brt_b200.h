/*
 * brt_b200 — C ABI of the B200-native routing hot path.
 *
 * One shared library (libbrt_b200.so) exports these entry points.  They take raw
 * device pointers, sizes and a CUDA stream; they never allocate device memory,
 * never synchronise the host with the device and never touch a tensor library.
 * Every function returns 0 on success or a brt_status code; the text of the last
 * error on the calling thread is available from brt_last_error().
 *
 * Each entry point names the interface of the reference project
 * (Raphael-Hao/brainstorm) that it stands in for, as path:line in that project.
 *
 * Conventions
 *   - all index, load, tag and mask arrays are int32, row-major, device memory;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - `dtype` is a brt_dtype; cell_size counts elements of that type per cell;
 *   - scratch buffers are caller-owned device memory, at least as large as the
 *     matching *_scratch_bytes() query says and 256-byte aligned; their contents
 *     on entry are irrelevant and they may be reused by the next call on the
 *     same stream.
 */
#ifndef BRT_B200_H_
#define BRT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define BRT_API __attribute__((visibility("default")))
#else
#define BRT_API
#endif

typedef enum brt_status {
  BRT_OK = 0,
  BRT_ERR_INVALID_ARGUMENT = 1, /* bad size, null pointer, unsupported flag combination */
  BRT_ERR_CUDA = 2,             /* a CUDA runtime call or launch failed */
  BRT_ERR_SCRATCH_TOO_SMALL = 3,
  BRT_ERR_UNSUPPORTED = 4,
  BRT_ERR_NCCL = 5,
  BRT_ERR_NOT_INITIALIZED = 6,
  BRT_ERR_TIMEOUT = 7 /* a bounded device-side wait ran out */
} brt_status;

typedef enum brt_dtype { BRT_F32 = 0, BRT_F16 = 1, BRT_BF16 = 2 } brt_dtype;

/* ABI revision; bumped on any signature change. */
BRT_API int brt_abi_version(void);
/* Message of the last failing call made by this thread ("" if none). */
BRT_API const char* brt_last_error(void);
/* Kernels this library has launched in the process so far (all threads, all devices).
 * Instrumentation for benchmarks; the reference has no counterpart. */
BRT_API uint64_t brt_kernel_launch_count(void);
/* Per-kernel device times for benchmarks (no counterpart in the reference).  While enabled,
 * the library records a CUDA event on the launching stream before and after each of its hot
 * kernels; brt_profile_report waits for the recorded launches, writes
 * {"kernel": {"launches": n, "total_ms": t}, ...} as JSON text into `out` and forgets them.
 * Leave it off (the default) while a stream is being captured into a CUDA graph. */
BRT_API void brt_profile_enable(int on);
BRT_API int brt_profile_report(char* out, size_t out_bytes);

/* ------------------------------------------------------------------ router: indices */

/* Scratch needed by brt_generate_indices_and_loads / brt_throttle_hotmask. */
BRT_API size_t brt_index_scratch_bytes(int64_t cell_num, int path_num);

/*
 * Replaces brt::router::GenerateIndicesAndLoads
 * (include/brt/router/location.h:29-39, src/router/location.cu:335-379).
 *
 * hot_mask[cell_num, path_num] -> indices[cell_num, path_num], loads[path_num].
 * Seat mode: indices[t,e] = mask[t,e] * (sum of mask[0..t, e]).  Tag mode:
 * indices[r-1, e] = t+1 for the r-th routed cell of path e, 0 elsewhere.
 * loads follow the reference's capacity rules (path_wise_padding only with
 * capacity_padding; capacity_padding needs supported_capacity_num >= 1).
 * `indices` is fully written (it does not have to be zeroed by the caller).
 * path_counts (optional, [path_num]) receives the cells per path that the indices hold, i.e.
 * the column sums of the mask before the capacity rules turn them into loads: what
 * brt_dispatch_with_indices_and_loads takes as `dense_counts`.
 */
BRT_API int brt_generate_indices_and_loads(const int32_t* hot_mask, int32_t* indices,
                                           int32_t* loads, int32_t* path_counts,
                                           int64_t cell_num, int path_num,
                                           const int32_t* supported_capacities,
                                           int supported_capacity_num, int capacity_padding,
                                           int path_wise_padding, int is_tag_index,
                                           void* scratch, size_t scratch_bytes, void* stream);

/*
 * No counterpart in the reference.
 *
 * Same result as brt_generate_indices_and_loads, for callers that are not allowed to
 * obtain device memory themselves and therefore cannot supply the scratch buffer: code
 * running under a memory planner that owns the whole device heap, or a plugin host that
 * hands out only the input and output tensors.  The scratch lives in a fixed array inside the
 * library image (brt_static_index_scratch_bytes() bytes, 2 MiB, held on every GPU that
 * loads the library until the process exits), so this call performs no device allocation
 * of any kind.
 *
 * Limits and rules:
 *   - masks whose scratch need exceeds the built-in array are refused with
 *     BRT_ERR_SCRATCH_TOO_SMALL and a message that states both sizes (roughly
 *     cell_num * path_num up to 7 million entries); nothing is launched in that case;
 *   - the first call on each device looks up the device address of the array (once, with
 *     that device current); make that first call before starting any stream capture;
 *   - all calls on a device share the one array: two calls whose kernels can overlap on
 *     the GPU (different streams without an ordering between them) race; calls ordered on
 *     one stream are safe, and nothing has to be cleared between them.
 */
BRT_API size_t brt_static_index_scratch_bytes(void);
BRT_API int brt_generate_indices_and_loads_static(const int32_t* hot_mask, int32_t* indices,
                                                  int32_t* loads, int64_t cell_num,
                                                  int path_num,
                                                  const int32_t* supported_capacities,
                                                  int supported_capacity_num,
                                                  int capacity_padding, int path_wise_padding,
                                                  int is_tag_index, void* stream);

/*
 * Bounded waits of the index kernels.  The single-launch scan lets a CTA wait for the column
 * sums of CTAs that started before it; the wait gives up after a fixed number of polls, the
 * kernel finishes with what it has (its outputs are then wrong) and records BRT_ERR_TIMEOUT
 * in a word of host-mapped memory.  No counterpart in the reference (its kernels have no
 * inter-CTA waits).
 *
 * brt_index_status        BRT_OK, or BRT_ERR_TIMEOUT once a scan of this process has given up;
 *                         read from host memory, no synchronisation.  Results of scans that
 *                         completed before the call are covered (synchronise first to cover
 *                         one that is still running).  The first call creates the word
 *                         (a set-up time allocation); brt_generate_indices_and_loads_static
 *                         reports through it only once it exists.
 * brt_index_status_reset  clears the word.
 * brt_index_set_test_hooks  for tests of the above: `spin_limit` polls per wait (<= 0: the
 *                         default) and, when `skip_first_run` != 0, a first run of tiles that
 *                         no CTA owns, so that the waits for its sums run out.
 */
BRT_API int brt_index_status(void);
BRT_API void brt_index_status_reset(void);
BRT_API void brt_index_set_test_hooks(int spin_limit, int skip_first_run);

/*
 * Replaces brt::router::ThrottleHotmask
 * (include/brt/router/location.h:13-19, src/router/location.cu:59-130,304-315).
 *
 * throttled[t,e] = (hotmask[t,e] == 1 && prefix[e] + sum(hotmask[0..t, e]) <= threshold[e]);
 * prefix[e] <- min(prefix[e] + sum(hotmask[:, e]), threshold[e]) in place (untouched when
 * cell_num == 0).  `throttled` is fully written.
 */
BRT_API int brt_throttle_hotmask(const int32_t* hotmask, int32_t* throttled, int32_t* prefix,
                                 const int32_t* threshold, int64_t cell_num, int path_num,
                                 void* scratch, size_t scratch_bytes, void* stream);

/*
 * brt_throttle_hotmask followed by brt_generate_indices_and_loads (seat indices) of the
 * throttled mask, in one pass over the mask and without the throttled mask ever reaching
 * memory: what python/brt/router/protocol/swin_moe.py:112-140 and
 * python/brt/router/fabric/generic.py:83-89 do in two operator calls
 * (src/router/location.cu:304-315 then :335-379).  The seat of a kept cell is its seat in the
 * unthrottled mask, and a cell is kept while prefix[e] + seat <= threshold[e], so one scan
 * yields both.
 *
 * indices[t,e] = seat if hot_mask[t,e] != 0 and prefix_in[e] + seat <= threshold[e], else 0;
 * loads[e] = the capacity rules of brt_generate_indices_and_loads applied to the number of
 * kept cells; prefix[e] <- min(prefix[e] + sum(hot_mask[:, e]), threshold[e]) in place.
 * throttled_mask (optional, [cell_num, path_num]) receives the throttled 0/1 mask as well.
 *
 * hot_mask must hold only 0 and 1 (what the protocols produce).  Another value makes the
 * kernel write zero indices and report BRT_ERR_INVALID_ARGUMENT through brt_index_status.
 * Returns BRT_ERR_UNSUPPORTED (nothing launched) when path_num is not a multiple of 4, an
 * array is not 16-byte aligned or the mask is too large for the single-launch scan; the
 * caller then uses the two entry points above.
 */
BRT_API int brt_throttle_and_generate_indices(
    const int32_t* hot_mask, int32_t* indices, int32_t* loads, int32_t* path_counts,
    int32_t* prefix, const int32_t* threshold, int32_t* throttled_mask, int64_t cell_num,
    int path_num,
    const int32_t* supported_capacities, int supported_capacity_num, int capacity_padding,
    int path_wise_padding, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Replaces brt::router::ConvertIndexFormat
 * (include/brt/router/location.h:21-27, src/router/location.cu:259-333).
 * tag_to_seat != 0: new[tag-1, e] = r+1 for rows r < loads[e] with a non-zero tag;
 * tag_to_seat == 0: new[seat-1, e] = t+1 for non-zero seats.  `new_indices` is
 * fully written.  Entries that would land outside [0, cell_num) are ignored.
 */
BRT_API int brt_convert_index_format(const int32_t* origin_indices, int32_t* new_indices,
                                     const int32_t* loads, int64_t cell_num, int path_num,
                                     int tag_to_seat, void* stream);

/* ------------------------------------------------------------------ router: fused gate */

typedef enum brt_gate_decision { BRT_GATE_TOPK = 0, BRT_GATE_THRESHOLD = 1 } brt_gate_decision;
typedef enum brt_route_output {
  BRT_ROUTE_MASK = 0,           /* out = hot mask, loads = cells routed to every path */
  BRT_ROUTE_THROTTLED_MASK = 1, /* out = hot mask cut at throttle_capacity, prefix updated */
  BRT_ROUTE_SEAT_INDICES = 2,   /* out = seat indices, loads as brt_generate_indices_and_loads */
  BRT_ROUTE_THROTTLED_SEAT_INDICES = 3 /* both: seat indices and loads of the hot mask cut at
                                          throttle_capacity, prefix updated
                                          (brt_throttle_and_generate_indices from scores) */
} brt_route_output;

/*
 * Route decision and index scan in one launch, straight from the gate's scores: what the
 * reference does with a protocol (torch.topk + scatter_, python/brt/router/protocol/topk.py:
 * 26-31; score > threshold with a residual path, protocol/threshold.py:23-39; the first pick
 * cut at the runtime capacity, protocol/swin_moe.py:69-80 with ThrottleHotmask,
 * src/router/location.cu:304-315) followed by GenerateIndicesAndLoads
 * (include/brt/router/location.h:29-39), without the hot mask ever reaching memory unless it
 * is the requested output.
 *
 *   scores   fp32 [cell_num, path_num], row-major
 *   decision BRT_GATE_TOPK: ones at the top_k largest scores of a cell (equal scores: the
 *            lower path wins; the reference leaves ties to torch.topk);
 *            BRT_GATE_THRESHOLD: ones where score > threshold, and residual_path (>= 0) for
 *            a cell that would otherwise go nowhere
 *   output   see brt_route_output; capacities / capacity_padding / path_wise_padding as in
 *            brt_generate_indices_and_loads (the two SEAT_INDICES outputs); prefix and
 *            throttle_capacity as in brt_throttle_hotmask (the two THROTTLED outputs)
 *   gates_out optional fp32 [cell_num, path_num]: picked scores divided by their sum
 *            (clamped at FLT_EPSILON), zero elsewhere (protocol/swin_moe.py:193-204)
 *   mask_out optional int32 [cell_num, path_num], the two SEAT_INDICES outputs only: the
 *            (throttled) hot mask beside its seat indices
 *   scratch  brt_index_scratch_bytes(cell_num, path_num) bytes
 *
 * Returns BRT_ERR_UNSUPPORTED (nothing launched) when path_num is not a multiple of 4 or
 * exceeds 256, an array is not 16-byte aligned, or the scores are too many for the
 * single-launch kernel; the caller then routes in two steps.
 */
BRT_API int brt_route_scores(const float* scores, int64_t cell_num, int path_num, int decision,
                             int top_k, float threshold, int residual_path, int output,
                             int32_t* out, int32_t* loads, int32_t* path_counts,
                             const int32_t* capacities,
                             int capacity_num, int capacity_padding, int path_wise_padding,
                             int32_t* prefix, const int32_t* throttle_capacity, float* gates_out,
                             int32_t* mask_out, void* scratch, size_t scratch_bytes,
                             void* stream);

/* ------------------------------------------------------------------ router: data movement */

/* Scratch needed by brt_dispatch_with_indices_and_loads for `total_rows` output rows. */
BRT_API size_t brt_dispatch_scratch_bytes(int64_t total_rows, int path_num);

/*
 * Replaces brt::router::DispatchWithIndicesAndLoads<T>
 * (include/brt/router/route.h:14-28, src/router/route.cu:13-206,284-465).
 *
 * 1-D routing: src[cell_num, cell_size]; 2-D routing: src[cell_num, path_num, cell_size]
 * (path e takes element e of each cell; no gates).  dst has `total_rows` rows:
 * path e starts at row e*max_path_load when max_path_load != 0, otherwise at
 * sum(loads[0..e)).  A cell goes to row base(e)+seat-1 when 0 < seat <= loads[e].
 * Rows of dst (and of new_tags) that no kept cell lands on are written as zero by
 * this call: the caller does not pre-zero anything.  gates (optional, 1-D only) has
 * the data's dtype and scales the copied row; old_tags/new_tags (optional, both or
 * neither) carry the cell tags.  is_tag_index != 0 reads route_indices as tag indices
 * (row i < loads[e] of path e pulls cell tag-1; a zero tag leaves the row zero).
 *
 * dense_counts (optional, seat indices only): the caller vouches that column e of
 * route_indices holds every seat 1 .. dense_counts[e] exactly once and zeros elsewhere, which
 * is what the index entry points write and report as `path_counts`.  The rows that stay empty
 * are then known without looking at the indices and the whole dispatch is ONE launch that
 * needs no scratch; without it (any index tensor) the call marks the rows it writes in
 * `scratch` (brt_dispatch_scratch_bytes) and zeroes the others with a second launch.
 */
BRT_API int brt_dispatch_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, const int32_t* old_tags, int32_t* new_tags, int64_t cell_num,
    int64_t cell_size, int path_num, int32_t max_path_load, int64_t total_rows,
    int is_1d_routing, int is_tag_index, int dtype, const int32_t* dense_counts, void* scratch,
    size_t scratch_bytes, void* stream);

/*
 * Replaces brt::router::CombineWithIndicesAndLoads<T>
 * (include/brt/router/route.h:30-44, src/router/route.cu:208-282,467-522).
 *
 * dst[t, :] = sum over paths e in ascending order with 0 < seat <= loads[e] of
 * src[base(e)+seat-1, :] (* gates[t,e]); every product and every add is rounded to
 * fp32 separately, the sum starts from +0.  is_residual == 0: every row of dst is
 * written (zero when the cell has no kept route).  is_residual != 0: only rows
 * with at least one kept route are replaced, the others keep the caller's data.
 * dtype is the element type of src/dst (16-bit types accumulate in fp32 and round
 * once on store); gates_dtype is BRT_F32 or equal to dtype.
 */
BRT_API int brt_combine_with_indices_and_loads(
    const void* src_data, void* dst_data, const void* gates, const int32_t* route_indices,
    const int32_t* loads, int64_t cell_num, int64_t cell_size, int path_num,
    int32_t max_path_load, int is_residual, int dtype, int gates_dtype, void* stream);

/*
 * Sum of rows by destination index: out_rows[o] = sum of in_rows[r] over the rows r with
 * row_index[r] == o, added in ascending r in fp32 (16-bit types are rounded once); rows of
 * `out_rows` that nobody points at come back as zeros.  This is the tag-index branch of
 * combine_with_indices_and_loads, which the reference's binding computes with torch
 * (scatter_reduce("sum") over the inverse indices of unique(tags),
 * src/backend/torch/router.cc:449-459) because its launcher has no tag-index combine
 * (src/router/route.cu:519-521).  Entries of row_index outside [0, rows_out) are ignored.
 * scratch: brt_sum_rows_scratch_bytes(rows_in, rows_out) bytes, 256-byte aligned.
 */
BRT_API size_t brt_sum_rows_scratch_bytes(int64_t rows_in, int64_t rows_out);
BRT_API int brt_sum_rows_by_index(const void* in_rows, const int32_t* row_index, void* out_rows,
                                  int64_t rows_in, int64_t rows_out, int64_t cell_size,
                                  int dtype, void* scratch, size_t scratch_bytes, void* stream);

/* ------------------------------------------------------------------ experts: grouped GEMM */

/*
 * The expert side of the dispatched layout: one linear layer per expert over the rows that
 * dispatch wrote for it, on the 5th-generation tensor cores (tcgen05.mma with accumulators in
 * tensor memory, operands staged by TMA).  Stands where the reference launches its
 * horizontally fused "homo" expert kernel on the dispatched buffer with the per-expert loads
 * (src/backend/torch/jit.cc:54-75, benchmark/switch_moe/switch_expert.py:62-99).
 *
 *   out[r, :] = act(rows[r, :] x weights[e]^T)   for the first loads[e] rows r of expert e
 *
 * rows [total_rows, in_features] bf16 as dispatch leaves them (expert e starts at row
 * e * max_path_load when max_path_load != 0, else at sum(loads[0..e)); weights
 * [path_num, out_features, in_features] bf16; out [total_rows, out_features] bf16; loads
 * [path_num] int32 ON THE DEVICE (nothing is read back to the host; with max_path_load != 0
 * loads above it are cut).  Rows of `out` beyond an expert's load are not written.
 * relu != 0 applies max(x, 0) before the rounding to bf16.
 * error_word: a zero-initialised 4-byte device word; a bounded wait inside the kernel that
 * runs out stores BRT_ERR_TIMEOUT there (the kernel then returns with `out` incomplete).
 * Returns BRT_ERR_UNSUPPORTED (nothing launched) unless in_features % 64 == 0 and
 * out_features % 128 == 0.
 */
BRT_API int brt_grouped_expert_gemm(const void* rows, const void* weights, void* out,
                                    const int32_t* loads, int path_num, int64_t total_rows,
                                    int32_t max_path_load, int64_t in_features,
                                    int64_t out_features, int relu, void* error_word,
                                    void* stream);

/* ------------------------------------------------------------------ distributed: rank reorder */

/*
 * Replaces brt::distributed::LocalityReorder
 * (include/brt/distributed/local_reorder.h:11-12, src/distributed/local_reorder.cu:15-63,143-149).
 * loads[c * world_size + o] = rows rank c received from rank o.  world_size rounds of
 * arg-max over the entries whose row and column are still free (ties: smallest flat index);
 * reorder_indices[c] = o; reordered_loads[r, c] = loads[r, reorder_indices[c]].
 * world_size <= 32.  All arrays are device memory; reordered_loads must not alias loads.
 */
BRT_API int brt_locality_reorder(const int32_t* loads, int world_size, int32_t* reorder_indices,
                                 int32_t* reordered_loads, void* stream);

/*
 * Replaces brt::distributed::GroupLocalityReorder
 * (include/brt/distributed/local_reorder.h:13-14, src/distributed/local_reorder.cu:65-141,151-159).
 * loads[(c * world_size + o) * group_size + g]; the matching runs on the sums over g (any
 * group_size; the reference's tree sum is only exact for powers of two and needs
 * group_size * world_size^2 <= 1024), and the o axis of the output is permuted:
 * reordered_loads[r, c, :] = loads[r, reorder_indices[c], :].
 */
BRT_API int brt_group_locality_reorder(const int32_t* loads, int group_size, int world_size,
                                       int32_t* reorder_indices, int32_t* reordered_loads,
                                       void* stream);

/* ------------------------------------------------------------------ distributed: NCCL exchange */

#define BRT_NCCL_UNIQUE_ID_BYTES 128

/*
 * Communicator bootstrap; replaces make_nccl_unique_id / init_nccl and NcclManager::Init
 * (src/backend/torch/distributed.cc:16-41, src/backend/torch/nccl_manager.cc:19-30).
 * Rank 0 fills a 128-byte id, the caller moves it to every rank, every rank calls
 * brt_nccl_init with the current CUDA device set.  A second brt_nccl_init is refused
 * (BRT_ERR_INVALID_ARGUMENT) and leaves the first communicator in place.
 */
BRT_API int brt_nccl_get_unique_id(void* out_id /* BRT_NCCL_UNIQUE_ID_BYTES, host */);
BRT_API int brt_nccl_init(const void* unique_id, int world_rank, int world_size);
BRT_API int brt_nccl_is_initialized(void);
BRT_API int brt_nccl_world(int* world_rank, int* world_size);
BRT_API int brt_nccl_destroy(void);

/*
 * Replace brt::distributed::BroadCast / Exchange / Scatter / Gather / AllToAll
 * (include/brt/distributed/collective.h:18-56, src/distributed/collective.cc:13-88): grouped
 * ncclSend/ncclRecv of raw bytes on the library's communicator.  Sizes are int64 bytes.
 * brt_scatter / brt_gather: `bytes` is the per-rank piece; the root's buffer holds
 * world_size pieces.  brt_all_to_all: piece i of send goes to rank i, piece i of recv comes
 * from rank i.
 */
BRT_API int brt_broadcast(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                          void* stream);
BRT_API int brt_exchange(const void* send_buffer, void* recv_buffer, int64_t bytes, int dest,
                         int source, void* stream);
BRT_API int brt_scatter(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                        void* stream);
BRT_API int brt_gather(const void* send_buffer, void* recv_buffer, int64_t bytes, int root,
                       void* stream);
BRT_API int brt_all_to_all(const void* send_buffer, void* recv_buffer, int64_t slice_bytes,
                           void* stream);

/*
 * Replaces brt::distributed::AsymmetryAllToAll and GroupAsymmetryAllToAll
 * (include/brt/distributed/collective.h:57-74, src/distributed/collective.cc:90-140).
 * Both buffers are world_size * group_size slots of slot_bytes; slot (i, j) sends its first
 * send_sizes[i*G+j] grains to rank i and receives recv_sizes[i*G+j] grains from rank i.
 * group_size == 1 is the ungrouped form.  send_sizes / recv_sizes are HOST arrays.
 */
BRT_API int brt_group_asymmetry_all_to_all(const void* send_buffer, void* recv_buffer,
                                           const int32_t* send_sizes, const int32_t* recv_sizes,
                                           int64_t grain_bytes, int64_t slot_bytes,
                                           int group_size, void* stream);

/*
 * Replaces brt::distributed::GroupSparseAllToAllForward (forward != 0) and
 * GroupSparseAllToAllBackward (forward == 0)
 * (include/brt/distributed/collective.h:75-93, src/distributed/collective.cc:142-224).
 * Forward: the send buffer is packed in [rank i][local expert j] order with
 * send_sizes[i*G+j] rows per bucket; the receive buffer is filled in [local expert j][rank i]
 * order with recv_sizes[j*W+i] rows per bucket.  Backward swaps the two walks.
 * stride_rows != 0 places buckets stride_rows rows apart (max_path_padding) instead of back
 * to back.  Row size is grain_bytes.  send_sizes / recv_sizes are HOST arrays.
 */
BRT_API int brt_group_sparse_all_to_all(const void* send_buffer, void* recv_buffer,
                                        const int32_t* send_sizes, const int32_t* recv_sizes,
                                        int64_t grain_bytes, int64_t stride_rows, int group_size,
                                        int forward, void* stream);

/* ------------------------------------------------------------------ distributed: NVLink peer exchange */

#define BRT_P2P_HANDLE_BYTES 64

/*
 * Same exchange patterns as brt_group_sparse_all_to_all (src/distributed/collective.cc:
 * 142-224 in the reference), moved by this library's own kernels over NVLink peer memory
 * instead of NCCL send/recv.  No counterpart in the reference for the mechanism.
 *
 * brt_p2p_alloc   allocates an arena on the current device, zero-fills it and exports it as a
 *                 CUDA IPC handle (BRT_P2P_HANDLE_BYTES bytes) that the caller moves to the
 *                 other ranks of the box.  Setup-time call (this one does allocate).
 * brt_p2p_open    maps another rank's arena into this process; brt_p2p_close unmaps it;
 *                 brt_p2p_free releases an arena made by brt_p2p_alloc.
 * brt_p2p_push    copies `copy_count` (<= 96) byte ranges of `src` to absolute destination
 *                 addresses (inside peers' arenas or local memory; all 16-byte aligned and
 *                 sized) and then stores `epoch` into slot `my_rank` of every rank's flag
 *                 array.  `my_done_counter` is a zero-initialised 4-byte word in local memory.
 *                 world_size == 0: no flag is raised (a plain multi-range copy).
 * brt_p2p_post    writes `n` int32 values (this rank's bucket sizes; n may be 0) into row
 *                 `my_rank` of the size board in every rank's arena and raises slot `my_rank`
 *                 of the given flag arrays: the size exchange that precedes a data exchange
 *                 (the reference does it with an NCCL all-to-all,
 *                 src/backend/torch/distributed.cc:777-783) and, at the same time, the signal
 *                 that this rank has finished everything it enqueued before the exchange.
 * brt_p2p_land    one exchange of variable-size buckets planned on the device: waits (bounded)
 *                 until every slot of `my_ready_flags` holds a value >= epoch, reads the size
 *                 matrix [sender][destination * group_size + expert] from device memory and
 *                 copies every bucket this rank holds straight to its row offset in the
 *                 destination's OUTPUT layout inside landing_ptrs[destination] (peers' arenas
 *                 and the local one), then stores `epoch` into slot `my_rank` of every rank's
 *                 arrival flag array.  layout BRT_P2P_SPARSE_FORWARD: this rank's rows are
 *                 ordered [destination rank][its local expert] and land ordered
 *                 [local expert][source rank] (GroupSparseAllToAllForward);
 *                 BRT_P2P_SPARSE_INVERSE: the inverse (GroupSparseAllToAllBackward);
 *                 stride_rows != 0: buckets sit stride_rows rows apart on both sides.
 *                 BRT_P2P_SLOTS: the padded-slot exchange (GroupAsymmetryAllToAll,
 *                 collective.cc:108-140): slot (i, j) of stride_rows rows sends its first
 *                 S[me][i*G+j] rows into slot (me, j) of rank i; BRT_P2P_SLOTS_BACK: the same
 *                 move with the sizes this rank received in the slot exchange the matrix
 *                 belongs to.  zero_tails (slot layouts): the rows of this rank's own slots
 *                 beyond what they receive are zeroed (the reference's zeros_like outputs).  If some rank's landed rows exceed
 *                 half_bytes nothing is copied (every rank takes the same decision from the
 *                 same matrix) but the flags are still raised.  `keep_matrix` (may be null)
 *                 receives a copy of the matrix.  At most 1024 buckets.  When the wait runs out
 *                 the kernel writes BRT_ERR_TIMEOUT to `status_word` (device) and
 *                 `host_status_word` (device address of host-mapped memory, may be null),
 *                 copies nothing, raises no flag and returns.
 * brt_p2p_wait    enqueues a kernel that returns once every slot of `my_flag_array` (except
 *                 slot `skip_rank`, -1 for none) holds a value >= epoch.  A wait for this
 *                 rank's own landing kernel passes its own rank as skip_rank, so that it only
 *                 ever waits for kernels running on other GPUs.  The wait is bounded by
 *                 `wait_limit_ns`: on expiry it reports like brt_p2p_land and returns; it
 *                 never blocks the GPU indefinitely.
 */
#define BRT_P2P_SPARSE_INVERSE 0
#define BRT_P2P_SPARSE_FORWARD 1
#define BRT_P2P_SLOTS 2
#define BRT_P2P_SLOTS_BACK 3

BRT_API int brt_p2p_alloc(size_t bytes, void** dev_ptr, void* ipc_handle_out);
BRT_API int brt_p2p_open(const void* ipc_handle, void** peer_ptr);
BRT_API int brt_p2p_close(void* peer_ptr);
BRT_API int brt_p2p_free(void* dev_ptr);
BRT_API int brt_p2p_push(const void* src, int copy_count, const int64_t* src_offsets,
                         void* const* dst_ptrs, const int64_t* bytes, int world_size,
                         int my_rank, uint64_t epoch, void* const* peer_flag_arrays,
                         void* my_done_counter, void* stream);
BRT_API int brt_p2p_post(const int32_t* values, int n, int world_size, int my_rank,
                         uint64_t epoch, void* const* peer_boards, void* const* peer_flag_arrays,
                         void* stream);
BRT_API int brt_p2p_land(const void* rows, const int32_t* size_matrix, int32_t* keep_matrix,
                         int world_size, int group_size, int my_rank, int layout,
                         int zero_tails, int64_t grain_bytes, int64_t stride_rows,
                         int64_t half_bytes,
                         void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
                         void* const* peer_arrive_flag_arrays, void* my_done_counter,
                         void* my_abort_word, void* status_word, void* host_status_word,
                         uint64_t wait_limit_ns, void* stream);
BRT_API int brt_p2p_wait(const void* my_flag_array, int world_size, int skip_rank,
                         uint64_t epoch, void* status_word, void* host_status_word,
                         uint64_t wait_limit_ns, void* stream);
/* brt_p2p_land with the dispatch in front of it folded in (see
 * brt_p2p_dispatch_forward_begin): cells `src_data[cell_num, row_bytes]` go, by dense seat
 * indices `route_indices[cell_num, world_size * group_size]`, straight to their rows in the
 * destinations' landing halves; the size matrix row of this rank holds the loads. */
BRT_API int brt_p2p_dispatch_land(
    const void* src_data, const int32_t* route_indices, const int32_t* dense_counts,
    int64_t cell_num, int64_t row_bytes, const int32_t* size_matrix, int32_t* keep_matrix,
    int world_size, int group_size, int my_rank, int64_t stride_rows, int64_t half_bytes,
    void* const* landing_ptrs, uint64_t epoch, const void* my_ready_flags,
    void* const* peer_arrive_flag_arrays, void* my_done_counter, void* my_abort_word,
    void* status_word, void* host_status_word, uint64_t wait_limit_ns, void* stream);

/*
 * Exchange context: the host side of the two sparse exchanges on top of the calls above.  It
 * owns the bookkeeping of one arena (the exchange counter that serves as flag epoch, which
 * landing half is current, the size matrices kept for the inverse exchanges, a pinned buffer
 * for the sizes, a host-mapped status word).  The arena is brt_p2p_control_bytes() of control
 * block followed by two landing halves of `half_bytes` each; `arenas[r]` is rank r's arena as
 * mapped in this process (`my_arena` for r == my_rank).  Every rank must issue the same
 * exchanges in the same order.
 *
 * The output of an exchange is NOT copied anywhere: `out_data` points into this rank's
 * landing half of that exchange.  The halves alternate, and a peer only writes into a half
 * after this rank has entered the exchange that uses it, so an output stays valid until this
 * rank's stream reaches the second exchange after the one that produced it; work that reads
 * it must be enqueued (on the same stream) before that exchange.
 *
 * `stages` selects which parts of an exchange a call enqueues (0 = all).  A rank of a real
 * job always passes 0.  Separate stages exist so that several ranks can be driven from ONE
 * stream of one GPU (tests): all posts first, then all landings, then all waits, so that no
 * kernel ever waits for a kernel enqueued behind it.
 *
 * `layout` is BRT_P2P_SPARSE_FORWARD / BRT_P2P_SPARSE_INVERSE for the packed exchange and
 * BRT_P2P_SLOTS / BRT_P2P_SLOTS_BACK for the padded-slot one (asymmetry_all_to_all and
 * size_known_group_asymmetry_all_to_all, src/backend/torch/distributed.cc:339-753), whose
 * buffers are world_size * group_size slots of `stride_rows` rows on both sides.
 *
 * brt_p2p_sparse_forward_begin   group_sparse_all_to_all, part 1 (collective.cc:142-185):
 *                 post of `sizes` (DEVICE vector of world_size * group_size row counts), the
 *                 landing kernel and the wait for the peers' rows on `main_stream`; the copy
 *                 of the gathered size matrix to the host on `side_stream`, ordered behind the
 *                 post.  BRT_ERR_UNSUPPORTED: too many buckets, nothing enqueued.
 * brt_p2p_dispatch_forward_begin the same exchange FUSED with the dispatch in front of it
 *                 (python/brt/router/fabric/distributed.py:35-97 in the reference runs
 *                 dispatch_with_indices_and_loads, then group_sparse_all_to_all): the landing
 *                 kernel is replaced by a dispatch kernel that reads the cells
 *                 `src_data[cell_num, row_bytes]` and stores every kept copy straight into the
 *                 destination rank's landing half; the bucket sizes are `loads` (DEVICE,
 *                 world_size * group_size).  Unweighted 1-D routing with dense seat indices
 *                 (`dense_counts` as for brt_dispatch_with_indices_and_loads).  Followed by
 *                 brt_p2p_sparse_forward_sizes like the unfused call.
 * brt_p2p_sparse_forward_sizes   part 2: waits for the size matrix only (the rows are still
 *                 moving); returns the matrix ([sender][destination * group_size + expert],
 *                 valid until the next begin), the identifier under which it is kept for the
 *                 inverse exchange, this rank's output (rows ordered [local expert][source],
 *                 row count) and whether every rank's rows fit its landing half: if not,
 *                 nothing was moved, every rank sees the same and moves its rows another way.
 * brt_p2p_sparse_backward        size_known_group_sparse_all_to_all (collective.cc:187-224) of
 *                 the forward exchange `exchange_id`: every bucket goes back to its offset in
 *                 its owner's original layout.  BRT_ERR_UNSUPPORTED (nothing enqueued, same on
 *                 every rank): the matrix is no longer kept (32 are) or some rank's rows do
 *                 not fit a landing half.
 * brt_p2p_ctx_status             BRT_OK, or BRT_ERR_TIMEOUT once a bounded wait of an exchange
 *                 of this context has run out (read from host memory, no synchronisation);
 *                 later exchanges are then refused until brt_p2p_ctx_reset_status, which
 *                 puts the context back into its initial state (flags, exchange counts, kept
 *                 matrices: after a failed wait the ranks may have counted differently).
 *                 Every rank resets, with a host barrier before and after, and CUDA graphs
 *                 captured before the reset are captured again.
 * brt_p2p_ctx_set_wait_limit     the bound of every wait (default 2 s: the largest skew
 *                 between ranks that an exchange tolerates).
 *
 * Exchanges without a host synchronisation, fit for CUDA graph capture.  The reference's
 * forward exchange hands its size tensors to the host (collective.cc:157-166 synchronises the
 * stream for them); a layer whose experts read their loads on the device does not need that:
 * brt_p2p_ctx_replay_begin       opens a section.  Its forward exchanges are issued without
 *                 BRT_P2P_STAGE_SIZES and with BRT_P2P_STAGE_STRICT, and are completed by
 * brt_p2p_forward_device_sizes   (in place of brt_p2p_sparse_forward_sizes): writes the rows
 *                 this rank receives, [local expert][source rank] int32, to device memory
 *                 (stream-ordered, no synchronisation) and returns this rank's output - the
 *                 landing half, `capacity_rows` rows of the exchange's row size of which the
 *                 first sum(received) are the output - and the identifier for
 *                 brt_p2p_sparse_backward, whose `out_rows` is then a capacity as well.
 *                 Rows that do not fit a landing half cannot be rerouted without the host:
 *                 nothing moves and BRT_ERR_UNSUPPORTED appears in brt_p2p_ctx_status.
 * brt_p2p_ctx_replay_end         closes the section.  Its kernels may be captured in a CUDA
 *                 graph and replayed, or issued again, any number of times, between
 *                 ordinary exchanges too: the epoch of the flags is counted on the device
 *                 (it advances whenever an exchange runs, not when it is issued), and the
 *                 section has size boards and kept matrices of its own.  A replay lands in
 *                 the halves named when the section was issued; all ranks must replay alike.
 *                 The sections alive at one time may hold 16 forward exchanges in all.
 */
#define BRT_P2P_STAGE_POST 1
#define BRT_P2P_STAGE_SIZES 2
#define BRT_P2P_STAGE_PUSH 4
#define BRT_P2P_STAGE_WAIT 8
#define BRT_P2P_STAGE_ALL 15
#define BRT_P2P_STAGE_STRICT 16

typedef struct brt_p2p_ctx brt_p2p_ctx;
BRT_API size_t brt_p2p_control_bytes(void);
BRT_API int brt_p2p_ctx_create(int world_size, int my_rank, void* my_arena,
                               void* const* arenas, size_t half_bytes, brt_p2p_ctx** out);
BRT_API void brt_p2p_ctx_destroy(brt_p2p_ctx* ctx);
BRT_API int brt_p2p_ctx_set_wait_limit(brt_p2p_ctx* ctx, uint64_t nanoseconds);
BRT_API int brt_p2p_ctx_status(const brt_p2p_ctx* ctx);
BRT_API int brt_p2p_ctx_reset_status(brt_p2p_ctx* ctx);
BRT_API uint64_t brt_p2p_ctx_exchanges(const brt_p2p_ctx* ctx);
/* Where the last forward and the last inverse landing kernel of this context spent their
 * time (device clock, after a device synchronisation).  nanoseconds[0..4] for the forward
 * kernel: waiting for every rank to enter the exchange (skew, not work); from there until the
 * arrival flags were raised; and, counted from the same instant, when CTA 0 had its plan,
 * when the first CTA left its copy loop and when the last one did.  [5..9]: the inverse. */
BRT_API int brt_p2p_ctx_trace(brt_p2p_ctx* ctx, uint64_t* nanoseconds);
BRT_API int brt_p2p_sparse_forward_begin(brt_p2p_ctx* ctx, const void* rows,
                                         const int32_t* sizes, int group_size,
                                         int64_t grain_bytes, int64_t stride_rows, int layout,
                                         void* main_stream, void* side_stream, int stages);
BRT_API int brt_p2p_dispatch_forward_begin(brt_p2p_ctx* ctx, const void* src_data,
                                           const int32_t* route_indices, const int32_t* loads,
                                           const int32_t* dense_counts, int64_t cell_num,
                                           int64_t row_bytes, int group_size,
                                           int64_t stride_rows, void* main_stream,
                                           void* side_stream, int stages);
BRT_API int brt_p2p_sparse_forward_sizes(brt_p2p_ctx* ctx, void* side_stream,
                                         const int32_t** size_matrix, int64_t* out_rows,
                                         int* fits, void** out_data, uint64_t* exchange_id);
BRT_API int brt_p2p_ctx_replay_begin(brt_p2p_ctx* ctx);
BRT_API int brt_p2p_ctx_replay_end(brt_p2p_ctx* ctx);
BRT_API int brt_p2p_forward_device_sizes(brt_p2p_ctx* ctx, int32_t* received_sizes,
                                         void* stream, void** out_data,
                                         int64_t* capacity_rows, uint64_t* exchange_id);
/*
 * The inverse exchange and the weighted combine in ONE kernel (replaces
 * size_known_group_sparse_all_to_all followed by combine_with_indices_and_loads in
 * python/brt/router/fabric/distributed.py:120-158): the combine of this rank's cells pulls
 * every kept route's row straight from the arena of the rank that hosts the expert (16-byte
 * peer loads), in the layout forward exchange `exchange_id` landed, folds in ascending path
 * order with the roundings of brt_combine_with_indices_and_loads and writes dst_data
 * [cell_num, row_bytes] (fully written; a cell without a kept route becomes zero).
 * `expert_rows_offset`: byte offset, inside the arena, of the first row of the expert outputs;
 * the same on every rank, inside the landing halves (the landed rows themselves when the
 * experts work in place, else a buffer the experts wrote).  route_indices and gates as for
 * brt_combine_with_indices_and_loads (seat indices, no residual); the loads are those of the
 * forward exchange.  Stages POST | PUSH | WAIT as for the other exchanges: the post says "my
 * expert outputs are complete", the wait returns once every rank has finished reading this
 * rank's rows.  BRT_ERR_UNSUPPORTED (nothing enqueued): the matrix is no longer kept.
 */
BRT_API int brt_p2p_combine_backward(brt_p2p_ctx* ctx, uint64_t exchange_id, int group_size,
                                     int64_t row_bytes, int64_t stride_rows,
                                     int64_t expert_rows_offset, const int32_t* route_indices,
                                     const void* gates, int gates_dtype, int dtype,
                                     int64_t cell_num, void* dst_data, void* main_stream,
                                     int stages);
BRT_API int brt_p2p_sparse_backward(brt_p2p_ctx* ctx, uint64_t exchange_id, int group_size,
                                    int64_t grain_bytes, int64_t stride_rows, int layout,
                                    int zero_tails, const void* rows, void* main_stream,
                                    int stages, void** out_data, int64_t* out_rows);

#ifdef __cplusplus
}
#endif
#endif /* BRT_B200_H_ */
