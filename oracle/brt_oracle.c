/*
 * CPU restatement of Brainstorm's routing hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared against, and the thing
 * the benchmark times as the CPU baseline.  Nothing in the shipped package may
 * import, link or call it.
 *
 * Every function states the reference source it follows (paths are relative to
 * the reference project root).  The arithmetic is integer/byte exact; floating
 * point follows the reference's operation order (one rounding per multiply, one
 * per add, paths in ascending order).
 *
 * Parity status: pinned.  The restatement reproduces the saved outputs of
 * sample/router/generate_indices.ipynb (seat indices, throttle) and the
 * round-trip identities of sample/cpp/dispatch.ipynb and
 * sample/distributed/sparse_a2a.py; see tests/test_oracle_golden.py.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off -shared; contraction
 * must stay off so that x*g and the add round separately)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2 };

/* ---- 16-bit float helpers ------------------------------------------------ */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}

static inline uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f; /* RNE */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}

static inline float load_as_f32(const void* p, int64_t i, int dtype) {
  if (dtype == ORACLE_F32) return ((const float*)p)[i];
  if (dtype == ORACLE_F16) return f16_to_f32(((const uint16_t*)p)[i]);
  return bf16_to_f32(((const uint16_t*)p)[i]);
}

static inline void store_from_f32(void* p, int64_t i, int dtype, float v) {
  if (dtype == ORACLE_F32)
    ((float*)p)[i] = v;
  else if (dtype == ORACLE_F16)
    ((uint16_t*)p)[i] = f32_to_f16(v);
  else
    ((uint16_t*)p)[i] = f32_to_bf16(v);
}

static inline int elem_size(int dtype) { return dtype == ORACLE_F32 ? 4 : 2; }

ORACLE_API int brt_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORACLE_API void brt_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---- loads rule ----------------------------------------------------------- */

/* src/router/location.cu:222-255: thread 0 of the path's block maps the real
 * load to the reported load. */
static int32_t map_load(int32_t real, int e, const int32_t* caps, int ncap, int capacity_padding,
                        int path_wise_padding) {
  if (capacity_padding && path_wise_padding) return caps[e];
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

/* src/router/location.cu:132-195 (per-path running sum, index = sum * mask),
 * :212-257 (loads), launcher :335-379 (path_wise_padding is only honoured when
 * capacity_padding is set; capacity_padding needs at least one capacity).
 * indices must be zero-filled by the caller, as the binding does
 * (src/backend/torch/router.cc:73).  Returns 0, or 1 on the launcher's CHECK. */
ORACLE_API int brt_oracle_generate_indices_and_loads(const int32_t* mask, int32_t* indices,
                                                     int32_t* loads, int64_t cell_num,
                                                     int path_num, const int32_t* caps, int ncap,
                                                     int capacity_padding, int path_wise_padding,
                                                     int is_tag_index) {
  if (capacity_padding && ncap < 1) return 1;
#pragma omp parallel for schedule(static)
  for (int e = 0; e < path_num; e++) {
    int32_t prefix = 0;
    for (int64_t t = 0; t < cell_num; t++) {
      int32_t m = mask[t * path_num + e];
      prefix += m;
      int32_t index = prefix * m;
      if (index != 0) {
        if (is_tag_index) {
          int64_t r = (int64_t)index - 1;
          if (r >= 0 && r < cell_num) indices[r * path_num + e] = (int32_t)(t + 1);
        } else {
          indices[t * path_num + e] = index;
        }
      }
    }
    loads[e] = map_load(prefix, e, caps, ncap, capacity_padding, path_wise_padding);
  }
  return 0;
}

/* src/router/location.cu:59-122.  The block walks its path in chunks of 1024
 * cells; a cell is kept when its mask is exactly 1 and prefix + running sum is
 * within the threshold; after each chunk the prefix absorbs the chunk's sum and
 * the walk stops once the threshold is reached.  prefix is updated in place.
 * throttled must be zero-filled by the caller (src/backend/torch/router.cc:26). */
ORACLE_API void brt_oracle_throttle_hotmask(const int32_t* mask, int32_t* throttled,
                                            int32_t* prefix, const int32_t* threshold,
                                            int64_t cell_num, int path_num) {
#pragma omp parallel for schedule(static)
  for (int e = 0; e < path_num; e++) {
    int32_t p = prefix[e];
    const int32_t thr = threshold[e];
    for (int64_t s = 0; s < cell_num; s += 1024) {
      int64_t end = s + 1024 < cell_num ? s + 1024 : cell_num;
      int32_t run = 0;
      for (int64_t t = s; t < end; t++) {
        int32_t m = mask[t * path_num + e];
        run += m;
        if (m == 1 && run + p <= thr) throttled[t * path_num + e] = 1;
      }
      p += run;
      if (p >= thr) {
        p = thr;
        break;
      }
    }
    prefix[e] = p;
  }
}

/* src/router/location.cu:259-302.  tag_to_seat selects the kernel exactly as
 * the launcher's flag does (:317-333).  The tag->seat kernel runs one block of
 * 1024 threads per path; a thread stops at the first zero tag it meets, so a
 * zero at row r hides rows r+1024, r+2048, ... of that path.  out must be
 * zero-filled by the caller. */
ORACLE_API void brt_oracle_convert_index_format(const int32_t* origin, int32_t* out,
                                                const int32_t* loads, int64_t cell_num,
                                                int path_num, int tag_to_seat) {
  if (!tag_to_seat) {
    for (int e = 0; e < path_num; e++)
      for (int64_t t = 0; t < cell_num; t++) {
        int32_t seat = origin[t * path_num + e];
        if (seat != 0) {
          int64_t r = (int64_t)seat - 1;
          if (r >= 0 && r < cell_num) out[r * path_num + e] = (int32_t)(t + 1);
        }
      }
  } else {
    for (int e = 0; e < path_num; e++) {
      int64_t load = loads[e];
      for (int lane = 0; lane < 1024; lane++) {
        for (int64_t r = lane; r < load; r += 1024) {
          int32_t tag = origin[r * path_num + e];
          if (tag == 0) break;
          int64_t c = (int64_t)tag - 1;
          if (c >= 0 && c < cell_num) out[c * path_num + e] = (int32_t)(r + 1);
        }
      }
    }
  }
}

/* ---- row addressing -------------------------------------------------------- */

/* src/router/route.cu:26-33: first output row of a path. */
static void path_bases(const int32_t* loads, int path_num, int32_t max_path_load, int64_t* base) {
  int64_t acc = 0;
  for (int e = 0; e < path_num; e++) {
    base[e] = max_path_load != 0 ? (int64_t)e * max_path_load : acc;
    acc += loads[e];
  }
}

static inline void copy_or_scale_row(const void* src, int64_t src_row, void* dst, int64_t dst_row,
                                     int64_t cell_size, int dtype, const void* gates,
                                     int64_t gate_idx) {
  const int es = elem_size(dtype);
  const char* s = (const char*)src + src_row * cell_size * es;
  char* d = (char*)dst + dst_row * cell_size * es;
  if (gates == NULL) {
    memcpy(d, s, (size_t)(cell_size * es));
    return;
  }
  /* src/router/route.cu:45-47: product formed in the data type, one rounding. */
  const float g = load_as_f32(gates, gate_idx, dtype);
  for (int64_t j = 0; j < cell_size; j++)
    store_from_f32(d, j, dtype, load_as_f32(s, j, dtype) * g);
}

/* Seat-index dispatch: src/router/route.cu:13-59 (1-D) and :116-158 (2-D).
 * 1-D: every path reads row t of in_data[cell_num, cell_size].
 * 2-D: path e reads in_data[t, e, :] (the binding hands the kernel a
 *      [path, cell, cell_size] transpose, src/backend/torch/router.cc:212).
 * out_data and new_tags must be zero-filled by the caller (router.cc:219,248).
 * Cells whose seat is 0 or beyond loads[e] are skipped. */
ORACLE_API void brt_oracle_dispatch_seat(const void* in_data, void* out_data, const void* gates,
                                         const int32_t* indices, const int32_t* loads,
                                         const int32_t* old_tags, int32_t* new_tags,
                                         int64_t cell_num, int64_t cell_size, int path_num,
                                         int32_t max_path_load, int is_1d, int dtype) {
  int64_t* base = (int64_t*)malloc(sizeof(int64_t) * (size_t)(path_num > 0 ? path_num : 1));
  path_bases(loads, path_num, max_path_load, base);
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < cell_num; t++) {
    for (int e = 0; e < path_num; e++) {
      int32_t seat = indices[t * path_num + e];
      if (seat == 0 || seat > loads[e]) continue;
      int64_t row = base[e] + seat - 1;
      int64_t src_row = is_1d ? t : t * path_num + e;
      copy_or_scale_row(in_data, src_row, out_data, row, cell_size, dtype, is_1d ? gates : NULL,
                        t * path_num + e);
      if (old_tags != NULL) new_tags[row] = old_tags[t];
    }
  }
  free(base);
}

/* Tag-index dispatch: src/router/route.cu:61-114 (1-D) and :160-206 (2-D).
 * grid.x = 512 blocks share a path; block b visits rows b, b+512, ... below
 * loads[e] and stops at the first zero tag it meets. */
ORACLE_API void brt_oracle_dispatch_tag(const void* in_data, void* out_data, const void* gates,
                                        const int32_t* indices, const int32_t* loads,
                                        const int32_t* old_tags, int32_t* new_tags,
                                        int64_t cell_num, int64_t cell_size, int path_num,
                                        int32_t max_path_load, int is_1d, int dtype) {
  int64_t* base = (int64_t*)malloc(sizeof(int64_t) * (size_t)(path_num > 0 ? path_num : 1));
  path_bases(loads, path_num, max_path_load, base);
  for (int e = 0; e < path_num; e++) {
    for (int b = 0; b < 512; b++) {
      for (int64_t i = b; i < cell_num; i += 512) {
        if (i >= loads[e]) continue;
        int32_t tag = indices[i * path_num + e];
        if (tag == 0) break;
        int64_t cell = (int64_t)tag - 1;
        int64_t row = base[e] + i;
        /* 2-D: element e of cell `cell` in the caller's [cell, path, :] layout,
         * which is what the kernel reads from its transposed copy. */
        int64_t src_row = is_1d ? cell : cell * path_num + e;
        copy_or_scale_row(in_data, src_row, out_data, row, cell_size, dtype,
                          is_1d ? gates : NULL, cell * path_num + e);
        if (old_tags != NULL) new_tags[row] = old_tags[cell];
      }
    }
  }
  free(base);
}

/* Seat-index combine: src/router/route.cu:208-248 and :250-282, launcher
 * :467-522.  For each cell, paths in ascending order; each term is rounded
 * (x * g) before it is added to the running fp32 sum.  is_residual: rows with at
 * least one kept route are zeroed first, other rows are left untouched;
 * otherwise out_data must be zero-filled by the caller (router.cc:441).
 * data_dtype selects how in/out elements are read and written (the reference
 * only has the fp32 instantiation, router.cc:435,443; 16-bit types accumulate in
 * fp32 and round once on store).  gates, if given, are fp32 unless
 * gates_dtype says otherwise. */
ORACLE_API void brt_oracle_combine_seat(const void* in_data, void* out_data, const void* gates,
                                        const int32_t* indices, const int32_t* loads,
                                        int64_t cell_num, int64_t cell_size, int path_num,
                                        int32_t max_path_load, int is_residual, int data_dtype,
                                        int gates_dtype) {
  int64_t* base = (int64_t*)malloc(sizeof(int64_t) * (size_t)(path_num > 0 ? path_num : 1));
  path_bases(loads, path_num, max_path_load, base);
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (size_t)(cell_size > 0 ? cell_size : 1));
#pragma omp for schedule(static)
    for (int64_t t = 0; t < cell_num; t++) {
      int routed = 0;
      for (int e = 0; e < path_num; e++) {
        int32_t seat = indices[t * path_num + e];
        if (seat == 0 || seat > loads[e]) continue;
        int64_t row = base[e] + seat - 1;
        if (!routed) {
          for (int64_t k = 0; k < cell_size; k++) acc[k] = 0.0f;
          routed = 1;
        }
        if (gates != NULL) {
          const float g = load_as_f32(gates, t * path_num + e, gates_dtype);
          for (int64_t k = 0; k < cell_size; k++) {
            const float term = load_as_f32(in_data, row * cell_size + k, data_dtype) * g;
            acc[k] = acc[k] + term;
          }
        } else {
          for (int64_t k = 0; k < cell_size; k++)
            acc[k] = acc[k] + load_as_f32(in_data, row * cell_size + k, data_dtype);
        }
      }
      if (routed) {
        for (int64_t k = 0; k < cell_size; k++)
          store_from_f32(out_data, t * cell_size + k, data_dtype, acc[k]);
      } else if (!is_residual) {
        for (int64_t k = 0; k < cell_size; k++)
          store_from_f32(out_data, t * cell_size + k, data_dtype, 0.0f);
      }
    }
    free(acc);
  }
  free(base);
}

/* ---- locality reorder ------------------------------------------------------ */

/* src/distributed/local_reorder.cu:15-63.  loads[c * W + o] = rows rank c got
 * from rank o.  W rounds: arg-max over the entries whose row and column are
 * still free (smallest flat index wins ties, CUB ArgMax), reorder[c] = o,
 * column c of the output is column o of the input. */
ORACLE_API void brt_oracle_locality_reorder(const int32_t* loads, int world_size,
                                            int32_t* reorder_indices, int32_t* reordered_loads) {
  const int W = world_size;
  int* row_used = (int*)calloc((size_t)W, sizeof(int));
  int* col_used = (int*)calloc((size_t)W, sizeof(int));
  for (int round = 0; round < W; round++) {
    int best = -1;
    int32_t best_v = 0;
    for (int i = 0; i < W * W; i++) {
      int c = i / W, o = i % W;
      int32_t v = (row_used[c] || col_used[o]) ? -1 : loads[i];
      if (best < 0 || v > best_v) {
        best = i;
        best_v = v;
      }
    }
    int c = best / W, o = best % W;
    reorder_indices[c] = o;
    row_used[c] = 1;
    col_used[o] = 1;
    for (int r = 0; r < W; r++) reordered_loads[r * W + c] = loads[r * W + o];
  }
  free(row_used);
  free(col_used);
}

/* src/distributed/local_reorder.cu:65-141.  loads[(c * W + o) * G + g]; the
 * matching runs on the per-(c, o) sums over g; the output permutes the o axis:
 * out[r, c, :] = in[r, reorder[c], :].  The reference's in-place tree sum is
 * only a full sum when G is a power of two; this restatement always sums all G
 * entries. */
ORACLE_API void brt_oracle_group_locality_reorder(const int32_t* loads, int group_size,
                                                  int world_size, int32_t* reorder_indices,
                                                  int32_t* reordered_loads) {
  const int W = world_size, G = group_size;
  int32_t* summed = (int32_t*)calloc((size_t)(W * W), sizeof(int32_t));
  int32_t* scratch = (int32_t*)calloc((size_t)(W * W), sizeof(int32_t));
  for (int i = 0; i < W * W; i++)
    for (int g = 0; g < G; g++) summed[i] += loads[(int64_t)i * G + g];
  brt_oracle_locality_reorder(summed, W, reorder_indices, scratch);
  for (int r = 0; r < W; r++)
    for (int c = 0; c < W; c++)
      for (int g = 0; g < G; g++)
        reordered_loads[((int64_t)r * W + c) * G + g] =
            loads[((int64_t)r * W + reorder_indices[c]) * G + g];
  free(summed);
  free(scratch);
}
