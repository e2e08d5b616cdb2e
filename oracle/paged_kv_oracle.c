/*
 * paged_kv_oracle.c -- plain-C restatement of the reference's numpy goldens
 * for the paged-KV decode path.  TEST INFRASTRUCTURE ONLY: it is the checker
 * for large cases and the timed CPU baseline, never part of the product.
 *
 * Arithmetic followed (reference project paths):
 *   paged attention   tests/st/test_custom_paged_attention.py:586-614 (inputs to float32,
 *                     optional (int8 + offset) * descale per (kv_head, head_dim) channel),
 *                     :701-731 (gather K/V rows through the block table),
 *                     :937-1003 (q heads h*g..(h+1)*g-1 use kv head h),
 *                     :788-822 (scores * scale (+ mask), max-subtracted softmax, P @ V),
 *                     :644-646 (length-0 sequences give zeros)
 *   cache scatter     tests/st/test_custom_reshape_and_cache.py:282-307; negative slots
 *                     skipped as in ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/
 *                     reshape_and_cache_npd.cpp:149-150
 *   quantising scatter (no reference counterpart, "parity unpinned"): the inverse of the
 *                     de-quantisation above with round-half-to-even and saturation as in
 *                     tests/st/test_custom_kv_rmsnorm_rope_cache.py:310-314
 *
 * All arithmetic is float32, like the golden.  Work is spread over
 * (sequence, kv head) pairs with OpenMP; `threads` <= 0 uses every core.
 *
 * Parity status: pinned for paged attention and the plain scatter by
 * tests/golden (outputs of the reference's own golden functions); checked
 * against the numpy restatement in the CPU test-suite.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PKO_F16 0
#define PKO_BF16 1
#define PKO_I8 2
#define PKO_F32 3

static inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal */
      exp = 127 - 15 + 1;
      while (!(man & 0x400u)) { man <<= 1; --exp; }
      man &= 0x3ffu;
      bits = sign | (exp << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline float bf16_to_float(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline float load_elem(const void *p, int dtype, int64_t i) {
  switch (dtype) {
    case PKO_F16: return half_to_float(((const uint16_t *)p)[i]);
    case PKO_BF16: return bf16_to_float(((const uint16_t *)p)[i]);
    case PKO_I8: return (float)((const int8_t *)p)[i];
    default: return ((const float *)p)[i];
  }
}

/* one row of `d` elements to float32, optionally (x + offset) * descale */
static void load_row(float *dst, const void *src, int dtype, int64_t off, int d, const float *descale,
                     const int32_t *offset) {
  for (int i = 0; i < d; ++i) {
    float v = load_elem(src, dtype, off + i);
    if (descale) {
      if (offset) v += (float)offset[i];
      v *= descale[i];
    }
    dst[i] = v;
  }
}

__attribute__((target_clones("default", "avx2", "avx512f")))
static float dot_f32(const float *a, const float *b, int n) {
  float s = 0.f;
#pragma omp simd reduction(+ : s)
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

__attribute__((target_clones("default", "avx2", "avx512f")))
static void axpy_f32(float *y, float a, const float *x, int n) {
  for (int i = 0; i < n; ++i) y[i] += a * x[i];
}

/*
 * out: float32 [batch, q_heads, head_dim].  mask: float32 or NULL; element
 * (b, hq, j) at mask[b * mask_batch_stride + hq * mask_head_stride + j].
 * Returns 0, or -1 on a block id outside the cache, -2 on allocation failure.
 */
int pko_paged_attention(const void *query, int q_dtype, const void *key_cache, const void *value_cache,
                        int kv_dtype, const int32_t *block_tables, const int32_t *context_lens, int batch,
                        int q_heads, int kv_heads, int head_dim, int block_size, int64_t num_blocks,
                        int max_blocks_per_seq, float scale, const float *k_descale, const int32_t *k_offset,
                        const float *v_descale, const int32_t *v_offset, const float *mask,
                        int64_t mask_batch_stride, int64_t mask_head_stride, float *out, int threads) {
  const int g = q_heads / kv_heads, d = head_dim;
  int status = 0;
  if (threads <= 0) threads = omp_get_max_threads();
  memset(out, 0, (size_t)batch * q_heads * d * sizeof(float));
  const int64_t pairs = (int64_t)batch * kv_heads;
#pragma omp parallel num_threads(threads)
  {
    float *qf = (float *)malloc((size_t)g * d * sizeof(float));
    float *row = (float *)malloc((size_t)d * sizeof(float));
    float *scores = NULL;
    size_t scores_cap = 0;
#pragma omp for schedule(dynamic, 1)
    for (int64_t pr = 0; pr < pairs; ++pr) {
      const int b = (int)(pr / kv_heads), h = (int)(pr % kv_heads);
      const int len = context_lens[b];
      if (len <= 0 || qf == NULL || row == NULL) {
        if (qf == NULL || row == NULL) status = -2;
        continue;
      }
      if ((size_t)g * len > scores_cap) {
        free(scores);
        scores_cap = (size_t)g * len;
        scores = (float *)malloc(scores_cap * sizeof(float));
        if (scores == NULL) { scores_cap = 0; status = -2; continue; }
      }
      for (int r = 0; r < g; ++r)
        for (int i = 0; i < d; ++i)
          qf[r * d + i] = load_elem(query, q_dtype, ((int64_t)b * q_heads + h * g + r) * d + i);
      const float *kd = k_descale ? k_descale + (int64_t)h * d : NULL;
      const int32_t *ko = (k_descale && k_offset) ? k_offset + (int64_t)h * d : NULL;
      const float *vd = v_descale ? v_descale + (int64_t)h * d : NULL;
      const int32_t *vo = (v_descale && v_offset) ? v_offset + (int64_t)h * d : NULL;
      int bad = 0;
      /* scores = q . K^T * scale (+ mask) */
      for (int j = 0; j < len; ++j) {
        const int64_t blk = block_tables[(int64_t)b * max_blocks_per_seq + j / block_size];
        if (blk < 0 || blk >= num_blocks) { bad = 1; break; }
        const int64_t off = ((blk * block_size + j % block_size) * kv_heads + h) * d;
        load_row(row, key_cache, kv_dtype, off, d, kd, ko);
        for (int r = 0; r < g; ++r) {
          float s = dot_f32(qf + r * d, row, d) * scale;
          if (mask) s += mask[b * mask_batch_stride + (int64_t)(h * g + r) * mask_head_stride + j];
          scores[(size_t)r * len + j] = s;
        }
      }
      if (bad) { status = -1; continue; }
      /* max-subtracted softmax, row by row */
      for (int r = 0; r < g; ++r) {
        float *s = scores + (size_t)r * len;
        float mx = s[0];
        for (int j = 1; j < len; ++j) mx = s[j] > mx ? s[j] : mx;
        float sum = 0.f;
        for (int j = 0; j < len; ++j) { s[j] = expf(s[j] - mx); sum += s[j]; }
        for (int j = 0; j < len; ++j) s[j] /= sum;
      }
      /* out = P @ V */
      for (int j = 0; j < len; ++j) {
        const int64_t blk = block_tables[(int64_t)b * max_blocks_per_seq + j / block_size];
        const int64_t off = ((blk * block_size + j % block_size) * kv_heads + h) * d;
        load_row(row, value_cache, kv_dtype, off, d, vd, vo);
        for (int r = 0; r < g; ++r)
          axpy_f32(out + ((int64_t)b * q_heads + h * g + r) * d, scores[(size_t)r * len + j], row, d);
      }
    }
    free(qf);
    free(row);
    free(scores);
  }
  return status;
}

/* Bit copy of token rows into cache slots; slots < 0 skipped.  Rows in bytes. */
void pko_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                           const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_bytes,
                           int64_t v_row_bytes, int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
  /* sequential semantics on duplicate slots (later rows win) need a serial loop; slots are unique
     in every use of this oracle, so rows are spread over threads */
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int64_t i = 0; i < num_tokens; ++i) {
    const int64_t s = slot_mapping[i];
    if (s < 0) continue;
    memcpy((char *)key_cache + s * k_row_bytes, (const char *)key + i * k_row_bytes, (size_t)k_row_bytes);
    if (value && value_cache)
      memcpy((char *)value_cache + s * v_row_bytes, (const char *)value + i * v_row_bytes, (size_t)v_row_bytes);
  }
}

static inline int8_t quant_one(float x, float descale, float offset) {
  float q = nearbyintf(x / descale) - offset; /* default rounding mode: half to even */
  if (q != q) q = 0.f;
  if (q > 127.f) q = 127.f;
  if (q < -128.f) q = -128.f;
  return (int8_t)q;
}

/* q = saturate_int8(rint(float32(x) / descale[c]) - offset[c]) per channel, then scatter. */
void pko_reshape_and_cache_quant(const void *key, const void *value, int in_dtype, int8_t *key_cache,
                                 int8_t *value_cache, const int32_t *slot_mapping, int64_t num_tokens,
                                 int64_t k_row_elems, int64_t v_row_elems, const float *k_descale,
                                 const int32_t *k_offset, const float *v_descale, const int32_t *v_offset,
                                 int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int64_t i = 0; i < num_tokens; ++i) {
    const int64_t s = slot_mapping[i];
    if (s < 0) continue;
    for (int64_t c = 0; c < k_row_elems; ++c)
      key_cache[s * k_row_elems + c] =
          quant_one(load_elem(key, in_dtype, i * k_row_elems + c), k_descale[c], k_offset ? (float)k_offset[c] : 0.f);
    if (value && value_cache)
      for (int64_t c = 0; c < v_row_elems; ++c)
        value_cache[s * v_row_elems + c] = quant_one(load_elem(value, in_dtype, i * v_row_elems + c), v_descale[c],
                                                     v_offset ? (float)v_offset[c] : 0.f);
  }
}

/* paged_cache_load, ND layout (tests/st/test_custom_paged_cache_load.py:35-76): gather the rows of
   every sequence; blocks with a negative id contribute no rows and do not advance the output row, the
   rows left at the end are zero.  Two passes: first output row of every sequence (serial prefix over
   the valid rows), then the copies, sequences spread over threads.  Rows in bytes.  Returns the
   number of rows written. */
int64_t pko_paged_cache_load(const void *key_cache, const void *value_cache, const int32_t *block_tables,
                             const int32_t *seq_lens, const int32_t *seq_starts, void *key_out, void *value_out,
                             int batch, int max_blocks, int block_size, int64_t k_row_bytes, int64_t v_row_bytes,
                             int64_t sum_tokens, int cumsum, int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
  int64_t *first = (int64_t *)malloc(sizeof(int64_t) * (size_t)(batch + 1));
  if (!first) return -1;
  first[0] = 0;
  for (int i = 0; i < batch; ++i) {
    const int n = cumsum ? seq_lens[i + 1] - seq_lens[i] : seq_lens[i];
    const int off = seq_starts ? seq_starts[i] / block_size : 0;
    int64_t rows = 0;
    for (int j = 0; j < n; j += block_size) {
      const int col = off + j / block_size;
      if (col < max_blocks && block_tables[(int64_t)i * max_blocks + col] >= 0)
        rows += (n - j < block_size) ? n - j : block_size;
    }
    first[i + 1] = first[i] + rows;
  }
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (int i = 0; i < batch; ++i) {
    const int n = cumsum ? seq_lens[i + 1] - seq_lens[i] : seq_lens[i];
    const int off = seq_starts ? seq_starts[i] / block_size : 0;
    int64_t row = first[i];
    for (int j = 0; j < n; j += block_size) {
      const int col = off + j / block_size;
      if (col >= max_blocks) break;
      const int64_t bid = block_tables[(int64_t)i * max_blocks + col];
      if (bid < 0) continue;
      const int64_t m = (n - j < block_size) ? n - j : block_size;
      memcpy((char *)key_out + row * k_row_bytes, (const char *)key_cache + bid * block_size * k_row_bytes,
             (size_t)(m * k_row_bytes));
      memcpy((char *)value_out + row * v_row_bytes, (const char *)value_cache + bid * block_size * v_row_bytes,
             (size_t)(m * v_row_bytes));
      row += m;
    }
  }
  const int64_t written = first[batch];
  free(first);
  if (written < sum_tokens) {
    memset((char *)key_out + written * k_row_bytes, 0, (size_t)((sum_tokens - written) * k_row_bytes));
    memset((char *)value_out + written * v_row_bytes, 0, (size_t)((sum_tokens - written) * v_row_bytes));
  }
  return written;
}

/* fa_update (tests/st/test_asd_faupdate.py:34-59): out[r] = sum_s exp(lse[s][r]) / sum_s' exp(lse[s'][r])
   * local_out[s][r], float32, rows spread over threads. */
void pko_fa_update(const float *lse, const float *local_out, float *out, int64_t rows, int head_size, int sp,
                   int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float sum = 0.f;
    for (int s = 0; s < sp; ++s) sum += expf(lse[(int64_t)s * rows + r]);
    float *o = out + r * head_size;
    for (int d = 0; d < head_size; ++d) o[d] = 0.f;
    for (int s = 0; s < sp; ++s) {
      const float w = expf(lse[(int64_t)s * rows + r]) / sum;
      const float *x = local_out + ((int64_t)s * rows + r) * head_size;
      for (int d = 0; d < head_size; ++d) o[d] += w * x[d];
    }
  }
}

int pko_max_threads(void) { return omp_get_max_threads(); }
