/*
 * TEST INFRASTRUCTURE - not part of the product.  Only tests/, the smoke check and the
 * CPU-baseline leg of bench.py may build, load or call this file.  libinfiniop never does.
 *
 * CPU restatement of the reference's checker for the paged decode path.  The reference has
 * no CPU kernel for these two operators (no CPU case in
 * src/infiniop/ops/paged_attention/operator.cc:42-69 and
 * src/infiniop/ops/paged_caching/operator.cc:38-64); what pins their results is the torch
 * code in its tests, and that is what is restated here:
 *
 *   oracle_paged_attention   test/infiniop/paged_attention.py:38-88
 *                            (ref_masked_attention, ref_single_query_cached_kv_attention)
 *   oracle_paged_caching     test/infiniop/paged_caching.py:25-55 (ref_paged_caching)
 *   oracle_paged_attention_prefill
 *                            test/infiniop/paged_attention_prefill.py:96-140
 *                            (ref_paged_attention_multi_turn: new token t of a chunk of n in a
 *                            sequence of total length L attends KV positions 0 .. L - n + t)
 *
 * plus the two edge cases those functions leave undefined and the reference kernels define:
 * a sequence with seq_len <= 0 leaves its output rows untouched
 * (src/infiniop/ops/paged_attention/cuda/kernel_v2.cuh:164-167) and a negative slot is skipped
 * (src/infiniop/ops/paged_caching/cuda/kernel.cuh:60-63).
 *
 * Parity pin: tests/test_oracle.py checks this file against tests/golden/*.npz, which were
 * produced by running the reference's own Python functions (tests/golden/make_golden.py).
 *
 * Two arithmetic modes:
 *   mode 0 "exact"     : everything in double from the exact fp16/bf16 input values; no
 *                        intermediate rounding.  The yardstick for error measurement.
 *   mode 1 "reference" : the roundings the torch reference performs - q.k accumulated in
 *                        fp32 and rounded to the tensor dtype, logits scaled in fp32, fp32
 *                        softmax, probabilities rounded to the tensor dtype, p.v accumulated
 *                        in fp32 and rounded to the tensor dtype.  Agrees with torch up to
 *                        summation order.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_DTYPE_F16 12
#define ORACLE_DTYPE_F32 13
#define ORACLE_DTYPE_BF16 19

/* ---- 16-bit float codecs ------------------------------------------------------------- */

static float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even on the upper 16 bits */
static uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static float f16_to_float(uint16_t h) {
    const int sign = (h >> 15) & 1;
    const int exp = (h >> 10) & 0x1f;
    const int man = h & 0x3ff;
    double v;
    if (exp == 0) {
        v = ldexp((double)man, -24);
    } else if (exp == 31) {
        v = man ? NAN : INFINITY;
    } else {
        v = ldexp((double)(man | 0x400), exp - 25);
    }
    return (float)(sign ? -v : v);
}

/* round-to-nearest-even to binary16 via exact double arithmetic */
static uint16_t float_to_f16(float f) {
    if (isnan(f)) {
        return 0x7e00;
    }
    const uint16_t sign = signbit(f) ? 0x8000u : 0u;
    double a = fabs((double)f);
    if (isinf(f) || a >= 65520.0) {
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a == 0.0) {
        return sign;
    }
    int e;
    (void)frexp(a, &e); /* a = m * 2^e, m in [0.5, 1)  => floor(log2 a) = e - 1 */
    int exp2 = e - 1;
    if (exp2 < -14) {
        exp2 = -14; /* subnormal range shares the smallest normal's quantum */
    }
    const double quantum = ldexp(1.0, exp2 - 10);
    const double q = nearbyint(a / quantum); /* ties to even under the default rounding mode */
    double r = q * quantum;
    if (r >= 65520.0) {
        return (uint16_t)(sign | 0x7c00u);
    }
    if (r == 0.0) {
        return sign;
    }
    (void)frexp(r, &e);
    exp2 = e - 1;
    if (exp2 < -14) {
        const uint16_t man = (uint16_t)nearbyint(ldexp(r, 24));
        return (uint16_t)(sign | man);
    }
    const uint16_t man = (uint16_t)(nearbyint(ldexp(r, 10 - exp2)) - 1024.0);
    return (uint16_t)(sign | ((uint16_t)(exp2 + 15) << 10) | man);
}

/* binary16 decode table: filled once (before any parallel region) so the hot loops stay cheap */
static float g_f16_table[65536];
static int g_f16_table_ready = 0;

static void ensure_f16_table(void) {
    if (!g_f16_table_ready) {
        for (uint32_t i = 0; i < 65536u; ++i) {
            g_f16_table[i] = f16_to_float((uint16_t)i);
        }
        g_f16_table_ready = 1;
    }
}

static inline float load16(const uint16_t *p, int dtype) {
    return dtype == ORACLE_DTYPE_BF16 ? bf16_to_float(*p) : g_f16_table[*p];
}

static inline float round16(float v, int dtype) {
    return dtype == ORACLE_DTYPE_BF16 ? bf16_to_float(float_to_bf16(v)) : f16_to_float(float_to_f16(v));
}

/* exported so the Python side can cross-check the codecs against numpy/torch */
uint16_t oracle_float_to_f16(float f) { return float_to_f16(f); }
uint16_t oracle_float_to_bf16(float f) { return float_to_bf16(f); }
float oracle_f16_to_float(uint16_t h) { return f16_to_float(h); }
float oracle_bf16_to_float(uint16_t h) { return bf16_to_float(h); }

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the number of OpenMP threads of later calls (a launcher may have exported OMP_NUM_THREADS=1 for its
 * worker processes; the timed CPU baseline wants every core the process may run on).  Returns the new count. */
int oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) {
        omp_set_num_threads(n);
    }
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* One query row (one q-head) against the first `len` tokens of one paged sequence.  `o` receives
 * value_size doubles.  Returns 0 or -5 (out of memory). */
static int attend_row(
    int mode, int dtype, double *o, const uint16_t *qv, int64_t len, int64_t kvh, int64_t h,
    const uint16_t *k_cache, ptrdiff_t k_block_stride, ptrdiff_t k_head_stride, ptrdiff_t k_row_stride,
    const uint16_t *v_cache, ptrdiff_t v_block_stride, ptrdiff_t v_head_stride, ptrdiff_t v_row_stride,
    const int64_t *block_table, const float *alibi_slopes, float scale,
    int64_t head_size, int64_t value_size, int64_t block_size) {
    float *qf = (float *)malloc(sizeof(float) * (size_t)head_size);
    double *logit = (double *)malloc(sizeof(double) * (size_t)len);
    double *acc = (double *)malloc(sizeof(double) * (size_t)value_size);
    if (!qf || !logit || !acc) {
        free(qf);
        free(logit);
        free(acc);
        return -5;
    }
    for (int64_t d = 0; d < head_size; ++d) {
        qf[d] = load16(qv + d, dtype);
    }

    /* logits = scale * (q . k) [+ slope * (t - (len - 1))] */
    double mx = -INFINITY;
    for (int64_t t = 0; t < len; ++t) {
        const int64_t blk = block_table[t / block_size];
        const uint16_t *kr = k_cache + blk * k_block_stride + kvh * k_head_stride + (t % block_size) * k_row_stride;
        double lg;
        if (mode == 0) {
            double dot = 0.0;
            for (int64_t d = 0; d < head_size; ++d) {
                dot += (double)qf[d] * (double)load16(kr + d, dtype);
            }
            lg = (double)scale * dot;
            if (alibi_slopes) {
                lg += (double)alibi_slopes[h] * (double)(t - len + 1);
            }
        } else {
            float dot = 0.f;
            for (int64_t d = 0; d < head_size; ++d) {
                dot += qf[d] * load16(kr + d, dtype);
            }
            float l32 = scale * round16(dot, dtype); /* einsum result is in the tensor dtype */
            if (alibi_slopes) {
                l32 += alibi_slopes[h] * (float)(t - len + 1);
            }
            lg = (double)l32;
        }
        logit[t] = lg;
        if (lg > mx) {
            mx = lg;
        }
    }

    /* softmax, then probabilities (rounded to the tensor dtype in mode 1) times V */
    double denom = 0.0;
    if (mode == 0) {
        for (int64_t t = 0; t < len; ++t) {
            logit[t] = exp(logit[t] - mx);
            denom += logit[t];
        }
    } else {
        float d32 = 0.f;
        for (int64_t t = 0; t < len; ++t) {
            const float e = expf((float)logit[t] - (float)mx);
            logit[t] = (double)e;
            d32 += e;
        }
        denom = (double)d32;
    }
    for (int64_t d = 0; d < value_size; ++d) {
        acc[d] = 0.0;
    }
    for (int64_t t = 0; t < len; ++t) {
        const int64_t blk = block_table[t / block_size];
        const uint16_t *vr = v_cache + blk * v_block_stride + kvh * v_head_stride + (t % block_size) * v_row_stride;
        if (mode == 0) {
            const double pw = logit[t] / denom;
            for (int64_t d = 0; d < value_size; ++d) {
                acc[d] += pw * (double)load16(vr + d, dtype);
            }
        } else {
            const float pw = round16((float)logit[t] / (float)denom, dtype);
            if (pw == 0.f) {
                continue;
            }
            for (int64_t d = 0; d < value_size; ++d) {
                acc[d] = (double)((float)acc[d] + pw * load16(vr + d, dtype));
            }
        }
    }
    for (int64_t d = 0; d < value_size; ++d) {
        o[d] = (mode == 0) ? acc[d] : (double)round16((float)acc[d], dtype);
    }
    free(qf);
    free(logit);
    free(acc);
    return 0;
}

/* ---- paged attention (decode) ----------------------------------------------------------
 * All strides are in elements.  out is dense double [num_seqs][num_heads][value_size]; rows of
 * sequences with seq_len <= 0 are not written.  Returns 0, or a negative code for a table
 * entry / length that points outside the pool.
 */
int oracle_paged_attention(
    int mode, int dtype,
    double *out,
    const uint16_t *q, ptrdiff_t q_seq_stride, ptrdiff_t q_head_stride,
    const uint16_t *k_cache, ptrdiff_t k_block_stride, ptrdiff_t k_head_stride, ptrdiff_t k_row_stride,
    const uint16_t *v_cache, ptrdiff_t v_block_stride, ptrdiff_t v_head_stride, ptrdiff_t v_row_stride,
    const int64_t *block_tables, ptrdiff_t bt_seq_stride,
    const int64_t *seq_lens,
    const float *alibi_slopes, /* may be NULL */
    float scale,
    int64_t num_seqs, int64_t num_heads, int64_t num_kv_heads,
    int64_t head_size, int64_t value_size, int64_t block_size,
    int64_t num_blocks, int64_t max_blocks_per_seq) {
    if (dtype != ORACLE_DTYPE_F16 && dtype != ORACLE_DTYPE_BF16) {
        return -1;
    }
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || block_size <= 0) {
        return -2;
    }
    const int64_t group = num_heads / num_kv_heads;
    int status = 0;
    ensure_f16_table();

    for (int64_t s = 0; s < num_seqs; ++s) {
        const int64_t len = seq_lens[s];
        if (len > max_blocks_per_seq * block_size) {
            return -3;
        }
        for (int64_t b = 0; b * block_size < len; ++b) {
            const int64_t blk = block_tables[s * bt_seq_stride + b];
            if (blk < 0 || blk >= num_blocks) {
                return -4;
            }
        }
    }

#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t s = 0; s < num_seqs; ++s) {
        for (int64_t h = 0; h < num_heads; ++h) {
            const int64_t len = seq_lens[s];
            if (len <= 0) {
                continue; /* output row untouched */
            }
            const int64_t kvh = h / group; /* repeat_interleave(keys, group, dim=1) */
            const int rc = attend_row(mode, dtype, out + (s * num_heads + h) * value_size,
                                      q + s * q_seq_stride + h * q_head_stride, len, kvh, h,
                                      k_cache, k_block_stride, k_head_stride, k_row_stride,
                                      v_cache, v_block_stride, v_head_stride, v_row_stride,
                                      block_tables + s * bt_seq_stride, alibi_slopes, scale,
                                      head_size, value_size, block_size);
            if (rc != 0) {
                status = rc;
            }
        }
    }
    return status;
}

/* ---- paged attention (prefill) -----------------------------------------------------------
 * q and out are packed over sequences: rows cum_q[i] .. cum_q[i+1]-1 are the new tokens of
 * sequence i, whose KV (new tokens included) is already in the cache and seq_lens[i] long.
 * out is dense double [total_q][num_heads][value_size]; rows no chunk covers are not written.
 */
int oracle_paged_attention_prefill(
    int mode, int dtype,
    double *out,
    const uint16_t *q, ptrdiff_t q_token_stride, ptrdiff_t q_head_stride,
    const uint16_t *k_cache, ptrdiff_t k_block_stride, ptrdiff_t k_head_stride, ptrdiff_t k_row_stride,
    const uint16_t *v_cache, ptrdiff_t v_block_stride, ptrdiff_t v_head_stride, ptrdiff_t v_row_stride,
    const int64_t *block_tables, ptrdiff_t bt_seq_stride,
    const int64_t *seq_lens, const int64_t *cum_q,
    const float *alibi_slopes, float scale,
    int64_t num_seqs, int64_t num_heads, int64_t num_kv_heads,
    int64_t head_size, int64_t value_size, int64_t block_size,
    int64_t num_blocks, int64_t max_blocks_per_seq) {
    if (dtype != ORACLE_DTYPE_F16 && dtype != ORACLE_DTYPE_BF16) {
        return -1;
    }
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || block_size <= 0) {
        return -2;
    }
    const int64_t group = num_heads / num_kv_heads;
    int status = 0;
    ensure_f16_table();
    for (int64_t s = 0; s < num_seqs; ++s) {
        const int64_t len = seq_lens[s];
        const int64_t n_new = cum_q[s + 1] - cum_q[s];
        if (n_new < 0 || len < n_new || len > max_blocks_per_seq * block_size) {
            return -3;
        }
        for (int64_t b = 0; b * block_size < len; ++b) {
            const int64_t blk = block_tables[s * bt_seq_stride + b];
            if (blk < 0 || blk >= num_blocks) {
                return -4;
            }
        }
    }
    for (int64_t s = 0; s < num_seqs; ++s) {
        const int64_t n_new = cum_q[s + 1] - cum_q[s];
        const int64_t cache_len = seq_lens[s] - n_new;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
        for (int64_t t = 0; t < n_new; ++t) {
            for (int64_t h = 0; h < num_heads; ++h) {
                const int64_t row = cum_q[s] + t;
                const int rc = attend_row(mode, dtype, out + (row * num_heads + h) * value_size,
                                          q + row * q_token_stride + h * q_head_stride, cache_len + t + 1, h / group, h,
                                          k_cache, k_block_stride, k_head_stride, k_row_stride,
                                          v_cache, v_block_stride, v_head_stride, v_row_stride,
                                          block_tables + s * bt_seq_stride, alibi_slopes, scale,
                                          head_size, value_size, block_size);
                if (rc != 0) {
                    status = rc;
                }
            }
        }
    }
    return status;
}

/* ---- paged caching ---------------------------------------------------------------------
 * Byte-exact scatter.  elem_size in bytes (2 or 4); strides in elements.  Tokens are applied in
 * index order, so with duplicate slots the last token wins (the GPU kernel leaves that case
 * unspecified, as the reference does).  Returns 0, or a negative code for an out-of-pool slot.
 */
int oracle_paged_caching(
    int64_t elem_size,
    unsigned char *k_cache, ptrdiff_t k_block_stride, ptrdiff_t k_head_stride, ptrdiff_t k_slot_stride,
    unsigned char *v_cache, ptrdiff_t v_block_stride, ptrdiff_t v_head_stride, ptrdiff_t v_slot_stride,
    const unsigned char *k, ptrdiff_t k_token_stride, ptrdiff_t k_src_head_stride,
    const unsigned char *v, ptrdiff_t v_token_stride, ptrdiff_t v_src_head_stride,
    const int64_t *slot_mapping,
    int64_t num_tokens, int64_t num_kv_heads, int64_t head_size, int64_t v_head_size,
    int64_t block_size, int64_t num_blocks) {
    if (block_size <= 0 || (elem_size != 2 && elem_size != 4)) {
        return -1;
    }
    for (int64_t i = 0; i < num_tokens; ++i) {
        const int64_t slot = slot_mapping[i];
        if (slot < 0) {
            continue; /* padding */
        }
        const int64_t blk = slot / block_size;
        const int64_t off = slot % block_size;
        if (blk >= num_blocks) {
            return -2;
        }
        for (int64_t h = 0; h < num_kv_heads; ++h) {
            memcpy(k_cache + (blk * k_block_stride + h * k_head_stride + off * k_slot_stride) * elem_size,
                   k + (i * k_token_stride + h * k_src_head_stride) * elem_size,
                   (size_t)(head_size * elem_size));
            memcpy(v_cache + (blk * v_block_stride + h * v_head_stride + off * v_slot_stride) * elem_size,
                   v + (i * v_token_stride + h * v_src_head_stride) * elem_size,
                   (size_t)(v_head_size * elem_size));
        }
    }
    return 0;
}
