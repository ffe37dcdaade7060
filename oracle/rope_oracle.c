/*
 * TEST INFRASTRUCTURE - not part of the product.  Only tests/, the smoke check and the
 * CPU-baseline leg of bench.py may build, load or call this file.  libinfiniop never does.
 *
 * CPU restatement of the reference's rotary embedding, the operator a decode layer applies to q
 * and to the new K row before infiniopPagedCaching.  Unlike the paged operators this one has a
 * CPU kernel in the reference, and that is what is restated:
 *
 *   oracle_rope   src/infiniop/ops/rope/cpu/rope_cpu.cc:34-105 (calculateRoPE: offsets from the
 *                 captured strides, position id -> table row, the pair (2i, 2i+1) for GPT-J and
 *                 (i, i + dhead/2) for GPT-NeoX, 16-bit operands widened to fp32,
 *                 y0 = x0 cos - x1 sin, y1 = x0 sin + x1 cos, F32 / F64 in their own type)
 *
 * One deliberate difference: the reference's fp32 -> fp16 helper truncates the mantissa
 * (src/utils/custom_types.cc:39-63) while its bf16 helper, its CUDA kernels and the torch checker
 * of its tests (test/infiniop/rope.py:87-123, `.to(dt)`) round to nearest even; this file rounds
 * to nearest even for both 16-bit types, which is what the checker pins.  A position id outside
 * [0, table_len) copies the row (the reference reads outside its tables there).
 *
 * Parity pin: tests/test_oracle.py checks this file bit for bit against tests/golden/rope_*.npz,
 * produced by running the reference's own checker `rotary_embedding` (tests/golden/make_golden.py).
 *
 * Compiled without floating-point contraction so that products and sums round separately, as
 * they do in the reference's build.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_DTYPE_F16 12
#define ORACLE_DTYPE_F32 13
#define ORACLE_DTYPE_F64 14
#define ORACLE_DTYPE_BF16 19

/* codecs of paged_oracle.c (same shared object) */
uint16_t oracle_float_to_f16(float f);
uint16_t oracle_float_to_bf16(float f);
float oracle_f16_to_float(uint16_t h);
float oracle_bf16_to_float(uint16_t h);

static float load_as_float(const void *base, ptrdiff_t i, int dtype) {
    switch (dtype) {
    case ORACLE_DTYPE_F16:
        return oracle_f16_to_float(((const uint16_t *)base)[i]);
    case ORACLE_DTYPE_BF16:
        return oracle_bf16_to_float(((const uint16_t *)base)[i]);
    default:
        return ((const float *)base)[i];
    }
}

static void store_from_float(void *base, ptrdiff_t i, int dtype, float v) {
    switch (dtype) {
    case ORACLE_DTYPE_F16:
        ((uint16_t *)base)[i] = oracle_float_to_f16(v);
        break;
    case ORACLE_DTYPE_BF16:
        ((uint16_t *)base)[i] = oracle_float_to_bf16(v);
        break;
    default:
        ((float *)base)[i] = v;
        break;
    }
}

static size_t elem_bytes(int dtype) {
    return dtype == ORACLE_DTYPE_F64 ? 8 : (dtype == ORACLE_DTYPE_F32 ? 4 : 2);
}

/*
 * y, x: [batch, seqlen, nhead, 2 * table_dim] with the given element strides (last stride 1);
 * pos_ids: int64, [seqlen] (pos_batch_stride 0) or [batch, seqlen] (pos_batch_stride seqlen);
 * tables: [table_len, table_dim] contiguous.  gpt_j: 1 interleaved pairs, 0 half against half.
 * y may be x.  Returns 0, or -1 for an unsupported dtype.
 */
int oracle_rope(
    int dtype, int gpt_j,
    void *y, ptrdiff_t y_stride_batch, ptrdiff_t y_stride_seqlen, ptrdiff_t y_stride_nhead,
    const void *x, ptrdiff_t x_stride_batch, ptrdiff_t x_stride_seqlen, ptrdiff_t x_stride_nhead,
    const int64_t *pos_ids, ptrdiff_t pos_batch_stride,
    const void *sin_table, const void *cos_table,
    int64_t batch, int64_t seqlen, int64_t nhead, int64_t table_dim, int64_t table_len) {
    if (dtype != ORACLE_DTYPE_F16 && dtype != ORACLE_DTYPE_BF16 && dtype != ORACLE_DTYPE_F32 && dtype != ORACLE_DTYPE_F64) {
        return -1;
    }
    const size_t es = elem_bytes(dtype);
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t h = 0; h < nhead; ++h) {
            for (int64_t tok = 0; tok < seqlen; ++tok) {
                const ptrdiff_t xo = b * x_stride_batch + tok * x_stride_seqlen + h * x_stride_nhead;
                const ptrdiff_t yo = b * y_stride_batch + tok * y_stride_seqlen + h * y_stride_nhead;
                const int64_t pos = pos_ids[b * pos_batch_stride + tok];
                if (pos < 0 || pos >= table_len) {
                    memmove((unsigned char *)y + (size_t)yo * es, (const unsigned char *)x + (size_t)xo * es, (size_t)(2 * table_dim) * es);
                    continue;
                }
                const ptrdiff_t to = pos * table_dim;
                for (int64_t i = 0; i < table_dim; ++i) {
                    const ptrdiff_t p0 = gpt_j ? 2 * i : i;
                    const ptrdiff_t p1 = gpt_j ? 2 * i + 1 : i + table_dim;
                    if (dtype == ORACLE_DTYPE_F64) {
                        const double x0 = ((const double *)x)[xo + p0], x1 = ((const double *)x)[xo + p1];
                        const double s = ((const double *)sin_table)[to + i], c = ((const double *)cos_table)[to + i];
                        const double y0 = x0 * c - x1 * s;
                        const double y1 = x0 * s + x1 * c;
                        ((double *)y)[yo + p0] = y0;
                        ((double *)y)[yo + p1] = y1;
                    } else {
                        const float x0 = load_as_float(x, xo + p0, dtype), x1 = load_as_float(x, xo + p1, dtype);
                        const float s = load_as_float(sin_table, to + i, dtype), c = load_as_float(cos_table, to + i, dtype);
                        const float y0 = x0 * c - x1 * s;
                        const float y1 = x0 * s + x1 * c;
                        store_from_float(y, yo + p0, dtype, y0);
                        store_from_float(y, yo + p1, dtype, y1);
                    }
                }
            }
        }
    }
    return 0;
}
