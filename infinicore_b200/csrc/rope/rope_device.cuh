// Device-side pieces of the rotary embedding, shared by infiniopRoPE and by the decode step that
// rotates q and the new K row on its way into the paged cache.
//
// Arithmetic follows reference src/infiniop/ops/rope/cpu/rope_cpu.cc:78-101: 16-bit operands are
// widened to fp32, y0 = x0 cos - x1 sin and y1 = x0 sin + x1 cos with every product and sum rounded
// on its own (the _rn intrinsics keep the compiler from fusing them), one rounding to nearest even
// back to the storage type.
#ifndef INFINIOP_B200_ROPE_DEVICE_CUH
#define INFINIOP_B200_ROPE_DEVICE_CUH

#include "infiniop.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace b200::rope {

// A position id of any integer type as an unsigned 64-bit value: negative ids become huge and fail
// the `< table_len` test like any other id outside the tables.
__device__ __forceinline__ unsigned long long loadPosition(const void *base, long long i, int dtype) {
    switch (dtype) {
    case INFINI_DTYPE_I8:
        return static_cast<unsigned long long>(static_cast<long long>(static_cast<const signed char *>(base)[i]));
    case INFINI_DTYPE_U8:
        return static_cast<const unsigned char *>(base)[i];
    case INFINI_DTYPE_I16:
        return static_cast<unsigned long long>(static_cast<long long>(static_cast<const short *>(base)[i]));
    case INFINI_DTYPE_U16:
        return static_cast<const unsigned short *>(base)[i];
    case INFINI_DTYPE_I32:
        return static_cast<unsigned long long>(static_cast<long long>(static_cast<const int *>(base)[i]));
    case INFINI_DTYPE_U32:
        return static_cast<const unsigned int *>(base)[i];
    case INFINI_DTYPE_I64:
        return static_cast<unsigned long long>(static_cast<const long long *>(base)[i]);
    default: // INFINI_DTYPE_U64
        return static_cast<const unsigned long long *>(base)[i];
    }
}

__host__ __device__ inline bool isIntegerDtype(int dtype) {
    return dtype == INFINI_DTYPE_I8 || dtype == INFINI_DTYPE_U8 || dtype == INFINI_DTYPE_I16 || dtype == INFINI_DTYPE_U16
        || dtype == INFINI_DTYPE_I32 || dtype == INFINI_DTYPE_U32 || dtype == INFINI_DTYPE_I64 || dtype == INFINI_DTYPE_U64;
}

__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ double widen(double v) { return v; }

__device__ __forceinline__ void narrow(__half &dst, float v) { dst = __float2half_rn(v); }
__device__ __forceinline__ void narrow(__nv_bfloat16 &dst, float v) { dst = __float2bfloat16_rn(v); }
__device__ __forceinline__ void narrow(float &dst, float v) { dst = v; }
__device__ __forceinline__ void narrow(double &dst, double v) { dst = v; }

__device__ __forceinline__ void rotatePair(float a, float b, float s, float c, float &ya, float &yb) {
    ya = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    yb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}
__device__ __forceinline__ void rotatePair(double a, double b, double s, double c, double &ya, double &yb) {
    ya = __dsub_rn(__dmul_rn(a, c), __dmul_rn(b, s));
    yb = __dadd_rn(__dmul_rn(a, s), __dmul_rn(b, c));
}

// Two fp32 values rounded (to nearest even) and packed by one paired conversion.
__device__ __forceinline__ uint32_t packPair(float lo, float hi, __half) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t packPair(float lo, float hi, __nv_bfloat16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// Eight 16-bit values moved as one 128-bit word.
template <typename T>
union Pack8 {
    uint4 bits;
    uint32_t words[4];
    T v[8];
};

// Work of one row is cut into items, one per thread: with `vec` (16-bit types, every address involved a
// multiple of 16 bytes, table_dim a multiple of 8) an item is 8 pairs for GPT-NeoX (one 128-bit word from
// each half of the row) or 4 pairs for GPT-J (one 128-bit word); otherwise an item is one pair.
template <bool kGptJ>
__host__ __device__ inline int itemsPerRow(int table_dim, bool vec) {
    return vec ? (kGptJ ? table_dim / 4 : table_dim / 8) : table_dim;
}

// The vector path in three phases, so that a caller can put the loads of several items in flight before the
// first of them is needed: (1) the item's words of x, (2) its words of the two table rows, (3) rotate and store.
template <typename T>
struct VecItem {
    Pack8<T> a, b; // GPT-NeoX: word of the first half, word of the second half; GPT-J: `a` only
};
template <typename T>
struct VecTables {
    Pack8<T> s, c; // GPT-J uses the first four values of each
};

template <typename T, bool kGptJ>
__device__ __forceinline__ void loadItemVec(VecItem<T> &in, const T *x, int table_dim, int item) {
    if constexpr (kGptJ) {
        in.a.bits = *reinterpret_cast<const uint4 *>(x + 8 * item);
    } else {
        in.a.bits = *reinterpret_cast<const uint4 *>(x + 8 * item);
        in.b.bits = *reinterpret_cast<const uint4 *>(x + table_dim + 8 * item);
    }
}

template <typename T, bool kGptJ>
__device__ __forceinline__ void loadTablesVec(VecTables<T> &t, const T *sin_row, const T *cos_row, int item) {
    if (sin_row == nullptr) {
        return;
    }
    if constexpr (kGptJ) {
        const uint2 s = *reinterpret_cast<const uint2 *>(sin_row + 4 * item);
        const uint2 c = *reinterpret_cast<const uint2 *>(cos_row + 4 * item);
        t.s.words[0] = s.x, t.s.words[1] = s.y;
        t.c.words[0] = c.x, t.c.words[1] = c.y;
    } else {
        t.s.bits = *reinterpret_cast<const uint4 *>(sin_row + 8 * item);
        t.c.bits = *reinterpret_cast<const uint4 *>(cos_row + 8 * item);
    }
}

template <typename T, bool kGptJ>
__device__ __forceinline__ void rotateStoreVec(T *y, const VecItem<T> &in, const VecTables<T> &t, bool in_table, int table_dim, int item) {
    if constexpr (kGptJ) {
        Pack8<T> out;
        if (!in_table) {
            out.bits = in.a.bits;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float ya, yb;
                rotatePair(widen(in.a.v[2 * j]), widen(in.a.v[2 * j + 1]), widen(t.s.v[j]), widen(t.c.v[j]), ya, yb);
                out.words[j] = packPair(ya, yb, T());
            }
        }
        *reinterpret_cast<uint4 *>(y + 8 * item) = out.bits;
    } else {
        Pack8<T> out_lo, out_hi;
        if (!in_table) {
            out_lo.bits = in.a.bits;
            out_hi.bits = in.b.bits;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                float ya0, yb0, ya1, yb1;
                rotatePair(widen(in.a.v[j]), widen(in.b.v[j]), widen(t.s.v[j]), widen(t.c.v[j]), ya0, yb0);
                rotatePair(widen(in.a.v[j + 1]), widen(in.b.v[j + 1]), widen(t.s.v[j + 1]), widen(t.c.v[j + 1]), ya1, yb1);
                out_lo.words[j / 2] = packPair(ya0, ya1, T());
                out_hi.words[j / 2] = packPair(yb0, yb1, T());
            }
        }
        *reinterpret_cast<uint4 *>(y + 8 * item) = out_lo.bits;
        *reinterpret_cast<uint4 *>(y + table_dim + 8 * item) = out_hi.bits;
    }
}

// Rotates item `item` of one row of `2 * table_dim` elements: y and x point at the row, sin_row / cos_row
// at the table rows of its position (null: the position is outside the tables, the item is copied).
// A thread reads both elements of each of its pairs before it writes either, and no pair is shared
// between threads, so y == x (in place) is fine.
template <typename T, bool kGptJ>
__device__ __forceinline__ void rotateItem(T *y, const T *x, const T *sin_row, const T *cos_row, int table_dim, int item, bool vec) {
    if constexpr (sizeof(T) == 2) {
        if (vec) {
            VecItem<T> in;
            VecTables<T> t;
            loadItemVec<T, kGptJ>(in, x, table_dim, item);
            loadTablesVec<T, kGptJ>(t, sin_row, cos_row, item);
            rotateStoreVec<T, kGptJ>(y, in, t, sin_row != nullptr, table_dim, item);
            return;
        }
    }
    const int a = kGptJ ? 2 * item : item;
    const int b = kGptJ ? 2 * item + 1 : item + table_dim;
    if (sin_row == nullptr) {
        const T xa = x[a], xb = x[b];
        y[a] = xa;
        y[b] = xb;
        return;
    }
    decltype(widen(x[0])) ya, yb;
    rotatePair(widen(x[a]), widen(x[b]), widen(sin_row[item]), widen(cos_row[item]), ya, yb);
    narrow(y[a], ya);
    narrow(y[b], yb);
}

} // namespace b200::rope

#endif
