// Device-side decoding of the packed GGUF weight rows (block layouts:
// tensor/dtype.go:102-151; arithmetic: tensor/quant.go:87-158,261-285).
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdint>

#include "yuuka_cuda.h"

namespace yk {

// Superblock = 256 consecutive elements of a row, for every dtype.
template <int DT> struct BlockTraits;
template <> struct BlockTraits<YUUKA_DTYPE_Q4_K> { static constexpr int sb_bytes = 144; };
template <> struct BlockTraits<YUUKA_DTYPE_Q5_K> { static constexpr int sb_bytes = 176; };
template <> struct BlockTraits<YUUKA_DTYPE_Q6_K> { static constexpr int sb_bytes = 210; };
template <> struct BlockTraits<YUUKA_DTYPE_Q8_0> { static constexpr int sb_bytes = 272; };
template <> struct BlockTraits<YUUKA_DTYPE_F16> { static constexpr int sb_bytes = 512; };
template <> struct BlockTraits<YUUKA_DTYPE_F32> { static constexpr int sb_bytes = 1024; };

__device__ __forceinline__ float ld_f16(const uint8_t * p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(p)));
}
__device__ __forceinline__ uint32_t ld_u16(const uint8_t * p) {
    return *reinterpret_cast<const uint16_t *>(p);
}
// 4 bytes from a 2-byte-aligned address
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t * p) {
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}

// 6-bit scale/min pair j of a Q4_K/Q5_K superblock (tensor/quant.go:96-103)
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t * q, int & sc, int & mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Eight consecutive elements [8*e8, 8*e8+8) of a packed row, as the CPU
// reference decodes them (same fp32 operations, same order).
template <int DT>
__device__ __forceinline__ void decode8(const uint8_t * row, int e8, float w[8]) {
    if constexpr (DT == YUUKA_DTYPE_F32) {
        const float * p = reinterpret_cast<const float *>(row) + e8 * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = p[i];
    } else if constexpr (DT == YUUKA_DTYPE_F16) {
        const uint8_t * p = row + e8 * 16;
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = ld_f16(p + 2 * i);
    } else if constexpr (DT == YUUKA_DTYPE_Q8_0) {
        const uint8_t * blk = row + (e8 >> 2) * 34;
        float d = ld_f16(blk);
        const uint8_t * q = blk + 2 + (e8 & 3) * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = d * (float)(int8_t)q[i];
    } else if constexpr (DT == YUUKA_DTYPE_Q4_K || DT == YUUKA_DTYPE_Q5_K) {
        constexpr int B = BlockTraits<DT>::sb_bytes;
        const uint8_t * blk = row + (e8 >> 5) * B;
        int idx = (e8 & 31) * 8, j64 = idx >> 6, half = (idx >> 5) & 1, l0 = idx & 31;
        float d = ld_f16(blk), dm = ld_f16(blk + 2);
        int sc, mn;
        scale_min_k4(2 * j64 + half, blk + 4, sc, mn);
        float d1 = d * (float)sc, m1 = dm * (float)mn;
        const uint8_t * ql = blk + (DT == YUUKA_DTYPE_Q4_K ? 16 : 48) + j64 * 32 + l0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int q = half ? (ql[i] >> 4) : (ql[i] & 0x0f);
            if constexpr (DT == YUUKA_DTYPE_Q5_K) {
                if (blk[16 + l0 + i] & (1 << (2 * j64 + half))) q += 16;
            }
            w[i] = d1 * (float)q - m1;
        }
    } else if constexpr (DT == YUUKA_DTYPE_Q6_K) {
        const uint8_t * blk = row + (e8 >> 5) * 210;
        int idx = (e8 & 31) * 8, n = idx >> 7, r = idx & 127, g = r >> 5, l0 = r & 31;
        float d = ld_f16(blk + 208);
        float ds = d * (float)(int8_t)blk[192 + n * 8 + (l0 >> 4) + 2 * g];
        const uint8_t * ql = blk + n * 64 + (g & 1) * 32 + l0;
        const uint8_t * qh = blk + 128 + n * 32 + l0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int q = ((ql[i] >> ((g >> 1) * 4)) & 0x0f) | (((qh[i] >> (2 * g)) & 3) << 4);
            w[i] = ds * (float)(q - 32);
        }
    }
}

// One element of a packed row (embedding gather).
__device__ __forceinline__ float dequant_elem(uint32_t dtype, const uint8_t * row, int i) {
    float w[8];
    switch (dtype) {
    case YUUKA_DTYPE_F32: return reinterpret_cast<const float *>(row)[i];
    case YUUKA_DTYPE_F16: return ld_f16(row + 2 * i);
    case YUUKA_DTYPE_Q8_0: decode8<YUUKA_DTYPE_Q8_0>(row, i >> 3, w); break;
    case YUUKA_DTYPE_Q4_K: decode8<YUUKA_DTYPE_Q4_K>(row, i >> 3, w); break;
    case YUUKA_DTYPE_Q5_K: decode8<YUUKA_DTYPE_Q5_K>(row, i >> 3, w); break;
    case YUUKA_DTYPE_Q6_K: decode8<YUUKA_DTYPE_Q6_K>(row, i >> 3, w); break;
    default: return 0.0f;
    }
    return w[i & 7];
}

// binary16 encode with the reference's rounding: half-up on the dropped bits
// (tensor/half.go:36-68), not ties-to-even. Keeps F16 KV rows bit-identical.
__device__ __forceinline__ uint16_t f32_to_f16_ref(float f) {
    uint32_t b = __float_as_uint(f);
    uint32_t sign = (b >> 16) & 0x8000u;
    int exp = (int)((b >> 23) & 0xff) - 127;
    uint32_t mant = b & 0x7fffffu;
    if (exp == 128) return (uint16_t)(sign | (mant ? 0x7e00u : 0x7c00u));
    if (exp > 15) return (uint16_t)(sign | 0x7c00u);
    if (exp < -24) return (uint16_t)sign;
    if (exp < -14) {
        uint32_t shift = (uint32_t)(-exp - 14);
        uint32_t rounded = (mant | 0x800000u) + (1u << (shift + 12));
        return (uint16_t)(sign | (rounded >> (shift + 13)));
    }
    uint32_t rounded = mant + 0x1000u;
    if (rounded & 0x800000u) {
        exp++;
        rounded = 0;
        if (exp > 15) return (uint16_t)(sign | 0x7c00u);
    }
    return (uint16_t)(sign | ((uint32_t)(exp + 15) << 10) | (rounded >> 13));
}

}  // namespace yk
