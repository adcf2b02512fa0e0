// Prepared activations: the form the MMA GEMM kernels read. For a row x[0..K):
//   xh[k]      = fp16(x[k]), natural order
//   xl[k]      = fp16(x[k] - xh[k]): the two halves together carry x to about 22 bits
//   xs16[k/16] = (hi, lo) fp16 pair of the sum of the sixteen values xh + xl
// The register-fed kernel multiplies the weights with both halves (two columns of the tensor-core
// product per activation row), so the fp16 operand type costs no accuracy; the tensor-memory kernel of
// wide passes reads xh alone. The sums feed the one extra MMA per superblock that applies the "- min"
// term of Q4_K / Q5_K. Row-wise producer kernels (RMSNorm, SwiGLU product, gated norms, attention merge)
// emit this form directly.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

namespace yk {

struct XPrepOut {
    __half * xh = nullptr;     // [rows][cols]
    __half * xl = nullptr;     // [rows][cols]
    __half2 * xs16 = nullptr;  // [rows][cols / 16]
};

// dst_* and v cover 16 consecutive elements starting at a multiple of 16
__device__ __forceinline__ void xprep_store16(__half * dst_hi, __half * dst_lo, __half2 * sum, const float (&v)[16]) {
    __half2 h[8], l[8];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        const float r0 = v[2 * i] - __low2float(h[i]), r1 = v[2 * i + 1] - __high2float(h[i]);
        l[i] = __floats2half2_rn(r0, r1);
        s += __low2float(h[i]) + __low2float(l[i]);
        s += __high2float(h[i]) + __high2float(l[i]);
    }
    uint4 * d = reinterpret_cast<uint4 *>(dst_hi);
    d[0] = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                      *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
    d[1] = make_uint4(*reinterpret_cast<uint32_t *>(&h[4]), *reinterpret_cast<uint32_t *>(&h[5]),
                      *reinterpret_cast<uint32_t *>(&h[6]), *reinterpret_cast<uint32_t *>(&h[7]));
    uint4 * e = reinterpret_cast<uint4 *>(dst_lo);
    e[0] = make_uint4(*reinterpret_cast<uint32_t *>(&l[0]), *reinterpret_cast<uint32_t *>(&l[1]),
                      *reinterpret_cast<uint32_t *>(&l[2]), *reinterpret_cast<uint32_t *>(&l[3]));
    e[1] = make_uint4(*reinterpret_cast<uint32_t *>(&l[4]), *reinterpret_cast<uint32_t *>(&l[5]),
                      *reinterpret_cast<uint32_t *>(&l[6]), *reinterpret_cast<uint32_t *>(&l[7]));
    const __half hi = __float2half_rn(s);
    const __half lo = __float2half_rn(s - __half2float(hi));
    *sum = __halves2half2(hi, lo);
}

// Both halves of one value.
__device__ __forceinline__ void xprep_split(float v, __half & hi, __half & lo) {
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

}  // namespace yk
