// Prepared activations: the form the MMA GEMM kernels read. For a row x[0..K):
//   xh[k]    = fp16(x[k]), natural order
//   xs16[k/16] = (hi, lo) fp16 pair of the sum of the sixteen rounded values
// The sums feed the one extra MMA per superblock that applies the "- min" /
// "- offset" term of the K-quant formats. Row-wise producer kernels (RMSNorm,
// SwiGLU product, gated norms, attention merge) emit this form directly.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

namespace yk {

struct XPrepOut {
    __half * xh = nullptr;     // [rows][cols]
    __half2 * xs16 = nullptr;  // [rows][cols / 16]
};

// dst and v cover 16 consecutive elements starting at a multiple of 16
__device__ __forceinline__ void xprep_store16(__half * dst, __half2 * sum, const float (&v)[16]) {
    __half2 h[8];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        s += __low2float(h[i]);
        s += __high2float(h[i]);
    }
    uint4 * d = reinterpret_cast<uint4 *>(dst);
    d[0] = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                      *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
    d[1] = make_uint4(*reinterpret_cast<uint32_t *>(&h[4]), *reinterpret_cast<uint32_t *>(&h[5]),
                      *reinterpret_cast<uint32_t *>(&h[6]), *reinterpret_cast<uint32_t *>(&h[7]));
    const __half hi = __float2half_rn(s);
    const __half lo = __float2half_rn(s - __half2float(hi));
    *sum = __halves2half2(hi, lo);
}

}  // namespace yk
