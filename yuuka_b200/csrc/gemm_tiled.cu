// Quantized GEMM over tile-ordered weights (see gemm_tiled.cuh for the layout):
//   out[m][n] = sum_k x[m][k] * W[n][k]
// Replaces, for the verify step, kernels/hip/gemm/lm_head.hip,
// gemv/gemv_quant.hip:317 and the small-row use of gemm/wmma_gemm.hip.
//
// mma route (register-fed, exact). A warp owns a 16-row tile and a range of superblocks. Per superblock it
// issues coalesced 16-byte-per-lane loads of the next record (register double buffer), decodes the current
// record's block headers into a per-warp table, and builds mma.sync.m16n8k16 A fragments that hold exactly
// representable integers: one LOP3 places a nibble in the mantissa of 1024.0 and one fma.f16x2 with
// (sc, -1024 sc) yields sc * q for Q4_K / Q5_K (6-bit scale times quant, at most 1953); Q6_K uses q - 32,
// Q8_0 uses q. What is not an integer is applied in fp32 to the fp32 products: the superblock's d and -dmin
// once per 256 columns (the "- m" term is one more MMA per 128 columns of the 6-bit mins against
// per-16-column sums of the activations), d * sc per 16-column group of Q6_K, d per 32-column block of Q8_0.
// Activations are staged once per CTA as two fp16 halves (hi + lo = 22 bits of x) that occupy neighbouring
// product columns and are added after the record loop. Warps of a CTA that share a row tile split K and are
// summed through shared memory in a fixed order; a split of K across CTAs (long rows) goes through a scratch
// buffer and is finished by the last CTA to arrive, also in a fixed order. Nothing here waits on another CTA.
//
// fp32 route (on request, for tight-tolerance checks): same loads, the reference's
// own fp32 decode (tensor/quant.go:105-125,261-285), CUDA-core FMAs.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "gemm_tiled.cuh"
#include "quant.cuh"
#include "xprep.cuh"

namespace yk {

constexpr int TW = 8;            // warps per CTA (fp32 kernel, tensor-memory kernels)
constexpr int MW = 16;           // warps per CTA of the register-fed mma kernel: one CTA per SM
constexpr int MMA_ROWS = 16;     // activation rows per launch of that kernel (two product columns each)
constexpr uint32_t H2_1024 = 0x64006400u;

__device__ __forceinline__ uint4 ldg_stream(const uint4 * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void * p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// asks L2 for bytes [0, bytes) at base, one 128-byte line per lane and step
__device__ __forceinline__ void prefetch_l2_range(const uint8_t * base, int bytes, int lane) {
    for (int off = lane * 128; off < bytes; off += 32 * 128) prefetch_l2(base + off);
}
// (a & b) | c as one three-input logic instruction
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t dup_lo(uint32_t v) { return __byte_perm(v, v, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t v) { return __byte_perm(v, v, 0x3232); }
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr uint32_t H2_NEG1024 = 0xE400E400u;  // -1024
constexpr uint32_t H2_INV16 = 0x2C002C00u;    // 1/16
constexpr uint32_t H2_NEG64 = 0xD400D400u;    // -64
constexpr uint32_t H2_NEG1 = 0xBC00BC00u;     // -1
constexpr uint32_t H2_NEG32 = 0xD000D000u;    // -32
constexpr uint32_t H2_1152 = 0x64806480u;     // 1024 + 128

// bytes (0,1) / (2,3) of v as half2 (1024 + b)
__device__ __forceinline__ uint32_t bytes01_h2(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4140); }
__device__ __forceinline__ uint32_t bytes23_h2(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4342); }
__device__ __forceinline__ uint32_t bytes02_h2(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4240); }
__device__ __forceinline__ uint32_t bytes13_h2(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4341); }

template <typename XT> __device__ __forceinline__ float xf(XT v);
template <> __device__ __forceinline__ float xf<float>(float v) { return v; }
template <> __device__ __forceinline__ float xf<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// eight consecutive activations (16-byte aligned) as floats
__device__ __forceinline__ void load8(const float * src, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 * src, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(src);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
}

// ===========================================================================
// Record layouts.
//
// Element order. Inside a superblock, sub-block k (32 elements) is split over
// the four lanes t that share a weight row: lane t holds elements 32k + 8t + b,
// b = 0..7, i.e. MMA (k, h) takes elements 32k + 8t + 4h + {0,1,2,3} from lane
// t. Activations therefore stay in natural order: the B fragments of MMAs
// (k,0) and (k,1) are the 16 bytes x[32k + 8t .. 32k + 8t + 7]. (Q6_K: lane t
// holds 32k + 4t + b and 32k + 16 + 4t + b, b = 0..3, see pos6; its B fragments
// are the 8 bytes at x[32k + 16h + 4t].) A 4-byte weight
// word stores its four elements in byte order (0, 2, 1, 3) so that the masks
// 0x000f000f / (>>8) give the (k-lo, k-hi) halves of an A fragment directly.
//
// map(p) gives, for byte p of a record, the source row (0..15) and the byte
// offset inside that row's superblock in the GGUF layout.

template <int DT> struct Codec;

__device__ __forceinline__ int elem_in_chunk8(int c8) {  // byte position 0..7 of an 8-byte piece -> element b
    const int h = c8 >> 2, pos = c8 & 3;
    return 4 * h + ((pos & 1) * 2 + (pos >> 1));  // pos 0,1,2,3 -> element 0,2,1,3
}
// Q6_K only: which of the 32 positions of a sub-block element b (0..7) of lane t is. Q6_K scales cover 16
// elements, so the first four elements of every lane come from the sub-block's first half and the last four
// from its second half: MMA (k, h) then multiplies exactly the 16-element group 2k + h, whose scale is
// applied to the product afterwards, in fp32. (The other types scale per 32 elements: position 8t + b.)
__device__ __forceinline__ int pos6(int t, int b) { return b < 4 ? 4 * t + b : 16 + 4 * t + (b - 4); }

template <> struct Codec<YUUKA_DTYPE_Q4_K> {
    static constexpr int SB = 144, REC = 16 * SB;
    static constexpr int SCL_STRIDE = 80, MN_STRIDE = 48, MN_OFF = 16 * SCL_STRIDE, TAB = MN_OFF + 16 * MN_STRIDE;
    struct Regs { uint4 q[4]; uint4 hdr; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) {
            const int q = p >> 4, c16 = p & 15, i = q >> 5, lane = q & 31, g = lane >> 2, t = lane & 3;
            const int j = 2 * (i & 1) + (c16 >> 3);
            r = g + 8 * (i >> 1);
            o = 16 + 32 * j + 8 * t + elem_in_chunk8(c16 & 7);
        } else { r = (p - 2048) >> 4; o = p & 15; }
    }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = ldg_stream(p + i * 32 + lane);
        r.hdr = ldg_stream(p + 128 + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q5_K> {
    static constexpr int SB = 176, REC = 16 * SB;
    static constexpr int SCL_STRIDE = 80, MN_STRIDE = 48, MN_OFF = 16 * SCL_STRIDE, TAB = MN_OFF + 16 * MN_STRIDE;
    struct Regs { uint4 q[4]; uint4 qh; uint4 hdr; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) {
            const int q = p >> 4, c16 = p & 15, i = q >> 5, lane = q & 31, g = lane >> 2, t = lane & 3;
            const int j = 2 * (i & 1) + (c16 >> 3);
            r = g + 8 * (i >> 1);
            o = 48 + 32 * j + 8 * t + elem_in_chunk8(c16 & 7);
        } else if (p < 2560) {
            const int lane = (p - 2048) >> 4, c16 = p & 15, g = lane >> 2, t = lane & 3;
            r = g + 8 * (c16 >> 3);
            o = 16 + 8 * t + elem_in_chunk8(c16 & 7);
        } else { r = (p - 2560) >> 4; o = p & 15; }
    }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = ldg_stream(p + i * 32 + lane);
        r.qh = ldg_stream(p + 128 + lane);
        r.hdr = ldg_stream(p + 160 + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q6_K> {
    static constexpr int SB = 210, REC = 16 * SB;
    static constexpr int SCL_STRIDE = 144, MN_STRIDE = 80, MN_OFF = 16 * SCL_STRIDE, TAB = MN_OFF + 16 * MN_STRIDE;
    struct Regs { uint4 ql[4]; uint4 qh[2]; uint4 sc; uint32_t d; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) {
            const int q = p >> 4, c16 = p & 15, i = q >> 5, lane = q & 31, g = lane >> 2, t = lane & 3;
            r = g + 8 * (i >> 1);
            o = 64 * (i & 1) + 32 * (c16 >> 3) + pos6(t, elem_in_chunk8(c16 & 7));
        } else if (p < 3072) {
            const int q = (p - 2048) >> 4, c16 = p & 15, lane = q & 31, g = lane >> 2, t = lane & 3;
            r = g + 8 * (q >> 5);
            o = 128 + 32 * (c16 >> 3) + pos6(t, elem_in_chunk8(c16 & 7));
        } else if (p < 3328) { r = (p - 3072) >> 4; o = 192 + (p & 15); }
        else { r = (p - 3328) >> 1; o = 208 + (p & 1); }
    }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
#pragma unroll
        for (int i = 0; i < 4; i++) r.ql[i] = ldg_stream(p + i * 32 + lane);
        r.qh[0] = ldg_stream(p + 128 + lane);
        r.qh[1] = ldg_stream(p + 160 + lane);
        r.sc = ldg_stream(p + 192 + (lane & 15));
        r.d = __ldg(reinterpret_cast<const uint16_t *>(rec + 3328) + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q8_0> {
    static constexpr int SB = 272, REC = 16 * SB;
    static constexpr int SCL_STRIDE = 48, MN_OFF = 0, TAB = 16 * SCL_STRIDE;
    struct Regs { uint4 q[8]; uint4 d; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 4096) {
            const int q = p >> 4, c16 = p & 15, i = q >> 5, lane = q & 31, g = lane >> 2, t = lane & 3;
            const int k = 2 * (i & 3) + (c16 >> 3);
            r = g + 8 * (i >> 2);
            o = 34 * k + 2 + 8 * t + elem_in_chunk8(c16 & 7);
        } else { r = (p - 4096) >> 4; const int k = (p & 15) >> 1; o = 34 * k + (p & 1); }
    }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = ldg_stream(p + i * 32 + lane);
        r.d = ldg_stream(p + 256 + (lane & 15));
    }
};

// ---------------------------------------------------------------------------
// tiling kernel: one thread per 16 output bytes

template <int DT>
__global__ void tile_weights_kernel(uint8_t * __restrict__ dst, const uint8_t * __restrict__ src, int n_out, int nsb,
                                    int64_t rb, int64_t n_chunks) {
    using C = Codec<DT>;
    for (int64_t ch = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; ch < n_chunks; ch += (int64_t)gridDim.x * blockDim.x) {
        const int64_t rec = ch / (C::REC / 16);
        const int p0 = (int)(ch - rec * (C::REC / 16)) * 16;
        const int64_t rt = rec / nsb, sb = rec - rt * nsb;
        uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
        for (int b = 0; b < 16; b++) {
            int r, o;
            C::map(p0 + b, r, o);
            const int64_t row = rt * 16 + r;
            uint32_t v = row < n_out ? src[row * rb + sb * C::SB + o] : 0u;
            w[b >> 2] |= v << (8 * (b & 3));
        }
        reinterpret_cast<uint4 *>(dst)[ch] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

void launch_tile_weights(cudaStream_t s, uint8_t * dst, const uint8_t * src, uint32_t dtype, int n_out, int n_in) {
    YK_REQUIRE(tiled_supported(dtype, n_in), YUUKA_ERR_UNSUPPORTED, "dtype %u / width %d has no tiled layout", dtype, n_in);
    const int nsb = n_in / 256;
    const int64_t n_chunks = (int64_t)tiled_bytes(dtype, n_out, n_in) / 16;
    const int64_t rb = (int64_t)row_bytes(dtype, n_in);
    int64_t blocks = (n_chunks + 255) / 256;
    if (blocks > 65535 * 16) blocks = 65535 * 16;
    switch (dtype) {
    case YUUKA_DTYPE_Q4_K: tile_weights_kernel<YUUKA_DTYPE_Q4_K><<<(unsigned)blocks, 256, 0, s>>>(dst, src, n_out, nsb, rb, n_chunks); break;
    case YUUKA_DTYPE_Q5_K: tile_weights_kernel<YUUKA_DTYPE_Q5_K><<<(unsigned)blocks, 256, 0, s>>>(dst, src, n_out, nsb, rb, n_chunks); break;
    case YUUKA_DTYPE_Q6_K: tile_weights_kernel<YUUKA_DTYPE_Q6_K><<<(unsigned)blocks, 256, 0, s>>>(dst, src, n_out, nsb, rb, n_chunks); break;
    default: tile_weights_kernel<YUUKA_DTYPE_Q8_0><<<(unsigned)blocks, 256, 0, s>>>(dst, src, n_out, nsb, rb, n_chunks); break;
    }
    YK_CUDA(cudaGetLastError());
}

// ===========================================================================
// Prepared activations: fp16 copy of x in natural order plus, per 16 elements,
// the sum of the rounded values as a (hi, lo) half pair. The MMA kernels read
// only this form; row-wise producer kernels can emit it directly.

template <typename XT>
__global__ void xprep_kernel(__half * __restrict__ xh, __half * __restrict__ xl, __half2 * __restrict__ xs16, const XT * __restrict__ x, int64_t ldx,
                             int K, int M) {
    const int groups = K >> 4;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * groups; i += gridDim.x * blockDim.x) {
        const int m = i / groups, gq = i - m * groups;
        float v[16];
        load8(x + (int64_t)m * ldx + gq * 16, *reinterpret_cast<float(*)[8]>(v));
        load8(x + (int64_t)m * ldx + gq * 16 + 8, *reinterpret_cast<float(*)[8]>(v + 8));
        xprep_store16(xh + (int64_t)m * K + gq * 16, xl + (int64_t)m * K + gq * 16, xs16 + (int64_t)m * groups + gq, v);
    }
}

template <typename XT>
static void launch_xprep(cudaStream_t s, __half * xh, __half * xl, __half2 * xs16, const XT * x, int64_t ldx, int K, int M) {
    const int total = M * (K / 16);
    xprep_kernel<XT><<<(total + 127) / 128, 128, 0, s>>>(xh, xl, xs16, x, ldx, K, M);
    YK_CUDA(cudaGetLastError());
}

// ===========================================================================
// header decode -> per-warp tables, and the per-superblock MMA sequence

// Q4_K / Q5_K header: hdr.x = d | dmin << 16, hdr.y/z/w = 12 scale bytes.
// scl[row][pair j] = {s_lo, -1024 s_lo, s_hi/16, -64 s_hi} (half2 each); mn2[row][sub] = (-min, -min).
template <typename C>
__device__ __forceinline__ void header_k4(const uint4 & hdr, int lane, uint8_t * tab) {
    const int r = lane & 15, hf = lane >> 4;  // hf: pairs 2hf, 2hf+1
    const uint32_t d2 = dup_lo(hdr.x), dm2 = dup_hi(hdr.x);
    const uint32_t w0 = hdr.y, w1 = hdr.z, w2 = hdr.w;
    const uint32_t sc4 = hf ? ((w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u)) : (w0 & 0x3f3f3f3fu);
    const uint32_t mn4 = hf ? (((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u)) : (w1 & 0x3f3f3f3fu);
    uint4 * scl = reinterpret_cast<uint4 *>(tab + r * C::SCL_STRIDE) + hf * 2;
    uint2 * mn2 = reinterpret_cast<uint2 *>(tab + C::MN_OFF + r * C::MN_STRIDE) + hf * 2;
#pragma unroll
    for (int jl = 0; jl < 2; jl++) {
        const uint32_t sp = h2_mul(h2_sub(jl ? bytes23_h2(sc4) : bytes01_h2(sc4), H2_1024), d2);
        const uint32_t mp = h2_mul(h2_sub(jl ? bytes23_h2(mn4) : bytes01_h2(mn4), H2_1024), dm2);
        const uint32_t slo = dup_lo(sp), shi = dup_hi(sp);
        scl[jl] = make_uint4(slo, h2_mul(slo, H2_NEG1024), h2_mul(shi, H2_INV16), h2_mul(shi, H2_NEG64));
        mn2[jl] = make_uint2(h2_mul(dup_lo(mp), H2_NEG1), h2_mul(dup_hi(mp), H2_NEG1));
    }
}

// Bit masks and the fp16 "1024" pattern as run-time values (kernel parameters). A LOP3 takes one
// immediate only; with two compile-time constants in (v & mask) | 0x6400'6400 the compiler emits two
// instructions per weight pair, with values it cannot see through it emits one.
struct DecodeConsts {
    uint32_t m0f;    // 0x000f000f
    uint32_t mf0;    // 0x00f000f0
    uint32_t magic;  // 0x64006400
    uint32_t h4;     // 0x00300030 (Q6_K high bits, low-nibble form); Q5_K: 0x00100010
    uint32_t h8;     // 0x03000300 (Q6_K high bits, high-nibble form); Q5_K: 0x01000100
};
inline DecodeConsts decode_consts(uint32_t dtype) {
    DecodeConsts c{0x000f000fu, 0x00f000f0u, 0x64006400u, 0x00300030u, 0x03000300u};
    if (dtype == YUUKA_DTYPE_Q5_K) {
        c.h4 = 0x00100010u;
        c.h8 = 0x01000100u;
    }
    return c;
}

// ---------------------------------------------------------------------------
// Scaled decode (tensor-memory route, gemm_umma.cuh): block headers become per-warp tables of fp16
// scales with which a packed weight turns into fp16(s * q) by one LOP3 and one fma.f16x2.

template <int DT, int NT> struct Mma;

template <int NT> struct Mma<YUUKA_DTYPE_Q4_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q4_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4<C>(r.hdr, lane, tab); }
};

template <int NT> struct Mma<YUUKA_DTYPE_Q5_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q5_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4<C>(r.hdr, lane, tab); }
    // bit k of every byte of hb -> bit `tgt` of bytes 0 and 2 (shift_bytes13: of bytes 1 and 3 moved down)
    // ... merged with the fp16 1024 pattern: ((hb shifted) & bit) | magic is one LOP3
    template <int K, int TGT, bool B13> __device__ static uint32_t hibit(uint32_t hb, uint32_t bit, uint32_t magic) {
        constexpr int from = K + (B13 ? 8 : 0);
        if constexpr (from >= TGT) return and_or(hb >> (from - TGT), bit, magic);
        else return and_or(hb << (TGT - from), bit, magic);
    }
    template <int K> __device__ static void sub(uint32_t vg, uint32_t vh, uint32_t hg, uint32_t hh, uint32_t s_g, uint32_t c_g,
                                                uint32_t s_h, uint32_t c_h, uint32_t (&a)[4], const DecodeConsts & kc) {
        constexpr bool hi = (K & 1) != 0;
        constexpr int tgt = hi ? 8 : 4;
        const uint32_t mask = hi ? kc.mf0 : kc.m0f, bit = hi ? kc.h8 : kc.h4;
        a[0] = h2_fma(and_or(vg, mask, hibit<K, tgt, false>(hg, bit, kc.magic)), s_g, c_g);
        a[1] = h2_fma(and_or(vh, mask, hibit<K, tgt, false>(hh, bit, kc.magic)), s_h, c_h);
        a[2] = h2_fma(and_or(vg >> 8, mask, hibit<K, tgt, true>(hg, bit, kc.magic)), s_g, c_g);
        a[3] = h2_fma(and_or(vh >> 8, mask, hibit<K, tgt, true>(hh, bit, kc.magic)), s_h, c_h);
    }
};

// Q6_K: scl[row][s16] = {s', c'} with (s, -1024 s) where the value sits in a low nibble
// (s16 % 8 < 4) and (s/16, -64 s) where it sits in a high nibble; mn2[row][s16] = (-32 s, -32 s).
template <int NT> struct Mma<YUUKA_DTYPE_Q6_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q6_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;  // hf: groups 8hf .. 8hf+7
        const uint32_t d2 = dup_lo(r.d);
        const uint32_t wa = (hf ? r.sc.z : r.sc.x) ^ 0x80808080u;  // groups +0..3: low-nibble form
        const uint32_t wb = (hf ? r.sc.w : r.sc.y) ^ 0x80808080u;  // groups +4..7: high-nibble form
        uint2 * scl = reinterpret_cast<uint2 *>(tab + row * C::SCL_STRIDE) + hf * 8;
        uint32_t * mn2 = reinterpret_cast<uint32_t *>(tab + C::MN_OFF + row * C::MN_STRIDE) + hf * 8;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t w = q < 2 ? wa : wb;
            const uint32_t sp = h2_mul(h2_sub((q & 1) ? bytes23_h2(w) : bytes01_h2(w), H2_1152), d2);
            const uint32_t s0 = dup_lo(sp), s1 = dup_hi(sp);
            if (q < 2) {
                scl[2 * q] = make_uint2(s0, h2_mul(s0, H2_NEG1024));
                scl[2 * q + 1] = make_uint2(s1, h2_mul(s1, H2_NEG1024));
            } else {
                scl[2 * q] = make_uint2(h2_mul(s0, H2_INV16), h2_mul(s0, H2_NEG64));
                scl[2 * q + 1] = make_uint2(h2_mul(s1, H2_INV16), h2_mul(s1, H2_NEG64));
            }
            mn2[2 * q] = h2_mul(s0, H2_NEG32);
            mn2[2 * q + 1] = h2_mul(s1, H2_NEG32);
        }
    }
};

// Q8_0: scl[row][block] = (s, s).
template <int NT> struct Mma<YUUKA_DTYPE_Q8_0, NT> {
    using C = Codec<YUUKA_DTYPE_Q8_0>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;
        const uint32_t da = hf ? r.d.z : r.d.x, db = hf ? r.d.w : r.d.y;
        uint32_t * scl = reinterpret_cast<uint32_t *>(tab + row * C::SCL_STRIDE) + hf * 4;
        scl[0] = dup_lo(da);
        scl[1] = dup_hi(da);
        scl[2] = dup_lo(db);
        scl[3] = dup_hi(db);
    }
};

// ---------------------------------------------------------------------------
// Exact decode (register-fed route, 1..16 activation rows per launch). The fp16 operand of the tensor core
// holds an integer that fp16 represents exactly, and every floating-point factor of the format is applied
// to the fp32 product afterwards, so the weights enter the sum with the value tensor/quant.go gives them:
//   Q4_K / Q5_K  w = d * (sc * q) - dmin * m: the operand is sc * q (at most 63 * 31), summed over the whole
//                superblock; m (at most 63) times the sums of the activations goes through one more MMA per
//                128 columns; d and dmin multiply the two fp32 sums once per superblock;
//   Q6_K         w = d * sc * (q - 32): the operand is q - 32; MMA (k, h) covers the 16-element group 2k + h
//                (see pos6), whose product is multiplied by d * sc;
//   Q8_0         w = d * q: the operand is q, the product of a 32-element block is multiplied by d.
// Activations enter as two fp16 halves, hi + lo, in neighbouring columns of the product (about 22 bits).

constexpr uint32_t H2_ONE = 0x3C003C00u;      // 1
constexpr uint32_t H2_NEG1056 = 0xE420E420u;  // -(1024 + 32)
constexpr uint32_t H2_NEG96 = 0xD600D600u;    // -(64 + 32)

template <int DT> struct XTab;
template <> struct XTab<YUUKA_DTYPE_Q4_K> {
    static constexpr int SCL_STRIDE = 80, MN_STRIDE = 48, MN_OFF = 16 * SCL_STRIDE, D_OFF = MN_OFF + 16 * MN_STRIDE,
                         TAB = D_OFF + 16 * 8;
    static constexpr bool SUMS = true;
    static constexpr int XT_BYTES = 16;  // bytes of activations a lane reads per sub-block and step of t
};
template <> struct XTab<YUUKA_DTYPE_Q5_K> : XTab<YUUKA_DTYPE_Q4_K> {};
template <> struct XTab<YUUKA_DTYPE_Q6_K> {
    static constexpr int DS_STRIDE = 80, TAB = 16 * DS_STRIDE;
    static constexpr bool SUMS = false;
    static constexpr int XT_BYTES = 8;
};
template <> struct XTab<YUUKA_DTYPE_Q8_0> {
    static constexpr int DS_STRIDE = 48, TAB = 16 * DS_STRIDE;
    static constexpr bool SUMS = false;
    static constexpr int XT_BYTES = 16;
};

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)(bits & 0xffffu))); }

__device__ __forceinline__ void mma16816_zero(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Q4_K / Q5_K header: hdr.x = d | dmin << 16, hdr.y/z/w = 12 scale bytes (getScaleMinK4, tensor/quant.go:96-103).
// scl[row][pair j] = {sc_lo, -1024 sc_lo, sc_hi / 16, -64 sc_hi} (half2 each, integers); mn2[row][sub] = (m, m);
// dd[row] = (d, -dmin) in fp32.
template <typename X>
__device__ __forceinline__ void header_k4_exact(const uint4 & hdr, int lane, uint8_t * tab) {
    const int r = lane & 15, hf = lane >> 4;  // hf: pairs 2hf, 2hf+1
    const uint32_t w0 = hdr.y, w1 = hdr.z, w2 = hdr.w;
    const uint32_t sc4 = hf ? ((w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u)) : (w0 & 0x3f3f3f3fu);
    const uint32_t mn4 = hf ? (((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u)) : (w1 & 0x3f3f3f3fu);
    uint4 * scl = reinterpret_cast<uint4 *>(tab + r * X::SCL_STRIDE) + hf * 2;
    uint2 * mn2 = reinterpret_cast<uint2 *>(tab + X::MN_OFF + r * X::MN_STRIDE) + hf * 2;
#pragma unroll
    for (int jl = 0; jl < 2; jl++) {
        const uint32_t sp = h2_sub(jl ? bytes23_h2(sc4) : bytes01_h2(sc4), H2_1024);
        const uint32_t mp = h2_sub(jl ? bytes23_h2(mn4) : bytes01_h2(mn4), H2_1024);
        const uint32_t slo = dup_lo(sp), shi = dup_hi(sp);
        scl[jl] = make_uint4(slo, h2_mul(slo, H2_NEG1024), h2_mul(shi, H2_INV16), h2_mul(shi, H2_NEG64));
        mn2[jl] = make_uint2(dup_lo(mp), dup_hi(mp));
    }
    if (hf == 0) reinterpret_cast<float2 *>(tab + X::D_OFF)[r] = make_float2(f16_bits_to_f32(hdr.x), -f16_bits_to_f32(hdr.x >> 16));
}

// One MMA adding  sum_s16 A[row][s16] * xsum[tok][s16]  for eight 16-element groups base..base+7.
// a_* are the (value, value) pairs for groups base+t and base+t+4 of rows g and g+8. A column that stands for
// the lo half of an activation row takes no part (the sums already hold hi + lo).
template <int NT>
__device__ __forceinline__ void sum_mma(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, int t, int s16_base,
                                        const uint8_t * const (&xsrow)[NT], bool lo_col, float (&acc)[NT][4]) {
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const uint32_t * xs = reinterpret_cast<const uint32_t *>(xsrow[j]) + s16_base;
        const uint32_t b0 = lo_col ? 0u : xs[t], b1 = lo_col ? 0u : xs[t + 4];
        mma16816(acc[j], a0, a1, a2, a3, b0, b1);
    }
}

// Two fp32 fused multiply-adds in one instruction (sm_100 packed f32x2): (a0, a1) += s * (t0, t1).
__device__ __forceinline__ void fma2(float & a0, float & a1, float s, float t0, float t1) {
    unsigned long long a, t, ss;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(t) : "f"(t0), "f"(t1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(ss) : "f"(s));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a) : "l"(ss), "l"(t));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(a));
}

// acc[j][c] += dg * q[j][c] (rows g: c < 2) or dh * q[j][c] (rows g + 8)
template <int NT>
__device__ __forceinline__ void fold_rows(float (&acc)[NT][4], const float (&q)[NT][4], float dg, float dh) {
#pragma unroll
    for (int j = 0; j < NT; j++) {
        fma2(acc[j][0], acc[j][1], dg, q[j][0], q[j][1]);
        fma2(acc[j][2], acc[j][3], dh, q[j][2], q[j][3]);
    }
}

// - dmin * sum_sub m[sub] * sum(x[sub]) of one Q4_K / Q5_K superblock
template <typename X, int NT>
__device__ __forceinline__ void min_part(const uint8_t * tab, int g, int t, int sbl, const uint8_t * const (&xsrow)[NT], bool lo_col,
                                         float (&acc)[NT][4], float ndmin_g, float ndmin_h) {
    float mq[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int c = 0; c < 4; c++) mq[j][c] = 0.0f;
    const uint32_t * mg = reinterpret_cast<const uint32_t *>(tab + X::MN_OFF + g * X::MN_STRIDE);
    const uint32_t * mh = reinterpret_cast<const uint32_t *>(tab + X::MN_OFF + (g + 8) * X::MN_STRIDE);
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int k0 = 4 * half + (t >> 1);  // 16-element group 8 half + t belongs to sub-block 4 half + t / 2
        sum_mma<NT>(mg[k0], mh[k0], mg[k0 + 2], mh[k0 + 2], t, sbl * 16 + 8 * half, xsrow, lo_col, mq);
    }
    fold_rows<NT>(acc, mq, ndmin_g, ndmin_h);
}

template <int DT, int NT> struct XMma;

template <int NT> struct XMma<YUUKA_DTYPE_Q4_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q4_K>;
    using X = XTab<YUUKA_DTYPE_Q4_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4_exact<X>(r.hdr, lane, tab); }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], bool lo_col, int sbl, float (&acc)[NT][4],
                               const DecodeConsts & kc) {
        const int g = lane >> 2, t = lane & 3;
        const float2 dg = reinterpret_cast<const float2 *>(tab + X::D_OFF)[g], dh = reinterpret_cast<const float2 *>(tab + X::D_OFF)[g + 8];
        min_part<X, NT>(tab, g, t, sbl, xsrow, lo_col, acc, dg.y, dh.y);
        float q[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) q[j][c] = 0.0f;
        const uint8_t * tg = tab + g * X::SCL_STRIDE, * th = tab + (g + 8) * X::SCL_STRIDE;
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
            const uint32_t qg[4] = {r.q[jj].x, r.q[jj].y, r.q[jj].z, r.q[jj].w};
            const uint32_t qh[4] = {r.q[2 + jj].x, r.q[2 + jj].y, r.q[2 + jj].z, r.q[2 + jj].w};
#pragma unroll
            for (int jl = 0; jl < 2; jl++) {
                const int j = 2 * jj + jl;
                const uint4 sg = reinterpret_cast<const uint4 *>(tg)[j], sh = reinterpret_cast<const uint4 *>(th)[j];
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    const uint32_t mask = n ? kc.mf0 : kc.m0f;
                    const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
                    uint32_t a[2][4];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t vg = qg[2 * jl + h], vh = qh[2 * jl + h];
                        a[h][0] = h2_fma(and_or(vg, mask, kc.magic), s_g, c_g);
                        a[h][1] = h2_fma(and_or(vh, mask, kc.magic), s_h, c_h);
                        a[h][2] = h2_fma(and_or(vg >> 8, mask, kc.magic), s_g, c_g);
                        a[h][3] = h2_fma(and_or(vh >> 8, mask, kc.magic), s_h, c_h);
                    }
                    const int k = 2 * j + n;
#pragma unroll
                    for (int jt = 0; jt < NT; jt++) {
                        const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 256 + 32 * k) * 2);
                        mma16816(q[jt], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma16816(q[jt], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                    }
                }
            }
        }
        fold_rows<NT>(acc, q, dg.x, dh.x);
    }
};

template <int NT> struct XMma<YUUKA_DTYPE_Q5_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q5_K>;
    using X = XTab<YUUKA_DTYPE_Q5_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4_exact<X>(r.hdr, lane, tab); }
    template <int K>
    __device__ static void subblock(const typename C::Regs & r, const uint8_t * tg, const uint8_t * th,
                                    const uint8_t * const (&xrow)[NT], int sbl, float (&q)[NT][4], const DecodeConsts & kc) {
        constexpr int j = K >> 1, n = K & 1, jj = j >> 1, jl = j & 1;
        const uint32_t qg[4] = {r.q[jj].x, r.q[jj].y, r.q[jj].z, r.q[jj].w};
        const uint32_t qh[4] = {r.q[2 + jj].x, r.q[2 + jj].y, r.q[2 + jj].z, r.q[2 + jj].w};
        const uint32_t hg[2] = {r.qh.x, r.qh.y}, hh[2] = {r.qh.z, r.qh.w};
        const uint4 sg = reinterpret_cast<const uint4 *>(tg)[j], sh = reinterpret_cast<const uint4 *>(th)[j];
        const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
        uint32_t a[2][4];
#pragma unroll
        for (int h = 0; h < 2; h++)
            Mma<YUUKA_DTYPE_Q5_K, 1>::template sub<K>(qg[2 * jl + h], qh[2 * jl + h], hg[h], hh[h], s_g, c_g, s_h, c_h, a[h], kc);
#pragma unroll
        for (int jt = 0; jt < NT; jt++) {
            const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 256 + 32 * K) * 2);
            mma16816(q[jt], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
            mma16816(q[jt], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
        }
    }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], bool lo_col, int sbl, float (&acc)[NT][4],
                               const DecodeConsts & kc) {
        const int g = lane >> 2, t = lane & 3;
        const float2 dg = reinterpret_cast<const float2 *>(tab + X::D_OFF)[g], dh = reinterpret_cast<const float2 *>(tab + X::D_OFF)[g + 8];
        min_part<X, NT>(tab, g, t, sbl, xsrow, lo_col, acc, dg.y, dh.y);
        float q[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) q[j][c] = 0.0f;
        const uint8_t * tg = tab + g * X::SCL_STRIDE, * th = tab + (g + 8) * X::SCL_STRIDE;
        subblock<0>(r, tg, th, xrow, sbl, q, kc); subblock<1>(r, tg, th, xrow, sbl, q, kc);
        subblock<2>(r, tg, th, xrow, sbl, q, kc); subblock<3>(r, tg, th, xrow, sbl, q, kc);
        subblock<4>(r, tg, th, xrow, sbl, q, kc); subblock<5>(r, tg, th, xrow, sbl, q, kc);
        subblock<6>(r, tg, th, xrow, sbl, q, kc); subblock<7>(r, tg, th, xrow, sbl, q, kc);
        fold_rows<NT>(acc, q, dg.x, dh.x);
    }
};

// Q6_K: ds[row][s16] = d * sc[s16] in fp32 (tensor/quant.go:261-285).
template <int NT> struct XMma<YUUKA_DTYPE_Q6_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q6_K>;
    using X = XTab<YUUKA_DTYPE_Q6_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;  // hf: groups 8hf .. 8hf+7
        const float d = f16_bits_to_f32(r.d);
        const uint32_t wa = hf ? r.sc.z : r.sc.x, wb = hf ? r.sc.w : r.sc.y;
        float4 * ds = reinterpret_cast<float4 *>(tab + row * X::DS_STRIDE) + hf * 2;
        ds[0] = make_float4(d * (float)(int8_t)(wa & 0xff), d * (float)(int8_t)((wa >> 8) & 0xff), d * (float)(int8_t)((wa >> 16) & 0xff),
                            d * (float)(int8_t)(wa >> 24));
        ds[1] = make_float4(d * (float)(int8_t)(wb & 0xff), d * (float)(int8_t)((wb >> 8) & 0xff), d * (float)(int8_t)((wb >> 16) & 0xff),
                            d * (float)(int8_t)(wb >> 24));
    }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], bool lo_col, int sbl, float (&acc)[NT][4],
                               const DecodeConsts & kc) {
        (void)xsrow;
        (void)lo_col;
        const int g = lane >> 2;
        const float4 * dsg = reinterpret_cast<const float4 *>(tab + g * X::DS_STRIDE);
        const float4 * dsh = reinterpret_cast<const float4 *>(tab + (g + 8) * X::DS_STRIDE);
#pragma unroll
        for (int n6 = 0; n6 < 2; n6++) {
            const uint32_t lg[4] = {r.ql[n6].x, r.ql[n6].y, r.ql[n6].z, r.ql[n6].w};
            const uint32_t lh[4] = {r.ql[2 + n6].x, r.ql[2 + n6].y, r.ql[2 + n6].z, r.ql[2 + n6].w};
            const uint32_t hg[2] = {n6 ? r.qh[0].z : r.qh[0].x, n6 ? r.qh[0].w : r.qh[0].y};
            const uint32_t hh[2] = {n6 ? r.qh[1].z : r.qh[1].x, n6 ? r.qh[1].w : r.qh[1].y};
            // scales of the eight groups 8 n6 .. 8 n6 + 7 of rows g and g + 8
            const float4 sga = dsg[2 * n6], sgb = dsg[2 * n6 + 1], sha = dsh[2 * n6], shb = dsh[2 * n6 + 1];
            const float sgv[8] = {sga.x, sga.y, sga.z, sga.w, sgb.x, sgb.y, sgb.z, sgb.w};
            const float shv[8] = {sha.x, sha.y, sha.z, sha.w, shb.x, shb.y, shb.z, shb.w};
#pragma unroll
            for (int hsel = 0; hsel < 2; hsel++) {
                const int lsh = 4 - 2 * hsel, rsh = 4 + 2 * hsel;
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int k = 4 * n6 + hsel + 2 * nib;  // sub-block; its groups are 2k and 2k + 1
                    const uint32_t qm = nib ? kc.mf0 : kc.m0f, hm = nib ? kc.h8 : kc.h4;
                    const uint32_t one = nib ? H2_INV16 : H2_ONE, off = nib ? H2_NEG96 : H2_NEG1056;
                    uint32_t a[2][4];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t vg = lg[2 * hsel + h], vh = lh[2 * hsel + h];
                        a[h][0] = h2_fma(and_or(vg, qm, and_or(hg[h] << lsh, hm, kc.magic)), one, off);
                        a[h][1] = h2_fma(and_or(vh, qm, and_or(hh[h] << lsh, hm, kc.magic)), one, off);
                        a[h][2] = h2_fma(and_or(vg >> 8, qm, and_or(hg[h] >> rsh, hm, kc.magic)), one, off);
                        a[h][3] = h2_fma(and_or(vh >> 8, qm, and_or(hh[h] >> rsh, hm, kc.magic)), one, off);
                    }
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int gi = 2 * (hsel + 2 * nib) + h;  // group 2k + h, counted from 8 n6
                        const float s_g = sgv[gi], s_h = shv[gi];
#pragma unroll
                        for (int jt = 0; jt < NT; jt++) {
                            const uint2 b = *reinterpret_cast<const uint2 *>(xrow[jt] + (sbl * 256 + 32 * k + 16 * h) * 2);
                            float tmp[4];
                            mma16816_zero(tmp, a[h][0], a[h][1], a[h][2], a[h][3], b.x, b.y);
                            fma2(acc[jt][0], acc[jt][1], s_g, tmp[0], tmp[1]);
                            fma2(acc[jt][2], acc[jt][3], s_h, tmp[2], tmp[3]);
                        }
                    }
                }
            }
        }
    }
};

// Q8_0: ds[row][block] = d in fp32. Bytes are biased by 128 to make them unsigned, converted exactly
// (1024 + 128 + q) and the bias subtracted exactly.
template <int NT> struct XMma<YUUKA_DTYPE_Q8_0, NT> {
    using C = Codec<YUUKA_DTYPE_Q8_0>;
    using X = XTab<YUUKA_DTYPE_Q8_0>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;
        const uint32_t da = hf ? r.d.z : r.d.x, db = hf ? r.d.w : r.d.y;
        float4 * ds = reinterpret_cast<float4 *>(tab + row * X::DS_STRIDE) + hf;
        ds[0] = make_float4(f16_bits_to_f32(da), f16_bits_to_f32(da >> 16), f16_bits_to_f32(db), f16_bits_to_f32(db >> 16));
    }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], bool lo_col, int sbl, float (&acc)[NT][4],
                               const DecodeConsts & kc) {
        (void)xsrow;
        (void)lo_col;
        (void)kc;
        const int g = lane >> 2;
        const float4 * dsg = reinterpret_cast<const float4 *>(tab + g * X::DS_STRIDE);
        const float4 * dsh = reinterpret_cast<const float4 *>(tab + (g + 8) * X::DS_STRIDE);
        const float4 g0 = dsg[0], g1 = dsg[1], h0 = dsh[0], h1 = dsh[1];
        const float sgv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float shv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const uint32_t qg[4] = {r.q[kk].x, r.q[kk].y, r.q[kk].z, r.q[kk].w};
            const uint32_t qh[4] = {r.q[4 + kk].x, r.q[4 + kk].y, r.q[4 + kk].z, r.q[4 + kk].w};
#pragma unroll
            for (int kl = 0; kl < 2; kl++) {
                const int k = 2 * kk + kl;
                uint32_t a[2][4];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t vg = qg[2 * kl + h] ^ 0x80808080u, vh = qh[2 * kl + h] ^ 0x80808080u;
                    a[h][0] = h2_sub(bytes02_h2(vg), H2_1152);
                    a[h][1] = h2_sub(bytes02_h2(vh), H2_1152);
                    a[h][2] = h2_sub(bytes13_h2(vg), H2_1152);
                    a[h][3] = h2_sub(bytes13_h2(vh), H2_1152);
                }
#pragma unroll
                for (int jt = 0; jt < NT; jt++) {
                    const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 256 + 32 * k) * 2);
                    float tmp[4];
                    mma16816_zero(tmp, a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                    mma16816(tmp, a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                    fma2(acc[jt][0], acc[jt][1], sgv[k], tmp[0], tmp[1]);
                    fma2(acc[jt][2], acc[jt][3], shv[k], tmp[2], tmp[3]);
                }
            }
        }
    }
};

// ===========================================================================
// mma kernel

__device__ int g_gemm_wait_expired = 0;

}  // namespace yk
#include "gemm_umma.cuh"
namespace yk {

struct TParams {
    DecodeConsts kc;
    const uint8_t * w;
    int N, nsb;
    const __half * xh;      // prepared activations [M][nsb * 256], hi halves
    const __half * xl;      // lo halves
    const __half2 * xs16;   // [M][nsb * 16]
    const void * x;         // fp32 route only
    int64_t ldx;
    int M;
    float * out;
    int64_t ldo;
    int accumulate;
    int TG, KS;        // row tiles per group, warps per row tile (TG * KS == warps of the CTA)
    int kchunks;       // gridDim.y
    int nsb_chunk;     // superblocks per CTA-level K chunk
    int n_groups;
    float * partial;
    int * counters;
    // optional (GROUPED kernels): per-blockIdx.z row segments, byte stride between expert matrices,
    // and the source row of every activation row
    const GemmSegment * segments;
    size_t expert_stride;
    const int32_t * row_index;
    // optional, RMSNorm folded into the GEMMs on either side of it (see NormFuse in gemm_tiled.cuh):
    // as the producer of a residual row this launch also writes x * nf_w * pre in prepared form (both
    // halves and the 16-column sums) and adds each row's sum of squares to nf_sumsq; as the consumer of
    // such rows it multiplies its output rows by scale / pre. pre is the previous norm's scale of the row
    // (from *_prev), which keeps the unnormalised values near unit range.
    const float * nf_w;
    const unsigned long long * nf_prev;  // producer: sums of squares behind `pre` (null: pre = 1)
    unsigned long long * nf_sumsq;
    __half * nf_xh;
    __half * nf_xl;
    __half2 * nf_xs16;
    const unsigned long long * cs_now;   // consumer: sums of squares of its input rows
    const unsigned long long * cs_prev;  // (null: pre = 1)
    float nf_eps;
    int nf_cols;                         // row width the sums of squares run over
    // optional (FOLD kernels): the matrix holds ffn_gate and ffn_up interleaved by row tile (tile 2i: gate
    // rows 16i.., tile 2i+1: up rows 16i..). Instead of `out` the launch writes silu(gate) * up
    // (forwardFFN, model/qwen35/forward.go:295-315) in prepared form, [M][N / 2].
    __half * sw_xh;
    __half * sw_xl;
    __half2 * sw_xs16;
    // optional: the matrix the next GEMM of the step will stream; its first bytes are asked into L2
    // while this kernel drains and the small kernels in between run
    const uint8_t * next_w;
    uint32_t next_lines;  // 128-byte lines
    int drop_copies;      // test hook (YUUKA_GEMM_TEST_DROP_COPIES): the activation copies are never issued
};

// 1 / rms of a row from its fixed-point sum of squares (2^-24 units). rmsNorm (model/qwen35/forward.go:
// 460-470) takes 1 / sqrt in f64 and rounds to f32; here it is the f32 reciprocal square root (2 ulp), in
// single precision throughout because every lane of every epilogue evaluates it: the f64 form cost more
// than the kernels it replaced. Producer and consumer use this same function, so `pre` cancels exactly.
constexpr float NF_INV_UNIT = 1.0f / 16777216.0f;
__device__ __forceinline__ float nf_scale(unsigned long long sumsq, int cols, float eps) {
    const float mean = __fdividef((float)sumsq * NF_INV_UNIT, (float)cols);
    return rsqrtf(mean + eps);
}
__device__ __forceinline__ unsigned long long nf_fixed(float v) { return (unsigned long long)(v * 16777216.0f); }
// silu(g) * u with the expression of silu_mul_kernel (elementwise.cu), so both forms give the same bits
__device__ __forceinline__ float swiglu(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

// One value of a prepared row: both halves into q_hi / q_lo, returns hi + lo (what the sums add up).
__device__ __forceinline__ float prep_value(float v, __half & q_hi, __half & q_lo) {
    xprep_split(v, q_hi, q_lo);
    return __half2float(q_hi) + __half2float(q_lo);
}
__device__ __forceinline__ __half2 prep_sum(float gs) {
    const __half hi = __float2half_rn(gs);
    return __halves2half2(hi, __float2half_rn(gs - __half2float(hi)));
}

// Register-fed kernel: one CTA of MW warps per SM, at most MMA_ROWS activation rows per launch. Row m of
// the activations occupies two columns of the tensor-core product, 2m (hi half) and 2m + 1 (lo half), which
// land in the same lane's accumulator pair and are added before anything else happens to them.
// GROUPED: blockIdx.z walks a device-built list of row segments, each bound to one expert's matrix
// (qwen35moe expert FFNs). A segment's rows are contiguous in the prepared-activation and output
// arrays unless row_index redirects the activation rows.
// FOLD: the RMSNorm on either side of this GEMM is folded into its epilogue (TParams::nf_* / cs_*).
template <int DT, int NT, bool GROUPED, bool FOLD>
__global__ void __launch_bounds__(MW * 32, 1) gemm_tiled_mma_kernel(const TParams p) {
    using C = Codec<DT>;
    using X = XTab<DT>;
    using MM = XMma<DT, NT>;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t xbar;
    __shared__ int last_flag;
    // folded norm: per input row scale / pre (consumer) and pre (producer); per warp the norm weights
    // of its row tile, fetched at the top of each group so that the epilogue does not wait on memory
    __shared__ float cs_s[FOLD ? MMA_ROWS : 1], pre_s[FOLD ? MMA_ROWS : 1], nw_s[FOLD ? 2 * MW * 16 : 1];
    const uint8_t * wbase = p.w;
    const __half * xhp = p.xh;
    const __half * xlp = p.xl;
    const __half2 * xsp = p.xs16;
    float * outp = p.out;
    int Mrows = p.M;
    const int32_t * row_index = nullptr;
    if constexpr (GROUPED) {
        // the segment list is written by the kernel before this one: nothing can start ahead of the wait
        pdl_trigger();
        pdl_wait();
        const GemmSegment sg = p.segments[blockIdx.z];
        if (sg.count <= 0) return;  // the whole CTA: unused slot of the segment list
        wbase += (size_t)sg.expert * p.expert_stride;
        Mrows = sg.count;
        outp += (int64_t)sg.row0 * p.ldo;
        if (p.row_index) row_index = p.row_index + sg.row0;
        else {
            xhp += (size_t)sg.row0 * p.nsb * 256;
            xlp += (size_t)sg.row0 * p.nsb * 256;
            xsp += (size_t)sg.row0 * p.nsb * 16;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int c0 = blockIdx.y * p.nsb_chunk;
    const int c1 = min(p.nsb, c0 + p.nsb_chunk);
    const int cnt = c1 - c0;
    const int xstride = p.nsb_chunk * 512 + 64;       // bytes of one fp16 half of a row (+64: bank spread)
    const int xsum_stride = p.nsb_chunk * 64 + 16;    // bytes of 16-element sums per row
    uint8_t * xs = smem;                              // [2 * Mrows]: row 2m = hi half of m, row 2m + 1 = lo half
    uint8_t * xsum = xs + (size_t)2 * Mrows * xstride;
    uint8_t * tabs = xsum + (X::SUMS ? (((size_t)Mrows * xsum_stride + 127) / 128) * 128 : 0);
    float * red = reinterpret_cast<float *>(tabs + MW * X::TAB);

    const int tile_in_group = warp / p.KS, kpart = warp - tile_in_group * p.KS;
    const int sb0 = c0 + (cnt * kpart) / p.KS, sb1 = c0 + (cnt * (kpart + 1)) / p.KS;
    const int n_tiles = (p.N + 15) >> 4;
    const size_t rec_row = (size_t)p.nsb * C::REC;

    // Weights do not depend on the previous kernel: start the first loads, and pull the rest of the
    // first group's records towards L2, before waiting for the kernel that produces x.
    pdl_trigger();
    int grp = blockIdx.x;
    typename C::Regs cur, nxt;
    {
        const int rt = min(grp * p.TG + tile_in_group, n_tiles - 1);
        if (sb0 < sb1) C::load(wbase + rt * rec_row + (size_t)sb0 * C::REC, lane, cur);
        if (sb0 + 1 < sb1) prefetch_l2_range(wbase + rt * rec_row + (size_t)(sb0 + 1) * C::REC, (sb1 - sb0 - 1) * C::REC, lane);
    }
    // (the barrier the activation copies complete on: set up while the previous kernel still runs)
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&xbar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();

    // ---- activations of this K chunk: one bulk copy per row and half, and one for the sums where the type
    // has a "- min" term, every row's copies issued by its own lane of the first warp ----
    if (warp == 0 && !p.drop_copies) {
        const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&xbar);
        const uint32_t row_bytes_x = (uint32_t)cnt * 512, row_bytes_s = X::SUMS ? (uint32_t)cnt * 64 : 0u;
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((2u * row_bytes_x + row_bytes_s) * Mrows)
                         : "memory");
        __syncwarp();
        for (int m = lane; m < Mrows; m += 32) {
            const size_t mr = row_index ? (size_t)row_index[m] : (size_t)m;
            const __half * srch = xhp + (mr * p.nsb + c0) * 256;
            const __half * srcl = xlp + (mr * p.nsb + c0) * 256;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(xs + (size_t)(2 * m) * xstride)),
                         "l"(srch), "r"(row_bytes_x), "r"(bar)
                         : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(xs + (size_t)(2 * m + 1) * xstride)),
                         "l"(srcl), "r"(row_bytes_x), "r"(bar)
                         : "memory");
            if constexpr (X::SUMS) {
                const __half2 * srcs = xsp + (mr * p.nsb + c0) * 16;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 (uint32_t)__cvta_generic_to_shared(xsum + (size_t)m * xsum_stride)),
                             "l"(srcs), "r"(row_bytes_s), "r"(bar)
                             : "memory");
            }
        }
    }
    if constexpr (FOLD) {
        const int m = (int)threadIdx.x - 32;  // second warp: the first issues the copies
        if (m >= 0 && m < MMA_ROWS) {
            float cs = 1.0f, pre = 1.0f;
            if (m < Mrows) {
                if (p.cs_now)
                    cs = nf_scale(__ldcg(p.cs_now + m), p.nf_cols, p.nf_eps) /
                         (p.cs_prev ? nf_scale(__ldcg(p.cs_prev + m), p.nf_cols, p.nf_eps) : 1.0f);
                if (p.nf_prev) pre = nf_scale(__ldcg(p.nf_prev + m), p.nf_cols, p.nf_eps);
            }
            cs_s[m] = cs;
            pre_s[m] = pre;
        }
        __syncthreads();  // the row scales are read by every warp's epilogue
    }
    {
        // bounded wait for the copies; on expiry the error word is set and the results are garbage
        const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&xbar);
        uint32_t ok = 0;
        const uint32_t limit = p.drop_copies ? (1u << 8) : (1u << 22);
        for (uint32_t i = 0; i < limit && !ok; i++) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(bar)
                : "memory");
        }
        if (!ok) atomicExch(&g_gemm_wait_expired, 1);
    }

    uint8_t * tab = tabs + warp * X::TAB;
    // column 8j + g of the product: activation row (8j + g) / 2, hi half if g is even
    const bool lo_col = (g & 1) != 0;
    const uint8_t * xrow[NT];
    const uint8_t * xsrow[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int col = min(8 * j + g, 2 * Mrows - 1);
        xrow[j] = xs + (size_t)col * xstride + t * X::XT_BYTES;
        xsrow[j] = xsum + (size_t)(col >> 1) * xsum_stride;
    }

    const DecodeConsts kc = p.kc;
    for (; grp < p.n_groups; grp += gridDim.x) {
        const int rt = grp * p.TG + tile_in_group;
        const int rtc = min(rt, n_tiles - 1);
        const uint8_t * tile = wbase + rtc * rec_row;
        // (two copies by group parity: a warp may start its next group while others still run the split-K tail)
        float * nw = nw_s + (FOLD ? (((grp - (int)blockIdx.x) / (int)gridDim.x) & 1) * (MW * 16) : 0);
        if (FOLD && p.nf_w && lane < 16) nw[warp * 16 + lane] = rt * 16 + lane < p.N ? p.nf_w[rt * 16 + lane] : 0.0f;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[j][c] = 0.0f;
        // the rest of this warp's records: get them moving from DRAM to L2 now; the register
        // double buffer below then only has to cover the L2 latency
        if (grp != (int)blockIdx.x && sb0 + 1 < sb1)
            prefetch_l2_range(tile + (size_t)(sb0 + 1) * C::REC, (sb1 - sb0 - 1) * C::REC, lane);

        for (int sb = sb0; sb < sb1; sb++) {
            // prefetch the next record of this tile, or the first record of the next group's tile
            if (sb + 1 < sb1) {
                C::load(tile + (size_t)(sb + 1) * C::REC, lane, nxt);
            } else if (grp + (int)gridDim.x < p.n_groups) {
                const int rtn = min((grp + (int)gridDim.x) * p.TG + tile_in_group, n_tiles - 1);
                C::load(wbase + rtn * rec_row + (size_t)sb0 * C::REC, lane, nxt);
            }
            MM::header(cur, lane, tab);
            __syncwarp();
            MM::run(cur, lane, tab, xrow, xsrow, lo_col, sb - c0, acc, kc);
            __syncwarp();
            cur = nxt;
        }

        // hi + lo columns of each activation row: lane (g, t) now holds, for row 4j + t, the sums of weight
        // rows g (vg) and g + 8 (vh) of its tile
        float vg[NT], vh[NT];
#pragma unroll
        for (int j = 0; j < NT; j++) {
            vg[j] = acc[j][0] + acc[j][1];
            vh[j] = acc[j][2] + acc[j][3];
        }

        // ---- reduce the K parts of a row tile inside the CTA ----
        if (p.KS > 1) {
            float * mine = red + warp * (NT * 64);
#pragma unroll
            for (int j = 0; j < NT; j++) {
                mine[(2 * j) * 32 + lane] = vg[j];
                mine[(2 * j + 1) * 32 + lane] = vh[j];
            }
            __syncthreads();
            if (kpart == 0) {
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    float sg = vg[j], sh = vh[j];
                    for (int k = 1; k < p.KS; k++) {
                        sg += red[(warp + k) * (NT * 64) + (2 * j) * 32 + lane];
                        sh += red[(warp + k) * (NT * 64) + (2 * j + 1) * 32 + lane];
                    }
                    vg[j] = sg;
                    vh[j] = sh;
                }
            }
        }
        // ---- epilogue ----
        const bool sw_direct = FOLD && p.sw_xh != nullptr && p.kchunks == 1;
        if (sw_direct) {
            // the up tile's warp hands its sums to the gate tile's warp (KS warps earlier) through its own slot of red
            const bool is_up = (tile_in_group & 1) != 0;
            if (kpart == 0 && is_up) {
                float * mine = red + warp * (NT * 64);
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    mine[(2 * j) * 32 + lane] = vg[j];
                    mine[(2 * j + 1) * 32 + lane] = vh[j];
                }
            }
            __syncthreads();
            if (kpart == 0 && !is_up && rt < n_tiles) {
                const float * upv = red + (warp + p.KS) * (NT * 64);
                const int half_n = p.N >> 1, col0 = (rt >> 1) * 16;
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    const int tok = 4 * j + t;
                    const bool tok_ok = tok < Mrows;
                    const float cs = cs_s[tok & (MMA_ROWS - 1)];
                    __half g_hi, g_lo, h_hi, h_lo;
                    float gs = prep_value(swiglu(vg[j] * cs, upv[(2 * j) * 32 + lane] * cs), g_hi, g_lo) +
                               prep_value(swiglu(vh[j] * cs, upv[(2 * j + 1) * 32 + lane] * cs), h_hi, h_lo);
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
                    if (tok_ok) {
                        const size_t at = (size_t)tok * half_n + col0 + g;
                        p.sw_xh[at] = g_hi;
                        p.sw_xl[at] = g_lo;
                        p.sw_xh[at + 8] = h_hi;
                        p.sw_xl[at + 8] = h_lo;
                        if (g == 0) p.sw_xs16[(size_t)tok * (half_n >> 4) + (rt >> 1)] = prep_sum(gs);
                    }
                }
            }
            __syncthreads();  // red is reused by the next group
        } else if (kpart == 0 && rt < n_tiles) {
            const int n_g = rt * 16 + g, n_h = n_g + 8;
            float * base = p.kchunks == 1 ? outp : p.partial + (size_t)blockIdx.y * Mrows * p.N;
            const int64_t ld = p.kchunks == 1 ? p.ldo : p.N;
            const bool produce = FOLD && p.nf_w != nullptr && p.kchunks == 1;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const int tok = 4 * j + t;
                const bool tok_ok = tok < Mrows;
                const float cs = FOLD ? cs_s[tok & (MMA_ROWS - 1)] : 1.0f;
                float v[2] = {0.0f, 0.0f};  // final values of columns n_g, n_h (producer only)
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const int n = hh ? n_h : n_g;
                    const float a = hh ? vh[j] : vg[j];
                    if (tok_ok && n < p.N) {
                        float * dst = base + (int64_t)tok * ld + n;
                        if (p.kchunks == 1) {
                            v[hh] = p.accumulate ? *dst + a * cs : a * cs;
                            *dst = v[hh];
                        } else {
                            __stcg(dst, a);
                        }
                    }
                }
                if (produce) {
                    // this tile is one 16-column group of the row: x * w * pre in both halves, the group sum, the squares
                    const float pre = pre_s[tok & (MMA_ROWS - 1)];
                    __half g_hi, g_lo, h_hi, h_lo;
                    float gs = prep_value(v[0] * pre * nw[warp * 16 + g], g_hi, g_lo) + prep_value(v[1] * pre * nw[warp * 16 + g + 8], h_hi, h_lo);
                    float sq = v[0] * v[0] + v[1] * v[1];
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) {
                        gs += __shfl_xor_sync(0xffffffffu, gs, o);
                        sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    }
                    if (tok_ok) {
                        if (n_g < p.N) {
                            p.nf_xh[(size_t)tok * p.N + n_g] = g_hi;
                            p.nf_xl[(size_t)tok * p.N + n_g] = g_lo;
                        }
                        if (n_h < p.N) {
                            p.nf_xh[(size_t)tok * p.N + n_h] = h_hi;
                            p.nf_xl[(size_t)tok * p.N + n_h] = h_lo;
                        }
                        if (g == 0) {
                            p.nf_xs16[(size_t)tok * (p.N >> 4) + rt] = prep_sum(gs);
                            atomicAdd(&p.nf_sumsq[tok], nf_fixed(sq));
                        }
                    }
                }
            }
        }
        if (p.kchunks > 1) {
            // K is also split across CTAs: the last CTA to finish a group sums the chunks in order
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) last_flag = atomicAdd(&p.counters[grp], 1) == p.kchunks - 1;
            __syncthreads();
            if (last_flag) {
                __threadfence();
                const int row0 = grp * p.TG * 16, nrows = min(p.TG * 16, p.N - row0);
                // (with the norm folded in, N is a multiple of 16: a half warp holds one 16-column group of a row)
                const int padded = (FOLD && p.nf_w) ? ((Mrows * nrows + 31) & ~31) : Mrows * nrows;
                if (FOLD && p.sw_xh) {
                    // gate and up columns of the group, 16 by 16 (nrows is a multiple of 32: row tiles come in pairs)
                    const int half_rows = nrows >> 1, half_n = p.N >> 1, live_n = Mrows * half_rows;
                    for (int i = threadIdx.x; i < ((live_n + 31) & ~31); i += MW * 32) {
                        const bool live = i < live_n;
                        const int tok = live ? i / half_rows : 0, cl = live ? i - tok * half_rows : 0;
                        const int n = row0 + (cl >> 4) * 32 + (cl & 15);
                        float gsum = 0.0f, usum = 0.0f;
                        if (live)
                            for (int q = 0; q < p.kchunks; q++) {
                                const float * src = p.partial + ((size_t)q * Mrows + tok) * p.N + n;
                                gsum += __ldcg(src);
                                usum += __ldcg(src + 16);
                            }
                        const float cs = cs_s[tok & (MMA_ROWS - 1)];
                        __half q_hi, q_lo;
                        float gs = prep_value(live ? swiglu(gsum * cs, usum * cs) : 0.0f, q_hi, q_lo);
#pragma unroll
                        for (int o = 1; o < 16; o <<= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
                        if (live) {
                            const int col = (row0 >> 1) + cl;
                            p.sw_xh[(size_t)tok * half_n + col] = q_hi;
                            p.sw_xl[(size_t)tok * half_n + col] = q_lo;
                            if ((lane & 15) == 0) p.sw_xs16[(size_t)tok * (half_n >> 4) + (col >> 4)] = prep_sum(gs);
                        }
                    }
                } else
                for (int i = threadIdx.x; i < padded; i += MW * 32) {
                    const bool live = i < Mrows * nrows;
                    const int tok = live ? i / nrows : 0, n = row0 + (live ? i - tok * nrows : 0);
                    float s = 0.0f;
                    if (live)
                        for (int q = 0; q < p.kchunks; q++) s += __ldcg(p.partial + ((size_t)q * Mrows + tok) * p.N + n);
                    if (FOLD) s *= cs_s[tok & (MMA_ROWS - 1)];
                    float v = 0.0f;
                    if (live) {
                        float * dst = outp + (int64_t)tok * p.ldo + n;
                        v = p.accumulate ? *dst + s : s;
                        *dst = v;
                    }
                    if (FOLD && p.nf_w) {
                        const int nl = n - row0;  // row tile nl / 16 of the group belongs to warp (nl / 16) * KS
                        __half q_hi, q_lo;
                        float gs = prep_value(live ? v * pre_s[tok & (MMA_ROWS - 1)] * nw[(nl >> 4) * p.KS * 16 + (nl & 15)] : 0.0f, q_hi, q_lo);
                        float sq = v * v;
#pragma unroll
                        for (int o = 1; o < 16; o <<= 1) {
                            gs += __shfl_xor_sync(0xffffffffu, gs, o);
                            sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        }
                        if (live) {
                            p.nf_xh[(size_t)tok * p.N + n] = q_hi;
                            p.nf_xl[(size_t)tok * p.N + n] = q_lo;
                            if ((lane & 15) == 0) {
                                p.nf_xs16[(size_t)tok * (p.N >> 4) + (n >> 4)] = prep_sum(gs);
                                atomicAdd(&p.nf_sumsq[tok], nf_fixed(sq));
                            }
                        }
                    }
                }
                if (threadIdx.x == 0) p.counters[grp] = 0;
            }
        } else if (p.KS > 1 && !sw_direct) {
            __syncthreads();  // red is reused by the next group
        }
    }

    pdl_trigger_late();
    if (p.next_w) {
        const uint32_t first = ((blockIdx.y * gridDim.x + blockIdx.x) * (MW * 32) + threadIdx.x);
        const uint32_t step = gridDim.x * gridDim.y * (MW * 32);
        for (uint32_t line = first; line < p.next_lines; line += step) prefetch_l2(p.next_w + (size_t)line * 128);
    }
}

// ===========================================================================
// fp32 kernel over the tiled layout: reference decode arithmetic, CUDA cores.
// A warp owns a row tile over all of K; lane (g, t) accumulates rows g and g+8
// over its share of the columns; the four lanes of a row are summed by shuffles.

constexpr int F32_MT = 4;

// value of element b (0..7) of an 8-byte piece stored as two shuffled words
__device__ __forceinline__ uint32_t piece_byte(uint32_t w0, uint32_t w1, int b) {
    const uint32_t w = (b & 4) ? w1 : w0;
    const int e = b & 3, pos = (e & 1) * 2 + (e >> 1);  // element 0,1,2,3 -> byte 0,2,1,3
    return (w >> (8 * pos)) & 0xffu;
}

template <int DT, typename XT>
__global__ void __launch_bounds__(TW * 32) gemm_tiled_fp32_kernel(const TParams p) {
    pdl_entry();
    using C = Codec<DT>;
    extern __shared__ __align__(16) float xf32[];  // [M][K]
    const int K = p.nsb * 256;
    {
        const XT * X = reinterpret_cast<const XT *>(p.x);
        for (int i = threadIdx.x; i < p.M * K; i += blockDim.x) {
            const int m = i / K, k = i - m * K;
            xf32[i] = xf<XT>(X[(int64_t)m * p.ldx + k]);
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n_tiles = (p.N + 15) >> 4;
    __shared__ __align__(16) uint8_t hdrs[TW][16 * 32];
    for (int rt = blockIdx.x * TW + warp; rt < n_tiles; rt += gridDim.x * TW) {
        float ag[F32_MT], ah[F32_MT];
#pragma unroll
        for (int m = 0; m < F32_MT; m++) ag[m] = ah[m] = 0.0f;
        for (int sb = 0; sb < p.nsb; sb++) {
            typename C::Regs r;
            const uint8_t * rec = p.w + ((size_t)rt * p.nsb + sb) * C::REC;
            C::load(rec, lane, r);
            const float * xb = xf32 + sb * 256;
            // eight consecutive elements e..e+7 of rows g and g+8
            auto fma8 = [&](int e, const float (&wg)[8], const float (&wh)[8]) {
#pragma unroll
                for (int m = 0; m < F32_MT; m++) {
                    if (m < p.M) {
                        const float4 x0 = *reinterpret_cast<const float4 *>(xb + m * K + e);
                        const float4 x1 = *reinterpret_cast<const float4 *>(xb + m * K + e + 4);
                        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int b = 0; b < 8; b++) {
                            ag[m] = fmaf(xv[b], wg[b], ag[m]);
                            ah[m] = fmaf(xv[b], wh[b], ah[m]);
                        }
                    }
                }
            };
            __syncwarp();
            if constexpr (DT == YUUKA_DTYPE_Q4_K || DT == YUUKA_DTYPE_Q5_K) {
                if (lane < 16) *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 16) = r.hdr;
                __syncwarp();
                const uint8_t * hg = hdrs[warp] + g * 16, * hh = hdrs[warp] + (g + 8) * 16;
                const float dg = ld_f16(hg), mg = ld_f16(hg + 2), dh = ld_f16(hh), mh = ld_f16(hh + 2);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint4 Qg = r.q[j >> 1], Qh = r.q[2 + (j >> 1)];
                    const uint32_t g0 = (j & 1) ? Qg.z : Qg.x, g1 = (j & 1) ? Qg.w : Qg.y;
                    const uint32_t h0 = (j & 1) ? Qh.z : Qh.x, h1 = (j & 1) ? Qh.w : Qh.y;
#pragma unroll
                    for (int n = 0; n < 2; n++) {
                        const int k = 2 * j + n;
                        int sc, mn;
                        scale_min_k4(k, hg + 4, sc, mn);
                        const float d1g = dg * (float)sc, m1g = mg * (float)mn;
                        scale_min_k4(k, hh + 4, sc, mn);
                        const float d1h = dh * (float)sc, m1h = mh * (float)mn;
                        float wg[8], wh[8];
#pragma unroll
                        for (int b = 0; b < 8; b++) {
                            int vg = (piece_byte(g0, g1, b) >> (4 * n)) & 15, vh = (piece_byte(h0, h1, b) >> (4 * n)) & 15;
                            if constexpr (DT == YUUKA_DTYPE_Q5_K) {
                                vg += ((piece_byte(r.qh.x, r.qh.y, b) >> k) & 1) << 4;
                                vh += ((piece_byte(r.qh.z, r.qh.w, b) >> k) & 1) << 4;
                            }
                            wg[b] = d1g * (float)vg - m1g;
                            wh[b] = d1h * (float)vh - m1h;
                        }
                        fma8(32 * k + 8 * t, wg, wh);
                    }
                }
            } else if constexpr (DT == YUUKA_DTYPE_Q6_K) {
                if (lane < 16) {
                    *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 32) = r.sc;
                    *reinterpret_cast<uint32_t *>(hdrs[warp] + lane * 32 + 16) = r.d;
                }
                __syncwarp();
                const int8_t * scg = reinterpret_cast<const int8_t *>(hdrs[warp] + g * 32);
                const int8_t * sch = reinterpret_cast<const int8_t *>(hdrs[warp] + (g + 8) * 32);
                const float dg = ld_f16(hdrs[warp] + g * 32 + 16), dh = ld_f16(hdrs[warp] + (g + 8) * 32 + 16);
                // four consecutive elements e..e+3 of rows g and g+8 (a lane's elements sit in two runs of four, pos6)
                auto fma4 = [&](int e, const float * wg, const float * wh) {
#pragma unroll
                    for (int m = 0; m < F32_MT; m++) {
                        if (m < p.M) {
                            const float4 x0 = *reinterpret_cast<const float4 *>(xb + m * K + e);
                            const float xv[4] = {x0.x, x0.y, x0.z, x0.w};
#pragma unroll
                            for (int b = 0; b < 4; b++) {
                                ag[m] = fmaf(xv[b], wg[b], ag[m]);
                                ah[m] = fmaf(xv[b], wh[b], ah[m]);
                            }
                        }
                    }
                };
#pragma unroll
                for (int n6 = 0; n6 < 2; n6++) {
                    const uint4 Lg = r.ql[n6], Lh = r.ql[2 + n6];
                    const uint32_t Hg0 = n6 ? r.qh[0].z : r.qh[0].x, Hg1 = n6 ? r.qh[0].w : r.qh[0].y;
                    const uint32_t Hh0 = n6 ? r.qh[1].z : r.qh[1].x, Hh1 = n6 ? r.qh[1].w : r.qh[1].y;
#pragma unroll
                    for (int g4 = 0; g4 < 4; g4++) {
                        const int hsel = g4 & 1, nib = g4 >> 1, k = 4 * n6 + g4;
                        const uint32_t g0 = hsel ? Lg.z : Lg.x, g1 = hsel ? Lg.w : Lg.y;
                        const uint32_t h0 = hsel ? Lh.z : Lh.x, h1 = hsel ? Lh.w : Lh.y;
                        float wg[8], wh[8];
#pragma unroll
                        for (int b = 0; b < 8; b++) {
                            // elements 0..3 belong to the 16-element group 2k, elements 4..7 to group 2k + 1
                            const float sg = dg * (float)scg[2 * k + (b >> 2)], sh = dh * (float)sch[2 * k + (b >> 2)];
                            const int vg = ((piece_byte(g0, g1, b) >> (4 * nib)) & 15) | (((piece_byte(Hg0, Hg1, b) >> (2 * g4)) & 3) << 4);
                            const int vh = ((piece_byte(h0, h1, b) >> (4 * nib)) & 15) | (((piece_byte(Hh0, Hh1, b) >> (2 * g4)) & 3) << 4);
                            wg[b] = sg * (float)(vg - 32);
                            wh[b] = sh * (float)(vh - 32);
                        }
                        fma4(32 * k + 4 * t, wg, wh);
                        fma4(32 * k + 16 + 4 * t, wg + 4, wh + 4);
                    }
                }
            } else {  // Q8_0
                if (lane < 16) *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 16) = r.d;
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float dg = ld_f16(hdrs[warp] + g * 16 + 2 * k), dh = ld_f16(hdrs[warp] + (g + 8) * 16 + 2 * k);
                    const uint4 Qg = r.q[k >> 1], Qh = r.q[4 + (k >> 1)];
                    const uint32_t g0 = (k & 1) ? Qg.z : Qg.x, g1 = (k & 1) ? Qg.w : Qg.y;
                    const uint32_t h0 = (k & 1) ? Qh.z : Qh.x, h1 = (k & 1) ? Qh.w : Qh.y;
                    float wg[8], wh[8];
#pragma unroll
                    for (int b = 0; b < 8; b++) {
                        wg[b] = dg * (float)(int8_t)piece_byte(g0, g1, b);
                        wh[b] = dh * (float)(int8_t)piece_byte(h0, h1, b);
                    }
                    fma8(32 * k + 8 * t, wg, wh);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < F32_MT; m++) {
            float vg = ag[m], vh = ah[m];
            vg += __shfl_xor_sync(0xffffffffu, vg, 1); vg += __shfl_xor_sync(0xffffffffu, vg, 2);
            vh += __shfl_xor_sync(0xffffffffu, vh, 1); vh += __shfl_xor_sync(0xffffffffu, vh, 2);
            if (t == 0 && m < p.M) {
                const int n_g = rt * 16 + g, n_h = n_g + 8;
                if (n_g < p.N) { float * d = p.out + (int64_t)m * p.ldo + n_g; *d = p.accumulate ? *d + vg : vg; }
                if (n_h < p.N) { float * d = p.out + (int64_t)m * p.ldo + n_h; *d = p.accumulate ? *d + vh : vh; }
            }
        }
    }
}

// ===========================================================================
// host side

struct TPlan {
    int TG, KS, kchunks, nsb_chunk, n_groups, grid_x;
    size_t smem;
};

static int xtab_of(uint32_t dtype) {
    switch (dtype) {
    case YUUKA_DTYPE_Q6_K: return XTab<YUUKA_DTYPE_Q6_K>::TAB;
    case YUUKA_DTYPE_Q8_0: return XTab<YUUKA_DTYPE_Q8_0>::TAB;
    default: return XTab<YUUKA_DTYPE_Q4_K>::TAB;
    }
}
static bool xtab_sums(uint32_t dtype) { return dtype == YUUKA_DTYPE_Q4_K || dtype == YUUKA_DTYPE_Q5_K; }
static int mma_nt(int m) { return (2 * m + 7) / 8; }  // product columns: two per activation row, eight per MMA tile

// dynamic shared memory of the register-fed kernel: both halves of m activation rows, their 16-column sums
// (types with a "- min" term), one table per warp, and the exchange area of the K parts / SwiGLU pairs
static size_t mma_smem(uint32_t dtype, int m, int nsb_chunk, int ks, bool paired = false) {
    size_t x = (size_t)2 * m * (nsb_chunk * 512 + 64);
    size_t xsum = xtab_sums(dtype) ? (((size_t)m * (nsb_chunk * 64 + 16) + 127) / 128) * 128 : 0;
    size_t red = (ks > 1 || paired) ? (size_t)MW * mma_nt(m) * 64 * 4 : 0;
    return x + xsum + (size_t)MW * xtab_of(dtype) + red;
}

// How a matrix is cut into work for m (at most MMA_ROWS) activation rows: `kchunks` K chunks across CTAs and
// KS warps per row tile inside a CTA (the other MW / KS row tiles of a group run beside it). The pair that
// minimises waves x (records per warp + 0.7) + 1.5 per K chunk beyond the first, where a wave is one
// (group, chunk) on every SM, 0.7 of a record stands for the fixed cost of a group (table set-up, reduction,
// epilogue) and 1.5 for a chunk's share of the partial sums and their last-arrival sum (measured on the 4B
// step at 9 rows: 2.68 ms per step with 1.5, 2.76 ms with 0.3, which splits the 2560-column matrices three
// ways across CTAs); ties go to fewer parts. Chunks start at what shared memory forces (the activations of all rows, both halves, must fit).
// paired: row tiles 2i and 2i+1 must share a CTA (SwiGLU epilogue): at most MW / 2 warps per row tile.
static void plan_tiled(const yuuka_device * dev, uint32_t dtype, int m, int n_out, int n_in, TPlan & pl, bool paired = false) {
    const int nsb = n_in / 256, n_tiles = (n_out + 15) / 16;
    const int slots = dev->sm_count;  // one CTA per SM
    const size_t budget = dev->prop.sharedMemPerBlockOptin - 4096;  // (static shared memory of the kernel: under 3 KB)
    int kc_fit = 1;
    while ((nsb + kc_fit - 1) / kc_fit > 1 && mma_smem(dtype, m, (nsb + kc_fit - 1) / kc_fit, 2, paired) > budget) kc_fit++;
    int ks = 1, kchunks = kc_fit;
    double best = 1e30;
    for (int kc = kc_fit; kc <= nsb && kc <= kc_fit + 3; kc++) {
        const int nsb_c = (nsb + kc - 1) / kc, real_kc = (nsb + nsb_c - 1) / nsb_c;
        if (real_kc != kc && kc != kc_fit) continue;  // same cut as a smaller count
        for (int k = 1; k <= (paired ? MW / 2 : MW); k *= 2) {
            if (k > 1 && nsb_c < k) break;  // every warp keeps at least one record
            if (mma_smem(dtype, m, nsb_c, k, paired) > budget) continue;
            const int groups = (n_tiles + MW / k - 1) / (MW / k);
            const int waves = (groups * real_kc + slots - 1) / slots;
            const double cost = waves * ((nsb_c + k - 1) / k + 0.7) + (real_kc > 1 ? 1.5 * (real_kc - 1) : 0.0);
            if (cost < best - 1e-9) {
                best = cost;
                ks = k;
                kchunks = real_kc;
            }
        }
    }
    pl.KS = ks;
    pl.TG = MW / ks;
    pl.n_groups = (n_tiles + pl.TG - 1) / pl.TG;
    pl.nsb_chunk = (nsb + kchunks - 1) / kchunks;
    pl.kchunks = (nsb + pl.nsb_chunk - 1) / pl.nsb_chunk;
    pl.smem = mma_smem(dtype, m, pl.nsb_chunk, ks, paired);
    int per = slots / pl.kchunks;
    if (per < 1) per = 1;
    pl.grid_x = pl.n_groups < per ? pl.n_groups : per;
}

// Rows from which the tensor-memory route takes over from 16-row passes of the register-fed kernel.
constexpr int UMMA_MIN_ROWS = 48;
constexpr int UMMA_EARLY_ROWS = 33;  // on request: where three passes of the register-fed route would begin

static bool umma_enabled() {
    static const bool on = [] {
        const char * e = getenv("YUUKA_CUDA_NO_UMMA");
        return !(e && e[0] == '1');
    }();
    return on;
}

// K splits of the tensor-memory route: enough CTAs to fill the machine when the matrix has few
// 128-row blocks, at least two superblocks each. `separate` (may be null: then the in-kernel sum is the only
// choice) is set when the parts are summed by a kernel of their own.
static bool umma_specialised();
static int umma_ksplit(const yuuka_device * dev, int n_out, int n_in, int rows, bool * separate) {
    const int n_blocks = (n_out + UM_ROWS - 1) / UM_ROWS, nsb = n_in / 256;
    int ks = dev->sm_count / n_blocks;
    if (ks > nsb / 2) ks = nsb / 2;
    if (separate) *separate = false;
    static const bool no_separate = [] { const char * e = getenv("YUUKA_CUDA_UMMA_INLINE_SUM"); return e && e[0] == '1'; }();
    // The decode of a narrow matrix (20 blocks of a 2560-row one) is spread over the whole machine and the parts
    // are summed by every SM in a second launch; the output must allow 16-byte stores. Measured on 2560 x 9216
    // against the in-kernel sum below: 38 vs 53-62 us at 48-96 rows, 59 vs 192 us at 512.
    if (separate && !no_separate && ks > 2 && (n_out & 3) == 0 && umma_specialised()) {
        *separate = true;
        return ks < 8 ? ks : 8;
    }
    // the last CTA of a block sums the parts alone: measured on 2560-row matrices, four parts pay up to
    // about 96 activation rows and two beyond (the sum grows with rows x parts, the decode it hides does not)
    const int cap = rows <= 96 ? 4 : 2;
    if (ks > cap) ks = cap;
    return ks < 1 ? 1 : ks;
}

static bool umma_specialised() {
    static const bool on = [] { const char * e = getenv("YUUKA_CUDA_UMMA_WS"); return !(e && e[0] == '0'); }();
    return on;
}

// Activation rows of one tensor-memory launch. YUUKA_CUDA_UMMA_ROWS=256 keeps the warp-specialised kernel to one
// accumulator.
static int umma_rows_per_launch() {
    static const int rows = [] {
        const char * e = getenv("YUUKA_CUDA_UMMA_ROWS");
        const int want = e ? atoi(e) : UM_MAX_N2;
        return want > UM_MAX_N && umma_specialised() ? UM_MAX_N2 : UM_MAX_N;
    }();
    return rows;
}

void gemm_tiled_scratch_need(const yuuka_device * dev, uint32_t w_dtype, int rows, int n_out, int n_in,
                             uint64_t * partial_floats, int * counters) {
    *partial_floats = 0;
    *counters = 0;
    if (!tiled_supported(w_dtype, n_in)) return;
    if (rows >= UMMA_EARLY_ROWS) {
        const int per_launch = rows < umma_rows_per_launch() ? rows : umma_rows_per_launch();
        // enough for this row count and for every smaller one (fewer rows may split K further)
        int ks = 1, worst = 0;
        for (int m = UMMA_EARLY_ROWS; m <= per_launch; m += (m < UMMA_MIN_ROWS ? UMMA_MIN_ROWS - m : 16)) {
            bool sep;
            const int k = umma_ksplit(dev, n_out, n_in, m, &sep);
            if (k > ks) ks = k;
            if (k * m > worst) worst = k * m;
        }
        {
            bool sep;
            const int k = umma_ksplit(dev, n_out, n_in, per_launch, &sep);
            if (k > ks) ks = k;
            if (k * per_launch > worst) worst = k * per_launch;
        }
        if (ks > 1) {
            *partial_floats = (uint64_t)worst * n_out;
            *counters = (n_out + UM_ROWS - 1) / UM_ROWS;
        }
    }
    for (int m : {rows < MMA_ROWS ? rows : MMA_ROWS, MMA_ROWS < rows ? rows % MMA_ROWS : 0}) {
        if (m <= 0) continue;
        for (bool paired : {false, true}) {
            TPlan pl;
            plan_tiled(dev, w_dtype, m, n_out, n_in, pl, paired);
            if (pl.kchunks > 1) {
                uint64_t need = (uint64_t)pl.kchunks * m * n_out;
                if (need > *partial_floats) *partial_floats = need;
                if (pl.n_groups > *counters) *counters = pl.n_groups;
            }
        }
    }
}

template <int DT, int NT>
static void launch_mma_inst(cudaStream_t s, const TiledGemmArgs & a, const XPrepOut & xp, int m0, int m, const TPlan & pl) {
    const bool fold = a.norm.produce_w || a.norm.consume_now || a.swiglu.xh;
    auto kern = fold ? gemm_tiled_mma_kernel<DT, NT, false, true> : gemm_tiled_mma_kernel<DT, NT, false, false>;
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    TParams p{};
    p.kc = decode_consts(DT);
    p.w = a.w;
    p.N = a.n_out;
    p.nsb = a.n_in / 256;
    p.xh = xp.xh + (int64_t)m0 * a.n_in;
    p.xl = xp.xl + (int64_t)m0 * a.n_in;
    p.xs16 = xp.xs16 + (int64_t)m0 * (a.n_in / 16);
    p.M = m;
    p.out = a.out + (int64_t)m0 * a.ldo;
    p.ldo = a.ldo;
    p.accumulate = (a.flags & YUUKA_GEMM_ACCUMULATE) ? 1 : 0;
    p.TG = pl.TG;
    p.KS = pl.KS;
    p.kchunks = pl.kchunks;
    p.nsb_chunk = pl.nsb_chunk;
    p.n_groups = pl.n_groups;
    p.partial = a.scratch ? a.scratch->partial : nullptr;
    p.counters = a.scratch ? a.scratch->counters : nullptr;
    if (a.norm.produce_w || a.norm.consume_now) {
        // (per-row arrays of the folded norm start at this launch's first row)
        p.nf_w = a.norm.produce_w;
        p.nf_prev = a.norm.produce_prev ? a.norm.produce_prev + m0 : nullptr;
        p.nf_sumsq = a.norm.produce_sumsq ? a.norm.produce_sumsq + m0 : nullptr;
        if (a.norm.produce_prep.xh) {
            p.nf_xh = a.norm.produce_prep.xh + (int64_t)m0 * a.n_out;
            p.nf_xl = a.norm.produce_prep.xl + (int64_t)m0 * a.n_out;
            p.nf_xs16 = a.norm.produce_prep.xs16 + (int64_t)m0 * (a.n_out / 16);
        }
        p.cs_now = a.norm.consume_now ? a.norm.consume_now + m0 : nullptr;
        p.cs_prev = a.norm.consume_prev ? a.norm.consume_prev + m0 : nullptr;
        p.nf_eps = a.norm.eps;
        p.nf_cols = a.norm.cols;
    }
    if (a.swiglu.xh) {
        p.sw_xh = a.swiglu.xh + (int64_t)m0 * (a.n_out / 2);
        p.sw_xl = a.swiglu.xl + (int64_t)m0 * (a.n_out / 2);
        p.sw_xs16 = a.swiglu.xs16 + (int64_t)m0 * (a.n_out / 32);
        p.nf_eps = a.norm.eps;
        p.nf_cols = a.norm.cols;
    }
    p.drop_copies = (a.flags & YUUKA_GEMM_TEST_DROP_COPIES) ? 1 : 0;
    if (a.next_w && m0 + MMA_ROWS >= a.rows) {
        p.next_w = a.next_w;
        p.next_lines = (uint32_t)(a.next_bytes / 128);
    }
    dim3 grid(pl.grid_x, pl.kchunks);
    launch_k(kern, grid, MW * 32, pl.smem, s, p);
    YK_CUDA(cudaGetLastError());
}

template <int DT>
static void launch_grouped_dt(const yuuka_device * dev, cudaStream_t s, const GroupedGemmArgs & a) {
    const int nsb = a.n_in / 256, n_tiles = (a.n_out + 15) / 16;
    constexpr int NT = (2 * GEMM_SEGMENT_ROWS + 7) / 8;
    TPlan pl;
    pl.KS = 1;
    pl.TG = MW;
    pl.n_groups = (n_tiles + MW - 1) / MW;
    pl.kchunks = 1;
    pl.nsb_chunk = nsb;
    pl.smem = mma_smem(DT, GEMM_SEGMENT_ROWS, nsb, 1);
    // row groups per CTA: a CTA stages a segment's activation rows once and then walks that many groups
    // (enough CTAs to fill the SMs about twice when every slot of the segment list is in use)
    int per = (int)((int64_t)pl.n_groups * a.max_segments / (2 * dev->sm_count));
    if (per < 1) per = 1;
    if (per > pl.n_groups) per = pl.n_groups;
    pl.grid_x = (pl.n_groups + per - 1) / per;
    YK_REQUIRE(pl.smem + 4096 <= dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_UNSUPPORTED,
               "grouped gemm: %d columns of activations do not fit shared memory", a.n_in);
    auto kern = gemm_tiled_mma_kernel<DT, NT, true, false>;
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    TParams p{};
    p.kc = decode_consts(DT);
    p.w = a.w;
    p.N = a.n_out;
    p.nsb = nsb;
    p.xh = a.xprep.xh;
    p.xl = a.xprep.xl;
    p.xs16 = a.xprep.xs16;
    p.M = GEMM_SEGMENT_ROWS;
    p.out = a.out;
    p.ldo = a.ldo;
    p.TG = pl.TG;
    p.KS = pl.KS;
    p.kchunks = 1;
    p.nsb_chunk = nsb;
    p.n_groups = pl.n_groups;
    p.segments = a.segments;
    p.expert_stride = a.expert_stride;
    p.row_index = a.row_index;
    dim3 grid(pl.grid_x, 1, a.max_segments);
    launch_k(kern, grid, MW * 32, pl.smem, s, p);
    YK_CUDA(cudaGetLastError());
}

int launch_gemm_tiled_grouped(const yuuka_device * dev, cudaStream_t stream, const GroupedGemmArgs & a) {
    YK_REQUIRE(a.w && a.xprep.xh && a.xprep.xl && a.xprep.xs16 && a.out && a.segments, YUUKA_ERR_INVALID_ARGUMENT, "grouped gemm: null operand");
    YK_REQUIRE(a.n_out > 0 && a.n_in > 0 && a.max_segments > 0 && a.max_segments <= 65535, YUUKA_ERR_INVALID_ARGUMENT,
               "grouped gemm: invalid shape");
    YK_REQUIRE(tiled_supported(a.w_dtype, a.n_in), YUUKA_ERR_UNSUPPORTED, "grouped gemm: dtype %u / width %d has no tiled layout",
               a.w_dtype, a.n_in);
    YK_REQUIRE(a.ldo >= a.n_out, YUUKA_ERR_INVALID_ARGUMENT, "grouped gemm: leading dimension too small");
    set_device(dev);
    switch (a.w_dtype) {
    case YUUKA_DTYPE_Q4_K: launch_grouped_dt<YUUKA_DTYPE_Q4_K>(dev, stream, a); break;
    case YUUKA_DTYPE_Q5_K: launch_grouped_dt<YUUKA_DTYPE_Q5_K>(dev, stream, a); break;
    case YUUKA_DTYPE_Q6_K: launch_grouped_dt<YUUKA_DTYPE_Q6_K>(dev, stream, a); break;
    case YUUKA_DTYPE_Q8_0: launch_grouped_dt<YUUKA_DTYPE_Q8_0>(dev, stream, a); break;
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "grouped gemm: dtype %u has no tiled kernels", a.w_dtype);
    }
    return 1;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda)
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                      const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static const TensorMapEncodeFn fn = [] {
        const char * e = getenv("YUUKA_CUDA_NO_TMA");
        if (e && e[0] == '1') return (TensorMapEncodeFn) nullptr;
        void * f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (TensorMapEncodeFn) nullptr;
        }
        return (TensorMapEncodeFn)f;
    }();
    return fn;
}

// 2-D map over prepared activations [m][k] (fp16, row-major): boxes of 64 columns x npad rows, 128-byte swizzle.
static bool make_x_map(CUtensorMap * map, const __half * xh, int m, int k, int npad) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc || ((uintptr_t)xh & 15) != 0) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)m};
    const cuuint64_t gstride[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)UM_KC, (cuuint32_t)npad};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)xh, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DT>
static int launch_umma_dt(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a, const __half * xh) {
    int launches = 0;
    const int n_blocks = (a.n_out + UM_ROWS - 1) / UM_ROWS;
    // rows per launch: 512 (two accumulators) with tensor-map copies and the warp-specialised kernel, 256 with the
    // one-accumulator kernel; the padded cp.async stages are larger, so fewer fit
    const bool want_tma = tensor_map_encoder() != nullptr;
    const bool ws = want_tma && umma_specialised();
    int max_n = ws ? umma_rows_per_launch() : UM_MAX_N;
    while (!want_tma && max_n > 16 &&
           (size_t)(UM_STAGES - 1) * (UM_A_BYTES + (size_t)(max_n / 8) * UM_B_SBO) + (size_t)TW * Codec<DT>::TAB + 1024 >
               dev->prop.sharedMemPerBlockOptin)
        max_n -= 16;
    for (int m0 = 0; m0 < a.rows; m0 += max_n) {
        const int m = a.rows - m0 < max_n ? a.rows - m0 : max_n;
        bool separate = false;
        const int ksplit = umma_ksplit(dev, a.n_out, a.n_in, m, ws && (a.ldo & 3) == 0 && ((uintptr_t)a.out & 15) == 0 ? &separate : nullptr);
        UParams p{};
        p.kc = decode_consts(DT);
        p.w = a.w;
        p.N = a.n_out;
        p.nsb = a.n_in / 256;
        p.xh = xh + (int64_t)m0 * a.n_in;
        p.M = m;
        p.npad = (m + 15) / 16 * 16;
        p.out = a.out + (int64_t)m0 * a.ldo;
        p.ldo = a.ldo;
        p.accumulate = (a.flags & YUUKA_GEMM_ACCUMULATE) ? 1 : 0;
        p.tmem_cols = 32;
        while ((int)p.tmem_cols < p.npad) p.tmem_cols *= 2;
        // instruction descriptor: D f32, A and B f16, both K-major, N = rows of the accumulator, M = 128
        const int n1 = p.npad < UM_MAX_N ? p.npad : UM_MAX_N;
        p.idesc = (1u << 4) | ((uint32_t)(n1 >> 3) << 17) | ((uint32_t)(UM_ROWS >> 4) << 24);
        p.idesc2 = p.npad > UM_MAX_N ? (1u << 4) | ((uint32_t)((p.npad - UM_MAX_N) >> 3) << 17) | ((uint32_t)(UM_ROWS >> 4) << 24) : 0u;
        p.box_rows = (uint32_t)n1;
        if (ksplit > 1) {
            YK_REQUIRE(a.scratch && a.scratch->partial_floats >= (uint64_t)ksplit * m * a.n_out &&
                           a.scratch->counter_count >= n_blocks,
                       YUUKA_ERR_INTERNAL, "umma gemm: split-K scratch is too small");
            p.partial = a.scratch->partial;
            p.counters = separate ? nullptr : a.scratch->counters;
        }
        alignas(64) CUtensorMap xmap;
        memset(&xmap, 0, sizeof(xmap));
        const bool tma = want_tma && make_x_map(&xmap, p.xh, m, a.n_in, (int)p.box_rows);
        YK_REQUIRE(tma || !want_tma, YUUKA_ERR_INTERNAL, "umma gemm: the tensor map of the activations could not be encoded");
        const size_t b_bytes = tma ? (size_t)(p.idesc2 ? 2 : 1) * p.box_rows * 128 : (size_t)(p.npad / 8) * UM_B_SBO;
        p.stages = UM_STAGES;
        const size_t tab_bytes = (size_t)(ws ? UM_DW : TW) * Codec<DT>::TAB;
        size_t smem = (size_t)p.stages * (UM_A_BYTES + b_bytes) + tab_bytes + 1024;
        while (smem > dev->prop.sharedMemPerBlockOptin && p.stages > 2) {
            p.stages--;
            smem = (size_t)p.stages * (UM_A_BYTES + b_bytes) + tab_bytes + 1024;
        }
        YK_REQUIRE(smem <= dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_INTERNAL, "umma gemm: stage buffers do not fit shared memory");
        auto kern = ws ? gemm_umma_ws_kernel<DT> : (tma ? gemm_umma_kernel<DT, true> : gemm_umma_kernel<DT, false>);
        YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int per_split = dev->sm_count / ksplit > 0 ? dev->sm_count / ksplit : 1;
        dim3 grid(n_blocks < per_split ? n_blocks : per_split, ksplit);
        launch_k(kern, grid, ws ? UM_WS_THREADS : TW * 32, smem, s, p, xmap);
        YK_CUDA(cudaGetLastError());
        launches++;
        if (separate && ksplit > 1) {
            const int64_t quads = (int64_t)m * (a.n_out / 4);
            const int64_t want = (quads + 255) / 256, most = (int64_t)dev->sm_count * 8;
            launch_k(umma_reduce_kernel, (int)(want < most ? want : most), 256, 0, s, p.out, p.ldo, (const float *)p.partial, ksplit, m,
                     a.n_out, p.accumulate);
            YK_CUDA(cudaGetLastError());
            launches++;
        }
    }
    return launches;
}

template <int DT>
static int launch_mma_dt(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a) {
    int launches = 0;
    XPrepOut xp = a.xprep;
    if (!xp.xh) {
        // activations arrive as f32 / bf16: convert once into the scratch
        YK_REQUIRE(a.x && a.scratch && a.scratch->xh && a.scratch->xl && a.scratch->xh_elems >= (uint64_t)a.rows * a.n_in,
                   YUUKA_ERR_INTERNAL, "gemm: no prepared activations and no scratch to prepare them in");
        if (a.x_dtype == YUUKA_DTYPE_F32)
            launch_xprep<float>(s, a.scratch->xh, a.scratch->xl, a.scratch->xs16, (const float *)a.x, a.ldx, a.n_in, a.rows);
        else
            launch_xprep<__nv_bfloat16>(s, a.scratch->xh, a.scratch->xl, a.scratch->xs16, (const __nv_bfloat16 *)a.x, a.ldx, a.n_in, a.rows);
        xp.xh = a.scratch->xh;
        xp.xl = a.scratch->xl;
        xp.xs16 = a.scratch->xs16;
        launches++;
    }
    if (a.rows >= (a.wide_from_33 ? UMMA_EARLY_ROWS : UMMA_MIN_ROWS) && umma_enabled() && !a.exact_only)
        return launches + launch_umma_dt<DT>(dev, s, a, xp.xh);
    YK_REQUIRE(xp.xl && xp.xs16, YUUKA_ERR_INTERNAL, "gemm: the prepared activations lack their lo halves or sums");
    for (int m0 = 0; m0 < a.rows; m0 += MMA_ROWS) {
        const int m = a.rows - m0 < MMA_ROWS ? a.rows - m0 : MMA_ROWS;
        TPlan pl;
        plan_tiled(dev, a.w_dtype, m, a.n_out, a.n_in, pl, a.swiglu.xh != nullptr);
        YK_REQUIRE(pl.smem + 4096 <= dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_UNSUPPORTED,
                   "gemm: activations of %d rows x %d columns do not fit shared memory", m, a.n_in);
        if (pl.kchunks > 1)
            YK_REQUIRE(a.scratch && a.scratch->partial_floats >= (uint64_t)pl.kchunks * m * a.n_out &&
                           a.scratch->counter_count >= pl.n_groups,
                       YUUKA_ERR_INTERNAL, "gemm: split-K scratch is too small");
        switch (mma_nt(m)) {
        case 1: launch_mma_inst<DT, 1>(s, a, xp, m0, m, pl); break;
        case 2: launch_mma_inst<DT, 2>(s, a, xp, m0, m, pl); break;
        case 3: launch_mma_inst<DT, 3>(s, a, xp, m0, m, pl); break;
        default: launch_mma_inst<DT, 4>(s, a, xp, m0, m, pl); break;
        }
        launches++;
    }
    return launches;
}

template <int DT, typename XT>
static int launch_fp32_dt(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a) {
    auto kern = gemm_tiled_fp32_kernel<DT, XT>;
    size_t smem_max = (size_t)F32_MT * a.n_in * sizeof(float);
    YK_REQUIRE(smem_max + 8192 <= dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_UNSUPPORTED,
               "gemm fp32 route: n_in %d does not fit shared memory", a.n_in);
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
    const int n_tiles = (a.n_out + 15) / 16;
    int grid = (n_tiles + TW - 1) / TW;
    if (grid > 4 * dev->sm_count) grid = 4 * dev->sm_count;
    int launches = 0;
    for (int m0 = 0; m0 < a.rows; m0 += F32_MT) {
        const int m = a.rows - m0 < F32_MT ? a.rows - m0 : F32_MT;
        TParams p{};
        p.w = a.w;
        p.N = a.n_out;
        p.nsb = a.n_in / 256;
        p.x = (const XT *)a.x + (int64_t)m0 * a.ldx;
        p.ldx = a.ldx;
        p.M = m;
        p.out = a.out + (int64_t)m0 * a.ldo;
        p.ldo = a.ldo;
        p.accumulate = (a.flags & YUUKA_GEMM_ACCUMULATE) ? 1 : 0;
        launch_k(kern, grid, TW * 32, (size_t)m * a.n_in * sizeof(float), s, p);
        YK_CUDA(cudaGetLastError());
        launches++;
    }
    return launches;
}

template <int DT>
static int launch_tiled_dt(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a, bool mma) {
    if (mma) return launch_mma_dt<DT>(dev, s, a);
    YK_REQUIRE(a.x, YUUKA_ERR_INVALID_ARGUMENT, "gemm fp32 route: needs the f32 / bf16 activations");
    return a.x_dtype == YUUKA_DTYPE_F32 ? launch_fp32_dt<DT, float>(dev, s, a) : launch_fp32_dt<DT, __nv_bfloat16>(dev, s, a);
}

int launch_gemm_tiled(const yuuka_device * dev, cudaStream_t stream, const TiledGemmArgs & a) {
    YK_REQUIRE(a.w && (a.x || a.xprep.xh) && a.out, YUUKA_ERR_INVALID_ARGUMENT, "gemm: null operand");
    YK_REQUIRE(a.rows > 0 && a.n_out > 0 && a.n_in > 0, YUUKA_ERR_INVALID_ARGUMENT, "gemm: invalid shape");
    if (a.swiglu.xh) {
        YK_REQUIRE(a.swiglu.xs16 && a.n_out % 32 == 0 && !(a.flags & YUUKA_GEMM_ACCUMULATE) && !a.norm.produce_w,
                   YUUKA_ERR_INVALID_ARGUMENT, "gemm: the SwiGLU epilogue needs gate and up tiles in pairs and a plain output");
        YK_REQUIRE(!a.norm.consume_now || a.norm.cols > 0, YUUKA_ERR_INVALID_ARGUMENT, "gemm: the folded RMSNorm needs the row width");
    }
    if (a.norm.produce_w || a.norm.consume_now || a.swiglu.xh) {
        const uint32_t route = a.path == YUUKA_GEMM_PATH_AUTO ? YUUKA_GEMM_PATH_MMA : a.path;
        YK_REQUIRE(route == YUUKA_GEMM_PATH_MMA && a.rows <= 32 && (a.rows < UMMA_MIN_ROWS || !umma_enabled()) &&
                       (!a.swiglu.xh || a.swiglu.xl) && (!a.norm.produce_w || a.norm.produce_prep.xl),
                   YUUKA_ERR_INTERNAL, "gemm: folded epilogues (RMSNorm, SwiGLU) run on the register-fed mma route only (1..32 rows)");
        YK_REQUIRE(!a.norm.produce_w || (a.n_out % 16 == 0 && a.norm.produce_sumsq && a.norm.produce_prep.xh && a.norm.produce_prep.xs16),
                   YUUKA_ERR_INVALID_ARGUMENT, "gemm: the folded RMSNorm needs a width that is a multiple of 16 and its outputs");
        YK_REQUIRE(a.swiglu.xh || a.norm.cols > 0, YUUKA_ERR_INVALID_ARGUMENT, "gemm: the folded RMSNorm needs the row width");
    }
    YK_REQUIRE(tiled_supported(a.w_dtype, a.n_in), YUUKA_ERR_UNSUPPORTED, "gemm: dtype %u / width %d has no tiled layout",
               a.w_dtype, a.n_in);
    YK_REQUIRE(a.x_dtype == YUUKA_DTYPE_F32 || a.x_dtype == YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
               "gemm: activation dtype %u is not F32 or BF16", a.x_dtype);
    YK_REQUIRE((!a.x || a.ldx >= a.n_in) && a.ldo >= a.n_out, YUUKA_ERR_INVALID_ARGUMENT, "gemm: leading dimension too small");
    uint32_t path = a.path == YUUKA_GEMM_PATH_AUTO ? YUUKA_GEMM_PATH_MMA : a.path;
    YK_REQUIRE(path == YUUKA_GEMM_PATH_FP32 || path == YUUKA_GEMM_PATH_MMA, YUUKA_ERR_INVALID_ARGUMENT,
               "gemm: unknown path %u", path);
    set_device(dev);
    const bool mma = path == YUUKA_GEMM_PATH_MMA;
    switch (a.w_dtype) {
    case YUUKA_DTYPE_Q4_K: return launch_tiled_dt<YUUKA_DTYPE_Q4_K>(dev, stream, a, mma);
    case YUUKA_DTYPE_Q5_K: return launch_tiled_dt<YUUKA_DTYPE_Q5_K>(dev, stream, a, mma);
    case YUUKA_DTYPE_Q6_K: return launch_tiled_dt<YUUKA_DTYPE_Q6_K>(dev, stream, a, mma);
    case YUUKA_DTYPE_Q8_0: return launch_tiled_dt<YUUKA_DTYPE_Q8_0>(dev, stream, a, mma);
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "gemm: dtype %u has no tiled kernels", a.w_dtype);
    }
    return 0;
}

// Loads the code of every kernel launch_gemm_tiled can choose. With CUDA's lazy module loading the first
// launch of a kernel makes the driver place its code in device memory; asking for the attributes does the
// same ahead of time, so that a caller who must not allocate later (yuuka_gemm_quant_static) pays here.
template <int DT>
static void preload_dt() {
    cudaFuncAttributes fa;
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_mma_kernel<DT, 1, false, false>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_mma_kernel<DT, 2, false, false>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_mma_kernel<DT, 3, false, false>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_mma_kernel<DT, 4, false, false>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_fp32_kernel<DT, float>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_tiled_fp32_kernel<DT, __nv_bfloat16>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_umma_ws_kernel<DT>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_umma_kernel<DT, true>));
    YK_CUDA(cudaFuncGetAttributes(&fa, gemm_umma_kernel<DT, false>));
}
void gemm_tiled_preload_kernels() {
    cudaFuncAttributes fa;
    preload_dt<YUUKA_DTYPE_Q4_K>();
    preload_dt<YUUKA_DTYPE_Q5_K>();
    preload_dt<YUUKA_DTYPE_Q6_K>();
    preload_dt<YUUKA_DTYPE_Q8_0>();
    YK_CUDA(cudaFuncGetAttributes(&fa, xprep_kernel<float>));
    YK_CUDA(cudaFuncGetAttributes(&fa, xprep_kernel<__nv_bfloat16>));
    YK_CUDA(cudaFuncGetAttributes(&fa, umma_reduce_kernel));
    tensor_map_encoder();  // the driver entry point look-up happens once, here
}

int read_gemm_wait_expired() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_wait_expired, sizeof(int));
    return v;
}
void clear_gemm_wait_expired() {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_wait_expired, &zero, sizeof(int));
}
void enqueue_gemm_wait_expired_read(cudaStream_t stream, int * out) {
    YK_CUDA(cudaMemcpyFromSymbolAsync(out, g_gemm_wait_expired, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
}

}  // namespace yk
