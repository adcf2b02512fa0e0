// Quantized GEMM over tile-ordered weights (see gemm_tiled.cuh for the layout):
//   out[m][n] = sum_k x[m][k] * W[n][k]
// Replaces, for the verify step, kernels/hip/gemm/lm_head.hip,
// gemv/gemv_quant.hip:317 and the small-row use of gemm/wmma_gemm.hip.
//
// mma route. A warp owns a 16-row tile and a range of superblocks. Per
// superblock it issues coalesced 16-byte-per-lane loads of the next record
// (register double buffer), decodes the current record's block headers into a
// per-warp scale table, and turns packed weights into fp16 directly in
// mma.sync.m16n8k16 A-fragment registers: one LOP3 places a nibble in the
// mantissa of 1024.0 and one fma.f16x2 with (s, -1024 s) yields s*q. The
// "- min" of Q4_K/Q5_K (and the -32 / -128 offsets of Q6_K / Q8_0) is not
// applied per weight: it is one more MMA per superblock against per-sub-block
// sums of the activations. Activations are staged once per CTA as fp16 in the
// k-order the fragments use. Warps of a CTA that share a row tile split K and
// are summed through shared memory in a fixed order; a split of K across CTAs
// (long rows) goes through a scratch buffer and is finished by the last CTA to
// arrive, also in a fixed order. Nothing here waits on another CTA.
//
// fp32 route (1-2 rows, tight-tolerance checks): same loads, the reference's
// own fp32 decode (tensor/quant.go:105-125,261-285), CUDA-core FMAs.
#include "gemm_tiled.cuh"
#include "quant.cuh"

namespace yk {

constexpr int TW = 8;            // warps per CTA
constexpr uint32_t H2_1024 = 0x64006400u;

__device__ __forceinline__ uint4 ldg_stream(const uint4 * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
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

// ===========================================================================
// Record layouts. map(p) gives, for byte p of a record, the source row (0..15)
// and the byte offset inside that row's superblock.

template <int DT> struct Codec;

// weight slot q = i*32 + lane: row g + 8*(i / per_half), 16-byte chunk t + 4*(i % per_half)
__device__ __forceinline__ void slot_row_chunk(int q, int per_half, int & r, int & c) {
    int i = q >> 5, lane = q & 31;
    r = (lane >> 2) + 8 * (i / per_half);
    c = (lane & 3) + 4 * (i % per_half);
}

template <> struct Codec<YUUKA_DTYPE_Q4_K> {
    static constexpr int SB = 144, REC = 16 * SB, NSUB = 8, TAB = 1024 + 512;
    struct Regs { uint4 q[4]; uint4 hdr; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) { int c; slot_row_chunk(p >> 4, 2, r, c); o = 16 + 16 * c + (p & 15); }
        else { r = (p - 2048) >> 4; o = p & 15; }
    }
    // element of the superblock that MMA (cc, n, w), lane t, slot s carries
    __device__ static int pair_slot(int e8, int & t) {  // e8: element / 8 within the superblock
        int e = e8 * 8, j = e >> 6, n = (e >> 5) & 1, tl = (e >> 4) & 1, wp = (e >> 3) & 1;
        t = 2 * (j & 1) + tl;
        return (j >> 1) * 4 + n * 2 + wp;
    }
    __device__ static int sub_of(int e) { return e >> 5; }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = ldg_stream(p + i * 32 + lane);
        r.hdr = ldg_stream(p + 128 + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q5_K> {
    static constexpr int SB = 176, REC = 16 * SB, NSUB = 8, TAB = 1024 + 512;
    struct Regs { uint4 q[4]; uint4 qh[2]; uint4 hdr; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) { int c; slot_row_chunk(p >> 4, 2, r, c); o = 48 + 16 * c + (p & 15); }
        else if (p < 2560) { r = (p - 2048) >> 5; o = 16 + ((p - 2048) & 31); }
        else { r = (p - 2560) >> 4; o = p & 15; }
    }
    __device__ static int pair_slot(int e8, int & t) { return Codec<YUUKA_DTYPE_Q4_K>::pair_slot(e8, t); }
    __device__ static int sub_of(int e) { return e >> 5; }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = ldg_stream(p + i * 32 + lane);
        r.qh[0] = ldg_stream(p + 128 + g * 2 + (t & 1));
        r.qh[1] = ldg_stream(p + 128 + (g + 8) * 2 + (t & 1));
        r.hdr = ldg_stream(p + 160 + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q6_K> {
    static constexpr int SB = 210, REC = 16 * SB, NSUB = 16, TAB = 2048 + 1024;
    struct Regs { uint4 ql[4]; uint4 qh[4]; uint4 sc; uint32_t d; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 2048) { int c; slot_row_chunk(p >> 4, 2, r, c); o = 16 * c + (p & 15); }
        else if (p < 3072) {
            int idx = (p - 2048) >> 4, h2 = idx & 1, g = (idx >> 1) & 7, i = idx >> 4;
            r = g + 8 * (i >> 1);
            o = 128 + 32 * (i & 1) + 16 * h2 + (p & 15);
        } else if (p < 3328) { r = (p - 3072) >> 4; o = 192 + (p & 15); }
        else { r = (p - 3328) >> 1; o = 208 + (p & 1); }
    }
    __device__ static int pair_slot(int e8, int & t) {
        int e = e8 * 8, cc = e >> 7, g4 = (e >> 5) & 3, tl = (e >> 4) & 1, wp = (e >> 3) & 1;
        t = 2 * (g4 & 1) + tl;
        return cc * 4 + (g4 >> 1) * 2 + wp;
    }
    __device__ static int sub_of(int e) { return e >> 4; }
    __device__ static void load(const uint8_t * rec, int lane, Regs & r) {
        const uint4 * p = reinterpret_cast<const uint4 *>(rec);
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; i++) r.ql[i] = ldg_stream(p + i * 32 + lane);
#pragma unroll
        for (int i = 0; i < 4; i++) r.qh[i] = ldg_stream(p + 128 + (i * 8 + g) * 2 + (t & 1));
        r.sc = ldg_stream(p + 192 + (lane & 15));
        r.d = __ldg(reinterpret_cast<const uint16_t *>(rec + 3328) + (lane & 15));
    }
};

template <> struct Codec<YUUKA_DTYPE_Q8_0> {
    static constexpr int SB = 272, REC = 16 * SB, NSUB = 8, TAB = 1024 + 512;
    struct Regs { uint4 q[8]; uint4 d; };
    __device__ static void map(int p, int & r, int & o) {
        if (p < 4096) {
            int c; slot_row_chunk(p >> 4, 4, r, c);
            o = 34 * (c >> 1) + 2 + 16 * (c & 1) + (p & 15);
        } else { r = (p - 4096) >> 4; int k = (p & 15) >> 1; o = 34 * k + (p & 1); }
    }
    __device__ static int pair_slot(int e8, int & t) {
        int e = e8 * 8, b = e >> 5, tl = (e >> 4) & 1, wp = (e >> 3) & 1;
        t = 2 * (b & 1) + tl;
        return (b >> 1) * 2 + wp;
    }
    __device__ static int sub_of(int e) { return e >> 5; }
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
// header decode -> per-warp tables, and the per-superblock MMA sequence

// Q4_K / Q5_K header word layout: hdr.x = d | dmin << 16, hdr.y/z/w = 12 scale bytes.
// Table: scl[row][pair j] = {s_lo, -1024 s_lo, s_hi/16, -64 s_hi} (half2 each, 16 B), mn2[row][sub] = (-min, -min).
__device__ __forceinline__ void header_k4(const uint4 & hdr, int lane, uint8_t * tab) {
    const int r = lane & 15, hf = lane >> 4;  // hf: pairs 2hf, 2hf+1
    const uint32_t d2 = dup_lo(hdr.x), dm2 = dup_hi(hdr.x);
    const uint32_t w0 = hdr.y, w1 = hdr.z, w2 = hdr.w;
    const uint32_t sc4 = hf ? ((w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u)) : (w0 & 0x3f3f3f3fu);
    const uint32_t mn4 = hf ? (((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u)) : (w1 & 0x3f3f3f3fu);
    uint4 * scl = reinterpret_cast<uint4 *>(tab) + r * 4 + hf * 2;
    uint2 * mn2 = reinterpret_cast<uint2 *>(tab + 1024) + r * 4 + hf * 2;
#pragma unroll
    for (int jl = 0; jl < 2; jl++) {
        const uint32_t sp = h2_mul(h2_sub(jl ? bytes23_h2(sc4) : bytes01_h2(sc4), H2_1024), d2);
        const uint32_t mp = h2_mul(h2_sub(jl ? bytes23_h2(mn4) : bytes01_h2(mn4), H2_1024), dm2);
        const uint32_t slo = dup_lo(sp), shi = dup_hi(sp);
        scl[jl] = make_uint4(slo, h2_mul(slo, H2_NEG1024), h2_mul(shi, H2_INV16), h2_mul(shi, H2_NEG64));
        mn2[jl] = make_uint2(h2_mul(dup_lo(mp), H2_NEG1), h2_mul(dup_hi(mp), H2_NEG1));
    }
}

template <int NT>
__device__ __forceinline__ void min_mma(const uint8_t * mn2, int stride_subs, int g, int t, int sub0,
                                        const uint8_t * const (&xsrow)[NT], int xs_off, float (&acc)[NT][4]) {
    const uint32_t * m = reinterpret_cast<const uint32_t *>(mn2);
    const uint32_t a0 = m[g * stride_subs + sub0 + t], a1 = m[(g + 8) * stride_subs + sub0 + t];
    const uint32_t a2 = m[g * stride_subs + sub0 + t + 4], a3 = m[(g + 8) * stride_subs + sub0 + t + 4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const uint32_t * xs = reinterpret_cast<const uint32_t *>(xsrow[j]) + xs_off + sub0;
        mma16816(acc[j], a0, a1, a2, a3, xs[t], xs[t + 4]);
    }
}

template <int DT, int NT> struct Mma;

template <int NT> struct Mma<YUUKA_DTYPE_Q4_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q4_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4(r.hdr, lane, tab); }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], int sbl, float (&acc)[NT][4]) {
        const int g = lane >> 2, t = lane & 3;
        const uint4 * scl = reinterpret_cast<const uint4 *>(tab);
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
            const int j = (t >> 1) + 2 * cc;
            const uint4 sg = scl[g * 4 + j], sh = scl[(g + 8) * 4 + j];
            const uint32_t qg[4] = {r.q[cc].x, r.q[cc].y, r.q[cc].z, r.q[cc].w};
            const uint32_t qh[4] = {r.q[2 + cc].x, r.q[2 + cc].y, r.q[2 + cc].z, r.q[2 + cc].w};
#pragma unroll
            for (int n = 0; n < 2; n++) {
                const uint32_t mask = n ? 0x00f000f0u : 0x000f000fu;
                const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
#pragma unroll
                for (int wp = 0; wp < 2; wp++) {
                    uint32_t a[2][4];
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const uint32_t vg = qg[2 * wp + k], vh = qh[2 * wp + k];
                        a[k][0] = h2_fma((vg & mask) | H2_1024, s_g, c_g);
                        a[k][1] = h2_fma((vh & mask) | H2_1024, s_h, c_h);
                        a[k][2] = h2_fma(((vg >> 8) & mask) | H2_1024, s_g, c_g);
                        a[k][3] = h2_fma(((vh >> 8) & mask) | H2_1024, s_h, c_h);
                    }
                    const int p = cc * 4 + n * 2 + wp;
#pragma unroll
                    for (int jt = 0; jt < NT; jt++) {
                        const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 8 + p) * 64);
                        mma16816(acc[jt], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma16816(acc[jt], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                    }
                }
            }
        }
        min_mma<NT>(tab + 1024, 8, g, t, 0, xsrow, sbl * 8, acc);
    }
};

template <int NT> struct Mma<YUUKA_DTYPE_Q5_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q5_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) { header_k4(r.hdr, lane, tab); }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], int sbl, float (&acc)[NT][4]) {
        const int g = lane >> 2, t = lane & 3;
        const uint4 * scl = reinterpret_cast<const uint4 *>(tab);
        const uint32_t hg[4] = {r.qh[0].x, r.qh[0].y, r.qh[0].z, r.qh[0].w};
        const uint32_t hh[4] = {r.qh[1].x, r.qh[1].y, r.qh[1].z, r.qh[1].w};
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
            const int j = (t >> 1) + 2 * cc;
            const uint4 sg = scl[g * 4 + j], sh = scl[(g + 8) * 4 + j];
            const uint32_t qg[4] = {r.q[cc].x, r.q[cc].y, r.q[cc].z, r.q[cc].w};
            const uint32_t qh[4] = {r.q[2 + cc].x, r.q[2 + cc].y, r.q[2 + cc].z, r.q[2 + cc].w};
#pragma unroll
            for (int n = 0; n < 2; n++) {
                const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
#pragma unroll
                for (int wp = 0; wp < 2; wp++) {
                    uint32_t a[2][4];
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int w = 2 * wp + k;
                        const uint32_t vg = qg[w], vh = qh[w];
                        const uint32_t bg = hg[w] >> (2 * j), bh = hh[w] >> (2 * j);  // bit 0: low nibble's fifth bit, bit 1: high nibble's
                        if (n == 0) {
                            a[k][0] = h2_fma((vg & 0x000f000fu) | ((bg << 4) & 0x00100010u) | H2_1024, s_g, c_g);
                            a[k][1] = h2_fma((vh & 0x000f000fu) | ((bh << 4) & 0x00100010u) | H2_1024, s_h, c_h);
                            a[k][2] = h2_fma(((vg >> 8) & 0x000f000fu) | ((bg >> 4) & 0x00100010u) | H2_1024, s_g, c_g);
                            a[k][3] = h2_fma(((vh >> 8) & 0x000f000fu) | ((bh >> 4) & 0x00100010u) | H2_1024, s_h, c_h);
                        } else {
                            a[k][0] = h2_fma((vg & 0x00f000f0u) | ((bg << 7) & 0x01000100u) | H2_1024, s_g, c_g);
                            a[k][1] = h2_fma((vh & 0x00f000f0u) | ((bh << 7) & 0x01000100u) | H2_1024, s_h, c_h);
                            a[k][2] = h2_fma(((vg >> 8) & 0x00f000f0u) | ((bg >> 1) & 0x01000100u) | H2_1024, s_g, c_g);
                            a[k][3] = h2_fma(((vh >> 8) & 0x00f000f0u) | ((bh >> 1) & 0x01000100u) | H2_1024, s_h, c_h);
                        }
                    }
                    const int p = cc * 4 + n * 2 + wp;
#pragma unroll
                    for (int jt = 0; jt < NT; jt++) {
                        const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 8 + p) * 64);
                        mma16816(acc[jt], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma16816(acc[jt], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                    }
                }
            }
        }
        min_mma<NT>(tab + 1024, 8, g, t, 0, xsrow, sbl * 8, acc);
    }
};

// Q6_K table: scl[row][sub k] = {s', c'} with (s, -1024 s) for low-nibble subs (k%8 < 4) and
// (s/16, -64 s) for high-nibble subs; mn2[row][k] = (-32 s, -32 s).
template <int NT> struct Mma<YUUKA_DTYPE_Q6_K, NT> {
    using C = Codec<YUUKA_DTYPE_Q6_K>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;  // hf: subs 8hf .. 8hf+7
        const uint32_t d2 = dup_lo(r.d);
        const uint32_t wa = (hf ? r.sc.z : r.sc.x) ^ 0x80808080u;  // subs +0..3: low-nibble form
        const uint32_t wb = (hf ? r.sc.w : r.sc.y) ^ 0x80808080u;  // subs +4..7: high-nibble form
        uint2 * scl = reinterpret_cast<uint2 *>(tab) + row * 16 + hf * 8;
        uint32_t * mn2 = reinterpret_cast<uint32_t *>(tab + 2048) + row * 16 + hf * 8;
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
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], int sbl, float (&acc)[NT][4]) {
        const int g = lane >> 2, t = lane & 3;
        const uint2 * scl = reinterpret_cast<const uint2 *>(tab);
        const int lsh = 4 - 2 * (t >> 1);  // brings this lane's two high bits to bit 4 (low nibble) / bit 8 (high nibble)
        const int rsh = 8 - lsh;
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
            const uint32_t qg[4] = {r.ql[cc].x, r.ql[cc].y, r.ql[cc].z, r.ql[cc].w};
            const uint32_t qh[4] = {r.ql[2 + cc].x, r.ql[2 + cc].y, r.ql[2 + cc].z, r.ql[2 + cc].w};
            const uint32_t hg[4] = {r.qh[cc].x, r.qh[cc].y, r.qh[cc].z, r.qh[cc].w};
            const uint32_t hh[4] = {r.qh[2 + cc].x, r.qh[2 + cc].y, r.qh[2 + cc].z, r.qh[2 + cc].w};
#pragma unroll
            for (int n = 0; n < 2; n++) {
                const int k = 8 * cc + 4 * n + t;
                const uint2 eg = scl[g * 16 + k], eh = scl[(g + 8) * 16 + k];
                const uint32_t qm = n ? 0x00f000f0u : 0x000f000fu, hm = n ? 0x03000300u : 0x00300030u;
#pragma unroll
                for (int wp = 0; wp < 2; wp++) {
                    uint32_t a[2][4];
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        const int w = 2 * wp + kk;
                        // bytes 0,2 take the high bits shifted left; bytes 1,3 come down by 8 first
                        a[kk][0] = h2_fma((qg[w] & qm) | ((hg[w] << lsh) & hm) | H2_1024, eg.x, eg.y);
                        a[kk][1] = h2_fma((qh[w] & qm) | ((hh[w] << lsh) & hm) | H2_1024, eh.x, eh.y);
                        a[kk][2] = h2_fma(((qg[w] >> 8) & qm) | ((hg[w] >> rsh) & hm) | H2_1024, eg.x, eg.y);
                        a[kk][3] = h2_fma(((qh[w] >> 8) & qm) | ((hh[w] >> rsh) & hm) | H2_1024, eh.x, eh.y);
                    }
                    const int p = cc * 4 + n * 2 + wp;
#pragma unroll
                    for (int jt = 0; jt < NT; jt++) {
                        const uint4 b = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 8 + p) * 64);
                        mma16816(acc[jt], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma16816(acc[jt], a[1][0], a[1][1], a[1][2], a[1][3], b.z, b.w);
                    }
                }
            }
        }
        min_mma<NT>(tab + 2048, 16, g, t, 0, xsrow, sbl * 16, acc);
        min_mma<NT>(tab + 2048, 16, g, t, 8, xsrow, sbl * 16, acc);
    }
};

// Q8_0 table: scl[row][block] = (s, s). Bytes are biased by 128 to make them unsigned, converted
// exactly (1024 + 128 + q), the bias subtracted exactly, then scaled: one rounding per weight.
template <int NT> struct Mma<YUUKA_DTYPE_Q8_0, NT> {
    using C = Codec<YUUKA_DTYPE_Q8_0>;
    __device__ static void header(const typename C::Regs & r, int lane, uint8_t * tab) {
        const int row = lane & 15, hf = lane >> 4;
        const uint32_t da = hf ? r.d.z : r.d.x, db = hf ? r.d.w : r.d.y;
        uint32_t * scl = reinterpret_cast<uint32_t *>(tab) + row * 8 + hf * 4;
        scl[0] = dup_lo(da);
        scl[1] = dup_hi(da);
        scl[2] = dup_lo(db);
        scl[3] = dup_hi(db);
    }
    __device__ static void run(const typename C::Regs & r, int lane, const uint8_t * tab, const uint8_t * const (&xrow)[NT],
                               const uint8_t * const (&xsrow)[NT], int sbl, float (&acc)[NT][4]) {
        (void)xsrow;
        const int g = lane >> 2, t = lane & 3;
        const uint32_t * scl = reinterpret_cast<const uint32_t *>(tab);
#pragma unroll
        for (int cs = 0; cs < 4; cs++) {
            const int b = 2 * cs + (t >> 1);
            const uint32_t sg = scl[g * 8 + b], sh = scl[(g + 8) * 8 + b];
            const uint32_t qg[4] = {r.q[cs].x, r.q[cs].y, r.q[cs].z, r.q[cs].w};
            const uint32_t qh[4] = {r.q[4 + cs].x, r.q[4 + cs].y, r.q[4 + cs].z, r.q[4 + cs].w};
#pragma unroll
            for (int wp = 0; wp < 2; wp++) {
                uint32_t a[2][4];
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    const uint32_t vg = qg[2 * wp + kk] ^ 0x80808080u, vh = qh[2 * wp + kk] ^ 0x80808080u;
                    a[kk][0] = h2_mul(h2_sub(bytes02_h2(vg), H2_1152), sg);
                    a[kk][1] = h2_mul(h2_sub(bytes02_h2(vh), H2_1152), sh);
                    a[kk][2] = h2_mul(h2_sub(bytes13_h2(vg), H2_1152), sg);
                    a[kk][3] = h2_mul(h2_sub(bytes13_h2(vh), H2_1152), sh);
                }
                const int p = cs * 2 + wp;
#pragma unroll
                for (int jt = 0; jt < NT; jt++) {
                    const uint4 bb = *reinterpret_cast<const uint4 *>(xrow[jt] + (sbl * 8 + p) * 64);
                    mma16816(acc[jt], a[0][0], a[0][1], a[0][2], a[0][3], bb.x, bb.y);
                    mma16816(acc[jt], a[1][0], a[1][1], a[1][2], a[1][3], bb.z, bb.w);
                }
            }
        }
    }
};

// ===========================================================================
// mma kernel

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

struct TParams {
    const uint8_t * w;
    int N, nsb;
    const void * x;
    int64_t ldx;
    int M;
    float * out;
    int64_t ldo;
    int accumulate;
    int TG, KS;        // row tiles per group, warps per row tile (TG * KS == TW)
    int kchunks;       // gridDim.y
    int nsb_chunk;     // superblocks per CTA-level K chunk
    int n_groups;
    float * partial;
    int * counters;
};

template <int DT, int NT, typename XT>
__global__ void __launch_bounds__(TW * 32, 2) gemm_tiled_mma_kernel(const TParams p) {
    using C = Codec<DT>;
    using MM = Mma<DT, NT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int c0 = blockIdx.y * p.nsb_chunk;
    const int c1 = min(p.nsb, c0 + p.nsb_chunk);
    const int cnt = c1 - c0;
    const int xstride = p.nsb_chunk * 512 + 64;           // bytes of fp16 activations per row
    const int xsum_stride = p.nsb_chunk * C::NSUB * 4;    // bytes of sub-block sums per row
    uint8_t * xs = smem;
    uint8_t * xsum = xs + (size_t)p.M * xstride;
    uint8_t * tabs = xsum + (((size_t)p.M * xsum_stride + 127) / 128) * 128;
    float * red = reinterpret_cast<float *>(tabs + TW * C::TAB);
    __shared__ int last_flag;

    const int tile_in_group = warp / p.KS, kpart = warp - tile_in_group * p.KS;
    const int sb0 = c0 + (cnt * kpart) / p.KS, sb1 = c0 + (cnt * (kpart + 1)) / p.KS;
    const int n_tiles = (p.N + 15) >> 4;
    const size_t rec_row = (size_t)p.nsb * C::REC;

    // Weights do not depend on the previous kernel: start the first loads before touching x.
    int grp = blockIdx.x;
    typename C::Regs cur, nxt;
    {
        const int rt = min(grp * p.TG + tile_in_group, n_tiles - 1);
        if (sb0 < sb1) C::load(p.w + rt * rec_row + (size_t)sb0 * C::REC, lane, cur);
    }

    // ---- stage activations of this K chunk: fp16 in fragment order, plus sub-block sums ----
    {
        const XT * X = reinterpret_cast<const XT *>(p.x);
        const int groups_per_row = cnt * 32;  // 8-element groups
        for (int i = threadIdx.x; i < p.M * groups_per_row; i += TW * 32) {
            const int m = i / groups_per_row, q = i - m * groups_per_row;
            const int sbl = q >> 5, e8 = q & 31;
            const XT * src = X + (int64_t)m * p.ldx + (int64_t)(c0 + sbl) * 256 + e8 * 8;
            float v[8];
            load8(src, v);
            const __half2 h0 = __floats2half2_rn(v[0], v[2]), h1 = __floats2half2_rn(v[1], v[3]);
            const __half2 h2 = __floats2half2_rn(v[4], v[6]), h3 = __floats2half2_rn(v[5], v[7]);
            int tt;
            const int pslot = C::pair_slot(e8, tt);
            uint4 pk;
            pk.x = *reinterpret_cast<const uint32_t *>(&h0);
            pk.y = *reinterpret_cast<const uint32_t *>(&h1);
            pk.z = *reinterpret_cast<const uint32_t *>(&h2);
            pk.w = *reinterpret_cast<const uint32_t *>(&h3);
            *reinterpret_cast<uint4 *>(xs + (size_t)m * xstride + ((sbl * 8 + pslot) * 4 + tt) * 16) = pk;
            // sums of the rounded values; groups of one sub-block sit in adjacent lanes
            float s8 = (__low2float(h0) + __high2float(h0)) + (__low2float(h1) + __high2float(h1)) +
                       (__low2float(h2) + __high2float(h2)) + (__low2float(h3) + __high2float(h3));
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
            if (C::NSUB == 8) s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
            const int per_sub = C::NSUB == 8 ? 4 : 2;
            if ((e8 & (per_sub - 1)) == 0) {
                const __half hi = __float2half_rn(s8);
                const __half lo = __float2half_rn(s8 - __half2float(hi));
                const __half2 hl = __halves2half2(hi, lo);
                *reinterpret_cast<__half2 *>(xsum + (size_t)m * xsum_stride + (sbl * C::NSUB + e8 / per_sub) * 4) = hl;
            }
        }
    }
    __syncthreads();

    uint8_t * tab = tabs + warp * C::TAB;
    const uint8_t * xrow[NT];
    const uint8_t * xsrow[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int tok = min(8 * j + g, p.M - 1);
        xrow[j] = xs + (size_t)tok * xstride + t * 16;
        xsrow[j] = xsum + (size_t)tok * xsum_stride;
    }

    for (; grp < p.n_groups; grp += gridDim.x) {
        const int rt = grp * p.TG + tile_in_group;
        const int rtc = min(rt, n_tiles - 1);
        const uint8_t * tile = p.w + rtc * rec_row;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[j][c] = 0.0f;

        for (int sb = sb0; sb < sb1; sb++) {
            // prefetch the next record of this tile, or the first record of the next group's tile
            if (sb + 1 < sb1) {
                C::load(tile + (size_t)(sb + 1) * C::REC, lane, nxt);
            } else if (grp + (int)gridDim.x < p.n_groups) {
                const int rtn = min((grp + (int)gridDim.x) * p.TG + tile_in_group, n_tiles - 1);
                C::load(p.w + rtn * rec_row + (size_t)sb0 * C::REC, lane, nxt);
            }
            MM::header(cur, lane, tab);
            __syncwarp();
            MM::run(cur, lane, tab, xrow, xsrow, sb - c0, acc);
            __syncwarp();
            cur = nxt;
        }

        // ---- reduce the K parts of a row tile inside the CTA ----
        if (p.KS > 1) {
            float * mine = red + warp * (NT * 128);
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int c = 0; c < 4; c++) mine[(j * 4 + c) * 32 + lane] = acc[j][c];
            __syncthreads();
            if (kpart == 0) {
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        float s = acc[j][c];
                        for (int k = 1; k < p.KS; k++) s += red[(warp + k) * (NT * 128) + (j * 4 + c) * 32 + lane];
                        acc[j][c] = s;
                    }
            }
        }
        // ---- epilogue ----
        if (kpart == 0 && rt < n_tiles) {
            const int n_g = rt * 16 + g, n_h = n_g + 8;
            float * base = p.kchunks == 1 ? p.out : p.partial + (size_t)blockIdx.y * p.M * p.N;
            const int64_t ld = p.kchunks == 1 ? p.ldo : p.N;
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int tok = 8 * j + 2 * t + (c & 1), n = (c & 2) ? n_h : n_g;
                    if (tok < p.M && n < p.N) {
                        float * dst = base + (int64_t)tok * ld + n;
                        if (p.kchunks == 1) *dst = p.accumulate ? *dst + acc[j][c] : acc[j][c];
                        else __stcg(dst, acc[j][c]);
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
                for (int i = threadIdx.x; i < p.M * nrows; i += TW * 32) {
                    const int tok = i / nrows, n = row0 + (i - tok * nrows);
                    float s = 0.0f;
                    for (int q = 0; q < p.kchunks; q++) s += __ldcg(p.partial + ((size_t)q * p.M + tok) * p.N + n);
                    float * dst = p.out + (int64_t)tok * p.ldo + n;
                    *dst = p.accumulate ? *dst + s : s;
                }
                if (threadIdx.x == 0) p.counters[grp] = 0;
            }
        } else if (p.KS > 1) {
            __syncthreads();  // red is reused by the next group
        }
    }
}

// ===========================================================================
// fp32 kernel over the tiled layout: reference decode arithmetic, CUDA cores.
// A warp owns a row tile over all of K; lane (g, t) accumulates rows g and g+8
// over its share of the columns; the four lanes of a row are summed by shuffles.

constexpr int F32_MT = 4;

template <int DT> struct F32Decode;

// calls f(e, wg[4], wh[4]) for every 4 consecutive elements e..e+3 this lane holds, rows g and g+8
template <> struct F32Decode<YUUKA_DTYPE_Q4_K> {
    template <bool Q5, typename R, typename F> __device__ static void each(const R & r, int lane, const uint8_t * hdr_g,
                                                                            const uint8_t * hdr_h, F f) {
        const int t = lane & 3;
        const float dg = ld_f16(hdr_g), mg = ld_f16(hdr_g + 2), dh = ld_f16(hdr_h), mh = ld_f16(hdr_h + 2);
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
            const int j = (t >> 1) + 2 * cc;
            const uint32_t qg[4] = {r.q[cc].x, r.q[cc].y, r.q[cc].z, r.q[cc].w};
            const uint32_t qh[4] = {r.q[2 + cc].x, r.q[2 + cc].y, r.q[2 + cc].z, r.q[2 + cc].w};
#pragma unroll
            for (int n = 0; n < 2; n++) {
                int sc, mn;
                scale_min_k4(2 * j + n, hdr_g + 4, sc, mn);
                const float d1g = dg * (float)sc, m1g = mg * (float)mn;
                scale_min_k4(2 * j + n, hdr_h + 4, sc, mn);
                const float d1h = dh * (float)sc, m1h = mh * (float)mn;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    float wg[4], wh[4];
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        int vg = (qg[w] >> (8 * b + 4 * n)) & 15, vh = (qh[w] >> (8 * b + 4 * n)) & 15;
                        if constexpr (Q5) {
                            const uint32_t bg = ((const uint32_t *)&r.qh[0])[w], bh = ((const uint32_t *)&r.qh[1])[w];
                            vg += ((bg >> (8 * b + 2 * j + n)) & 1) << 4;
                            vh += ((bh >> (8 * b + 2 * j + n)) & 1) << 4;
                        }
                        wg[b] = d1g * (float)vg - m1g;
                        wh[b] = d1h * (float)vh - m1h;
                    }
                    f(64 * j + 32 * n + 16 * (t & 1) + 4 * w, wg, wh);
                }
            }
        }
    }
};

template <int DT, typename XT>
__global__ void __launch_bounds__(TW * 32) gemm_tiled_fp32_kernel(const TParams p) {
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
            auto fma4 = [&](int e, const float (&wg)[4], const float (&wh)[4]) {
#pragma unroll
                for (int m = 0; m < F32_MT; m++) {
                    if (m < p.M) {
                        const float4 xv = *reinterpret_cast<const float4 *>(xb + m * K + e);
                        ag[m] = fmaf(xv.x, wg[0], ag[m]); ag[m] = fmaf(xv.y, wg[1], ag[m]);
                        ag[m] = fmaf(xv.z, wg[2], ag[m]); ag[m] = fmaf(xv.w, wg[3], ag[m]);
                        ah[m] = fmaf(xv.x, wh[0], ah[m]); ah[m] = fmaf(xv.y, wh[1], ah[m]);
                        ah[m] = fmaf(xv.z, wh[2], ah[m]); ah[m] = fmaf(xv.w, wh[3], ah[m]);
                    }
                }
            };
            if constexpr (DT == YUUKA_DTYPE_Q4_K || DT == YUUKA_DTYPE_Q5_K) {
                // headers through shared memory: lane r holds row r's 16 bytes
                __syncwarp();
                if (lane < 16) *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 16) = r.hdr;
                __syncwarp();
                F32Decode<YUUKA_DTYPE_Q4_K>::template each<DT == YUUKA_DTYPE_Q5_K>(r, lane, hdrs[warp] + g * 16,
                                                                          hdrs[warp] + (g + 8) * 16, fma4);
            } else if constexpr (DT == YUUKA_DTYPE_Q6_K) {
                __syncwarp();
                if (lane < 16) {
                    *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 32) = r.sc;
                    *reinterpret_cast<uint32_t *>(hdrs[warp] + lane * 32 + 16) = r.d;
                }
                __syncwarp();
                const int8_t * scg = reinterpret_cast<const int8_t *>(hdrs[warp] + g * 32);
                const int8_t * sch = reinterpret_cast<const int8_t *>(hdrs[warp] + (g + 8) * 32);
                const float dg = ld_f16(hdrs[warp] + g * 32 + 16), dh = ld_f16(hdrs[warp] + (g + 8) * 32 + 16);
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
                    const uint32_t qg[4] = {r.ql[cc].x, r.ql[cc].y, r.ql[cc].z, r.ql[cc].w};
                    const uint32_t qh[4] = {r.ql[2 + cc].x, r.ql[2 + cc].y, r.ql[2 + cc].z, r.ql[2 + cc].w};
                    const uint32_t hg[4] = {r.qh[cc].x, r.qh[cc].y, r.qh[cc].z, r.qh[cc].w};
                    const uint32_t hh[4] = {r.qh[2 + cc].x, r.qh[2 + cc].y, r.qh[2 + cc].z, r.qh[2 + cc].w};
#pragma unroll
                    for (int n = 0; n < 2; n++) {
                        const int g4 = (t >> 1) + 2 * n, k = 8 * cc + 4 * n + t;
                        const float sg = dg * (float)scg[k], sh = dh * (float)sch[k];
#pragma unroll
                        for (int w = 0; w < 4; w++) {
                            float wg[4], wh[4];
#pragma unroll
                            for (int b = 0; b < 4; b++) {
                                const int vg = ((qg[w] >> (8 * b + 4 * n)) & 15) | (((hg[w] >> (8 * b + 2 * g4)) & 3) << 4);
                                const int vh = ((qh[w] >> (8 * b + 4 * n)) & 15) | (((hh[w] >> (8 * b + 2 * g4)) & 3) << 4);
                                wg[b] = sg * (float)(vg - 32);
                                wh[b] = sh * (float)(vh - 32);
                            }
                            fma4(128 * cc + 32 * g4 + 16 * (t & 1) + 4 * w, wg, wh);
                        }
                    }
                }
            } else {  // Q8_0
                __syncwarp();
                if (lane < 16) *reinterpret_cast<uint4 *>(hdrs[warp] + lane * 16) = r.d;
                __syncwarp();
#pragma unroll
                for (int cs = 0; cs < 4; cs++) {
                    const int b8 = 2 * cs + (t >> 1);
                    const float dg = ld_f16(hdrs[warp] + g * 16 + 2 * b8), dh = ld_f16(hdrs[warp] + (g + 8) * 16 + 2 * b8);
                    const uint32_t qg[4] = {r.q[cs].x, r.q[cs].y, r.q[cs].z, r.q[cs].w};
                    const uint32_t qh[4] = {r.q[4 + cs].x, r.q[4 + cs].y, r.q[4 + cs].z, r.q[4 + cs].w};
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        float wg[4], wh[4];
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            wg[b] = dg * (float)(int8_t)(qg[w] >> (8 * b));
                            wh[b] = dh * (float)(int8_t)(qh[w] >> (8 * b));
                        }
                        fma4(32 * b8 + 16 * (t & 1) + 4 * w, wg, wh);
                    }
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

static int nsub_of(uint32_t dtype) { return dtype == YUUKA_DTYPE_Q6_K ? 16 : 8; }
static int tab_of(uint32_t dtype) { return dtype == YUUKA_DTYPE_Q6_K ? 3072 : 1536; }

static size_t mma_smem(uint32_t dtype, int m, int nsb_chunk, int nt, int ks) {
    size_t x = (size_t)m * (nsb_chunk * 512 + 64);
    size_t xsum = (((size_t)m * nsb_chunk * nsub_of(dtype) * 4 + 127) / 128) * 128;
    size_t red = ks > 1 ? (size_t)TW * nt * 128 * 4 : 0;
    return x + xsum + (size_t)TW * tab_of(dtype) + red;
}

static void plan_tiled(const yuuka_device * dev, uint32_t dtype, int m, int n_out, int n_in, TPlan & pl) {
    const int nsb = n_in / 256, n_tiles = (n_out + 15) / 16;
    const int nt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
    const int slots = 2 * dev->sm_count;  // CTAs that can be resident (two per SM)
    // warps per row tile: as many K parts as needed to give every resident CTA a group
    int ks = 1;
    while (ks < TW && (n_tiles * ks) / TW < slots * 4 / 5 && nsb / (2 * ks) >= 1) ks *= 2;
    pl.KS = ks;
    pl.TG = TW / ks;
    pl.n_groups = (n_tiles + pl.TG - 1) / pl.TG;
    // CTA-level K chunks: when even KS = TW leaves SMs idle, or the activations do not fit two CTAs per SM
    int kchunks = 1;
    const size_t budget = (dev->prop.sharedMemPerMultiprocessor - 2048) / 2 < dev->prop.sharedMemPerBlockOptin
                              ? (dev->prop.sharedMemPerMultiprocessor - 2048) / 2
                              : dev->prop.sharedMemPerBlockOptin;
    while (true) {
        int nsb_chunk = (nsb + kchunks - 1) / kchunks;
        bool fits = mma_smem(dtype, m, nsb_chunk, nt, ks) <= budget;
        bool enough = pl.n_groups * kchunks >= slots / 2 || nsb_chunk < 2 * ks || nsb_chunk <= 2;
        if (fits && enough) break;
        if (nsb_chunk == 1) break;
        kchunks++;
    }
    pl.nsb_chunk = (nsb + kchunks - 1) / kchunks;
    pl.kchunks = (nsb + pl.nsb_chunk - 1) / pl.nsb_chunk;
    pl.smem = mma_smem(dtype, m, pl.nsb_chunk, nt, ks);
    int per = slots / pl.kchunks;
    if (per < 1) per = 1;
    pl.grid_x = pl.n_groups < per ? pl.n_groups : per;
}

void gemm_tiled_scratch_need(const yuuka_device * dev, uint32_t w_dtype, int rows, int n_out, int n_in,
                             uint64_t * partial_floats, int * counters) {
    *partial_floats = 0;
    *counters = 0;
    if (!tiled_supported(w_dtype, n_in)) return;
    for (int m : {rows < 32 ? rows : 32, 32 < rows ? rows % 32 : 0}) {
        if (m <= 0 || m <= 2) continue;
        TPlan pl;
        plan_tiled(dev, w_dtype, m, n_out, n_in, pl);
        if (pl.kchunks > 1) {
            uint64_t need = (uint64_t)pl.kchunks * m * n_out;
            if (need > *partial_floats) *partial_floats = need;
            if (pl.n_groups > *counters) *counters = pl.n_groups;
        }
    }
}

template <int DT, int NT, typename XT>
static void launch_mma_inst(cudaStream_t s, const TiledGemmArgs & a, int m0, int m, const TPlan & pl) {
    auto kern = gemm_tiled_mma_kernel<DT, NT, XT>;
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    TParams p;
    p.w = a.w;
    p.N = a.n_out;
    p.nsb = a.n_in / 256;
    p.x = (const XT *)a.x + (int64_t)m0 * a.ldx;
    p.ldx = a.ldx;
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
    dim3 grid(pl.grid_x, pl.kchunks);
    kern<<<grid, TW * 32, pl.smem, s>>>(p);
    YK_CUDA(cudaGetLastError());
}

template <int DT, typename XT>
static int launch_mma_dt(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a) {
    int launches = 0;
    for (int m0 = 0; m0 < a.rows; m0 += 32) {
        const int m = a.rows - m0 < 32 ? a.rows - m0 : 32;
        TPlan pl;
        plan_tiled(dev, a.w_dtype, m, a.n_out, a.n_in, pl);
        YK_REQUIRE(pl.smem <= dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_UNSUPPORTED,
                   "gemm: activations of %d rows x %d columns do not fit shared memory", m, a.n_in);
        if (pl.kchunks > 1)
            YK_REQUIRE(a.scratch && a.scratch->partial_floats >= (uint64_t)pl.kchunks * m * a.n_out &&
                           a.scratch->counter_count >= pl.n_groups,
                       YUUKA_ERR_INTERNAL, "gemm: split-K scratch is too small");
        if (m <= 8) launch_mma_inst<DT, 1, XT>(s, a, m0, m, pl);
        else if (m <= 16) launch_mma_inst<DT, 2, XT>(s, a, m0, m, pl);
        else launch_mma_inst<DT, 4, XT>(s, a, m0, m, pl);
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
        kern<<<grid, TW * 32, (size_t)m * a.n_in * sizeof(float), s>>>(p);
        YK_CUDA(cudaGetLastError());
        launches++;
    }
    return launches;
}

template <typename XT>
static int launch_tiled_x(const yuuka_device * dev, cudaStream_t s, const TiledGemmArgs & a, bool mma) {
    switch (a.w_dtype) {
    case YUUKA_DTYPE_Q4_K: return mma ? launch_mma_dt<YUUKA_DTYPE_Q4_K, XT>(dev, s, a) : launch_fp32_dt<YUUKA_DTYPE_Q4_K, XT>(dev, s, a);
    case YUUKA_DTYPE_Q5_K: return mma ? launch_mma_dt<YUUKA_DTYPE_Q5_K, XT>(dev, s, a) : launch_fp32_dt<YUUKA_DTYPE_Q5_K, XT>(dev, s, a);
    case YUUKA_DTYPE_Q6_K: return mma ? launch_mma_dt<YUUKA_DTYPE_Q6_K, XT>(dev, s, a) : launch_fp32_dt<YUUKA_DTYPE_Q6_K, XT>(dev, s, a);
    case YUUKA_DTYPE_Q8_0: return mma ? launch_mma_dt<YUUKA_DTYPE_Q8_0, XT>(dev, s, a) : launch_fp32_dt<YUUKA_DTYPE_Q8_0, XT>(dev, s, a);
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "gemm: dtype %u has no tiled kernels", a.w_dtype);
    }
    return 0;
}

int launch_gemm_tiled(const yuuka_device * dev, cudaStream_t stream, const TiledGemmArgs & a) {
    YK_REQUIRE(a.w && a.x && a.out, YUUKA_ERR_INVALID_ARGUMENT, "gemm: null operand");
    YK_REQUIRE(a.rows > 0 && a.n_out > 0 && a.n_in > 0, YUUKA_ERR_INVALID_ARGUMENT, "gemm: invalid shape");
    YK_REQUIRE(tiled_supported(a.w_dtype, a.n_in), YUUKA_ERR_UNSUPPORTED, "gemm: dtype %u / width %d has no tiled layout",
               a.w_dtype, a.n_in);
    YK_REQUIRE(a.x_dtype == YUUKA_DTYPE_F32 || a.x_dtype == YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
               "gemm: activation dtype %u is not F32 or BF16", a.x_dtype);
    YK_REQUIRE(a.ldx >= a.n_in && a.ldo >= a.n_out, YUUKA_ERR_INVALID_ARGUMENT, "gemm: leading dimension too small");
    uint32_t path = a.path == YUUKA_GEMM_PATH_AUTO ? (a.rows <= 2 ? YUUKA_GEMM_PATH_FP32 : YUUKA_GEMM_PATH_MMA) : a.path;
    YK_REQUIRE(path == YUUKA_GEMM_PATH_FP32 || path == YUUKA_GEMM_PATH_MMA, YUUKA_ERR_INVALID_ARGUMENT,
               "gemm: unknown path %u", path);
    set_device(dev);
    const bool mma = path == YUUKA_GEMM_PATH_MMA;
    return a.x_dtype == YUUKA_DTYPE_F32 ? launch_tiled_x<float>(dev, stream, a, mma)
                                        : launch_tiled_x<__nv_bfloat16>(dev, stream, a, mma);
}

}  // namespace yk
