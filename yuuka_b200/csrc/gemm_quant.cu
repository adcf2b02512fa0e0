// Quantized dequant-GEMM over the draft rows of a verify step:
//   out[m][n] = sum_k x[m][k] * W[n][k],  W in packed GGUF rows (Q4_K/Q5_K/Q6_K/Q8_0/F16/F32)
// (replaces kernels/hip/gemm/lm_head.hip, gemv/gemv_quant.hip:317 and the
// verify-sized use of gemm/wmma_gemm.hip in the reference).
//
// Two routes:
//  * fp32: warp-per-row CUDA-core dot products with the reference's own fp32
//    decode (tensor/quant.go). The FP32 pipe of an SM sustains 128 FMA/clk,
//    which at B200's HBM rate is only ~3 rows of a 4.5-bit matrix, so this
//    route serves 1-2 rows and tight-tolerance checks.
//  * mma: packed rows stream through a shared-memory ring filled by bulk
//    asynchronous copies (cp.async.bulk + mbarrier), are decoded to fp16 in
//    registers directly into mma.sync A fragments, multiplied with fp16
//    activations staged once per CTA, accumulated in fp32. Split-K partials
//    are reduced by the last CTA to arrive at a tile, in a fixed order.
#include "gemm_quant.cuh"
#include "quant.cuh"

namespace yk {

__device__ int g_device_error = 0;

int read_device_error(const yuuka_device * dev) {
    set_device(dev);
    int v = 0;
    YK_CUDA(cudaMemcpyFromSymbol(&v, g_device_error, sizeof(int)));
    return v;
}

// ===========================================================================
// fp32 route

constexpr int FP32_MT = 4;  // activation rows per pass

template <typename XT> __device__ __forceinline__ float x_to_f32(XT v);
template <> __device__ __forceinline__ float x_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float x_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <int DT, typename XT>
__global__ void __launch_bounds__(256) gemm_q_fp32_kernel(const uint8_t * __restrict__ W, int64_t rb, int N, int K,
                                                           const XT * __restrict__ X, int64_t ldx, int M,
                                                           float * __restrict__ out, int64_t ldo, int accumulate) {
    extern __shared__ __align__(16) float xs[];  // [M][K]
    for (int i = threadIdx.x; i < M * K; i += blockDim.x) {
        int m = i / K, k = i - m * K;
        xs[i] = x_to_f32<XT>(X[(int64_t)m * ldx + k]);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = K >> 3;
    for (int n = blockIdx.x * 8 + warp; n < N; n += gridDim.x * 8) {
        const uint8_t * row = W + (int64_t)n * rb;
        float acc[FP32_MT];
#pragma unroll
        for (int m = 0; m < FP32_MT; m++) acc[m] = 0.0f;
        for (int e8 = lane; e8 < groups; e8 += 32) {
            float w[8];
            decode8<DT>(row, e8, w);
#pragma unroll
            for (int m = 0; m < FP32_MT; m++) {
                if (m < M) {
                    const float4 * xp = reinterpret_cast<const float4 *>(xs + m * K + e8 * 8);
                    float4 a = xp[0], b = xp[1];
                    acc[m] = fmaf(a.x, w[0], acc[m]);
                    acc[m] = fmaf(a.y, w[1], acc[m]);
                    acc[m] = fmaf(a.z, w[2], acc[m]);
                    acc[m] = fmaf(a.w, w[3], acc[m]);
                    acc[m] = fmaf(b.x, w[4], acc[m]);
                    acc[m] = fmaf(b.y, w[5], acc[m]);
                    acc[m] = fmaf(b.z, w[6], acc[m]);
                    acc[m] = fmaf(b.w, w[7], acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < FP32_MT; m++) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < M) {
                float * dst = out + (int64_t)m * ldo + n;
                *dst = accumulate ? *dst + v : v;
            }
        }
    }
}

template <int DT, typename XT>
static int launch_fp32_t(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a) {
    int launches = 0;
    int64_t rb = (int64_t)row_bytes(a.w_dtype, a.n_in);
    auto kern = gemm_q_fp32_kernel<DT, XT>;
    size_t smem_max = (size_t)FP32_MT * a.n_in * sizeof(float);
    YK_REQUIRE(smem_max <= (size_t)dev->prop.sharedMemPerBlockOptin, YUUKA_ERR_UNSUPPORTED,
               "gemm_quant fp32 route: n_in %d does not fit shared memory", a.n_in);
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
    int grid = (a.n_out + 7) / 8;
    int cap = dev->sm_count * 8;
    if (grid > cap) grid = cap;
    for (int m0 = 0; m0 < a.rows; m0 += FP32_MT) {
        int m = a.rows - m0 < FP32_MT ? a.rows - m0 : FP32_MT;
        size_t smem = (size_t)m * a.n_in * sizeof(float);
        kern<<<grid, 256, smem, stream>>>(a.w, rb, a.n_out, a.n_in, (const XT *)a.x + (int64_t)m0 * a.ldx, a.ldx, m,
                                          a.out + (int64_t)m0 * a.ldo, a.ldo, (a.flags & YUUKA_GEMM_ACCUMULATE) ? 1 : 0);
        YK_CUDA(cudaGetLastError());
        launches++;
    }
    return launches;
}

template <typename XT>
static int launch_fp32(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a) {
    switch (a.w_dtype) {
    case YUUKA_DTYPE_F32: return launch_fp32_t<YUUKA_DTYPE_F32, XT>(dev, stream, a);
    case YUUKA_DTYPE_F16: return launch_fp32_t<YUUKA_DTYPE_F16, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q8_0: return launch_fp32_t<YUUKA_DTYPE_Q8_0, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q4_K: return launch_fp32_t<YUUKA_DTYPE_Q4_K, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q5_K: return launch_fp32_t<YUUKA_DTYPE_Q5_K, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q6_K: return launch_fp32_t<YUUKA_DTYPE_Q6_K, XT>(dev, stream, a);
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "gemm_quant: unsupported weight dtype %u", a.w_dtype);
    }
    return 0;
}

// ===========================================================================
// mma route

constexpr int MAX_STAGES = 8;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // bounded mbarrier polling

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Polls with an iteration limit. On expiry sets the CTA poison word and the
// device error word; every later wait of the CTA then returns at once.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, volatile int * poison, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*poison) return false;
    }
    *poison = 1;
    atomicExch(&g_device_error, code);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void * dst, const void * src, uint32_t bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t h2_bcast(float v) {
    __half2 h = __float2half2_rn(v);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// u32 from a 2-byte aligned shared address: two aligned words and a funnel shift.
__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t * p) {
    uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t * q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
    return __funnelshift_r(q[0], q[1], (uint32_t)(a & 2) * 8);
}
// two consecutive u32 from a 2-byte aligned shared address
__device__ __forceinline__ void lds_u32x2_a2(const uint8_t * p, uint32_t & v0, uint32_t & v1) {
    uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t * q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
    uint32_t sh = (uint32_t)(a & 2) * 8;
    uint32_t w0 = q[0], w1 = q[1], w2 = q[2];
    v0 = __funnelshift_r(w0, w1, sh);
    v1 = __funnelshift_r(w1, w2, sh);
}

constexpr uint32_t H2_1024 = 0x64006400u;
constexpr uint32_t H2_1056 = 0x64206420u;
constexpr uint32_t H2_1152 = 0x64806480u;
constexpr uint32_t H2_INV16 = 0x2C002C00u;
constexpr uint32_t H2_NEG64 = 0xD400D400u;

// Activation order inside one 64-element unit. MMA i (0..3) of the unit covers
// elements (i>>1)*32 + 8t + (i&1)*4 + {0,2 | 1,3} for the four lanes t that
// share a weight row; position p = t*16 + i*4 + s holds that element, so one
// lane reads its four B fragments with two 16-byte loads.
__device__ __forceinline__ int unit_pos_of_group4(int e) {  // e multiple of 4, within the unit
    int hi = e >> 5, r = e & 31, t = r >> 3, w = (r >> 2) & 1;
    return t * 16 + (hi * 2 + w) * 4;
}

struct MmaParams {
    const uint8_t * w;
    int64_t rb;
    int N, K;
    const void * x;
    int64_t ldx;
    int M;
    float * out;
    int64_t ldo;
    int accumulate;
    int ksplit;      // gridDim.y
    int nsb_part;    // superblocks per K part
    int stages;
    float * partial;
    int * counters;
};

// Per-(row, superblock) scale tables written by the header decode.
//  Q4_K/Q5_K: 8 x {half2 scale, half2 -min}         (64 B)
//  Q6_K     : 16 x half2 scale                       (64 B)
//  Q8_0     : 8 x half2 scale                        (32 B, stride 64)
constexpr int TAB_STRIDE = 64;

template <int DT>
__device__ __forceinline__ void decode_header(const uint8_t * blk, uint8_t * tab) {
    uint32_t * t32 = reinterpret_cast<uint32_t *>(tab);
    if constexpr (DT == YUUKA_DTYPE_Q4_K || DT == YUUKA_DTYPE_Q5_K) {
        const uint32_t * h = reinterpret_cast<const uint32_t *>(blk);
        uint32_t dd = h[0], w0 = h[1], w1 = h[2], w2 = h[3];
        float d = __half2float(__ushort_as_half((uint16_t)(dd & 0xffff)));
        float dm = __half2float(__ushort_as_half((uint16_t)(dd >> 16)));
        uint32_t sc_lo = w0 & 0x3f3f3f3fu, mn_lo = w1 & 0x3f3f3f3fu;
        uint32_t sc_hi = (w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u);
        uint32_t mn_hi = ((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            uint32_t sc = ((j < 4 ? sc_lo : sc_hi) >> (8 * (j & 3))) & 0xff;
            uint32_t mn = ((j < 4 ? mn_lo : mn_hi) >> (8 * (j & 3))) & 0xff;
            t32[2 * j] = h2_bcast(d * (float)sc);
            t32[2 * j + 1] = h2_bcast(-(dm * (float)mn));
        }
    } else if constexpr (DT == YUUKA_DTYPE_Q6_K) {
        float d = ld_f16(blk + 208);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            uint32_t s2 = ld_u16(blk + 192 + 2 * j);
            t32[2 * j] = h2_bcast(d * (float)(int8_t)(s2 & 0xff));
            t32[2 * j + 1] = h2_bcast(d * (float)(int8_t)(s2 >> 8));
        }
    } else if constexpr (DT == YUUKA_DTYPE_Q8_0) {
#pragma unroll
        for (int j = 0; j < 8; j++) t32[j] = h2_bcast(ld_f16(blk + 34 * j));
    }
}

// A fragments of the four MMAs of unit u (0..3) of one superblock, for the two
// rows (blk_g, blk_h) this lane holds. a[i][0..3] = {row g k-lo, row g+8 k-lo,
// row g k-hi, row g+8 k-hi}.
template <int DT>
__device__ __forceinline__ void decode_unit(const uint8_t * blk_g, const uint8_t * blk_h, const uint8_t * tab_g,
                                            const uint8_t * tab_h, int u, int t, uint32_t a[4][4]) {
    if constexpr (DT == YUUKA_DTYPE_Q4_K || DT == YUUKA_DTYPE_Q5_K) {
        constexpr int QS = DT == YUUKA_DTYPE_Q4_K ? 16 : 48;
        const uint2 vg = *reinterpret_cast<const uint2 *>(blk_g + QS + u * 32 + t * 8);
        const uint2 vh = *reinterpret_cast<const uint2 *>(blk_h + QS + u * 32 + t * 8);
        const uint4 sg = *reinterpret_cast<const uint4 *>(tab_g + u * 16);  // {sL, -mL, sH, -mH}
        const uint4 sh = *reinterpret_cast<const uint4 *>(tab_h + u * 16);
        uint32_t hg0 = 0, hg1 = 0, hh0 = 0, hh1 = 0;
        if constexpr (DT == YUUKA_DTYPE_Q5_K) {
            const uint2 qg = *reinterpret_cast<const uint2 *>(blk_g + 16 + t * 8);
            const uint2 qh = *reinterpret_cast<const uint2 *>(blk_h + 16 + t * 8);
            hg0 = qg.x >> (2 * u); hg1 = qg.y >> (2 * u);
            hh0 = qh.x >> (2 * u); hh1 = qh.y >> (2 * u);
        }
        auto lo = [&](uint32_t v, uint32_t hb, uint32_t s, uint32_t nm) {
            uint32_t h = (v & 0x000f000fu) | H2_1024;
            if constexpr (DT == YUUKA_DTYPE_Q5_K) h |= (hb & 0x00010001u) << 4;
            return h2_fma(h2_sub(h, H2_1024), s, nm);
        };
        auto hi = [&](uint32_t v, uint32_t hb, uint32_t s, uint32_t nm) {
            if constexpr (DT == YUUKA_DTYPE_Q5_K) {
                uint32_t h = ((v >> 4) & 0x000f000fu) | ((hb & 0x00020002u) << 3) | H2_1024;
                return h2_fma(h2_sub(h, H2_1024), s, nm);
            } else {
                uint32_t h = (v & 0x00f000f0u) | H2_1024;
                return h2_fma(h2_fma(h, H2_INV16, H2_NEG64), s, nm);
            }
        };
        a[0][0] = lo(vg.x, hg0, sg.x, sg.y);      a[0][1] = lo(vh.x, hh0, sh.x, sh.y);
        a[0][2] = lo(vg.x >> 8, hg0 >> 8, sg.x, sg.y); a[0][3] = lo(vh.x >> 8, hh0 >> 8, sh.x, sh.y);
        a[1][0] = lo(vg.y, hg1, sg.x, sg.y);      a[1][1] = lo(vh.y, hh1, sh.x, sh.y);
        a[1][2] = lo(vg.y >> 8, hg1 >> 8, sg.x, sg.y); a[1][3] = lo(vh.y >> 8, hh1 >> 8, sh.x, sh.y);
        a[2][0] = hi(vg.x, hg0, sg.z, sg.w);      a[2][1] = hi(vh.x, hh0, sh.z, sh.w);
        a[2][2] = hi(vg.x >> 8, hg0 >> 8, sg.z, sg.w); a[2][3] = hi(vh.x >> 8, hh0 >> 8, sh.z, sh.w);
        a[3][0] = hi(vg.y, hg1, sg.z, sg.w);      a[3][1] = hi(vh.y, hh1, sh.z, sh.w);
        a[3][2] = hi(vg.y >> 8, hg1 >> 8, sg.z, sg.w); a[3][3] = hi(vh.y >> 8, hh1 >> 8, sh.z, sh.w);
    } else if constexpr (DT == YUUKA_DTYPE_Q6_K) {
        // unit u: half n = u>>1; which = u&1 selects g in {0,1} (low nibbles) or {2,3} (high nibbles)
        const int n = u >> 1, which = u & 1;
        const uint32_t * sg = reinterpret_cast<const uint32_t *>(tab_g) + n * 8 + (t >> 1);
        const uint32_t * sh = reinterpret_cast<const uint32_t *>(tab_h) + n * 8 + (t >> 1);
        auto build = [&](const uint8_t * blk, const uint32_t * sc, int col) {
            uint32_t A0, A1, B0, B1, H0, H1;
            lds_u32x2_a2(blk + n * 64 + t * 8, A0, A1);
            lds_u32x2_a2(blk + n * 64 + 32 + t * 8, B0, B1);
            lds_u32x2_a2(blk + 128 + n * 32 + t * 8, H0, H1);
            if (which) { A0 >>= 4; A1 >>= 4; B0 >>= 4; B1 >>= 4; H0 >>= 4; H1 >>= 4; }
            const uint32_t s_a = sc[which * 4], s_b = sc[which * 4 + 2];  // scale index 2g + (t>>1), g = 2*which (+1)
            auto cv = [&](uint32_t q, uint32_t hb, uint32_t s) {
                uint32_t h = (q & 0x000f000fu) | ((hb << 4) & 0x00300030u) | H2_1024;
                return h2_mul(h2_sub(h, H2_1056), s);
            };
            a[0][col] = cv(A0, H0, s_a);           a[0][col + 2] = cv(A0 >> 8, H0 >> 8, s_a);
            a[1][col] = cv(A1, H1, s_a);           a[1][col + 2] = cv(A1 >> 8, H1 >> 8, s_a);
            a[2][col] = cv(B0, H0 >> 2, s_b);      a[2][col + 2] = cv(B0 >> 8, H0 >> 10, s_b);
            a[3][col] = cv(B1, H1 >> 2, s_b);      a[3][col + 2] = cv(B1 >> 8, H1 >> 10, s_b);
        };
        build(blk_g, sg, 0);
        build(blk_h, sh, 1);
    } else if constexpr (DT == YUUKA_DTYPE_Q8_0) {
        auto build = [&](const uint8_t * blk, const uint8_t * tab, int col) {
            const uint32_t * sc = reinterpret_cast<const uint32_t *>(tab) + 2 * u;
            uint32_t A0, A1, B0, B1;
            lds_u32x2_a2(blk + 34 * (2 * u) + 2 + t * 8, A0, A1);
            lds_u32x2_a2(blk + 34 * (2 * u + 1) + 2 + t * 8, B0, B1);
            auto cv = [&](uint32_t q, uint32_t s) {
                uint32_t h = ((q ^ 0x00800080u) & 0x00ff00ffu) | H2_1024;
                return h2_mul(h2_sub(h, H2_1152), s);
            };
            a[0][col] = cv(A0, sc[0]); a[0][col + 2] = cv(A0 >> 8, sc[0]);
            a[1][col] = cv(A1, sc[0]); a[1][col + 2] = cv(A1 >> 8, sc[0]);
            a[2][col] = cv(B0, sc[1]); a[2][col + 2] = cv(B0 >> 8, sc[1]);
            a[3][col] = cv(B1, sc[1]); a[3][col + 2] = cv(B1 >> 8, sc[1]);
        };
        build(blk_g, tab_g, 0);
        build(blk_h, tab_h, 1);
    }
}

template <int DT, int SBS> struct SlotBytes {
    static constexpr int seg = BlockTraits<DT>::sb_bytes * SBS;
    static constexpr int value = ((seg + 15 + 15) / 16) * 16 + 16;
};

template <int DT, int NW, int SBS, int NT, typename XT>
__global__ void __launch_bounds__((NW + 1) * 32, 1) gemm_q_mma_kernel(const MmaParams p) {
    constexpr int SB = BlockTraits<DT>::sb_bytes;
    constexpr int SLOT = SlotBytes<DT, SBS>::value;
    constexpr int TILE_ROWS = NW * 16;
    constexpr int STAGE_BYTES = TILE_ROWS * SLOT;
    constexpr int TAB_BYTES = 16 * SBS * TAB_STRIDE;  // per warp

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    uint64_t * empty = full + MAX_STAGES;
    volatile int * poison = reinterpret_cast<volatile int *>(empty + MAX_STAGES);
    int * last_flag = const_cast<int *>(poison) + 1;
    uint8_t * tabs = smem + 256;
    uint8_t * xs = tabs + NW * TAB_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;
    const int sb0 = blockIdx.y * p.nsb_part;
    const int sb1 = min(nsb, sb0 + p.nsb_part);
    const int kp = (sb1 - sb0) * 256;
    const int xstride = p.nsb_part * 512 + 16;  // bytes per activation row
    uint8_t * ring = xs + (((size_t)p.M * xstride + 127) / 128) * 128;
    const int kstages = (sb1 - sb0 + SBS - 1) / SBS;
    const int n_tiles = (p.N + TILE_ROWS - 1) / TILE_ROWS;
    const int stages = p.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NW);
        }
        *poison = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == NW) {
        // ---- producer warp: one bulk copy per (row, stage) ----
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            for (int ks = 0; ks < kstages; ks++, it++) {
                const int slot = it % stages;
                const uint32_t parity = ((it / stages) & 1) ^ 1;
                if (!mbar_wait(&empty[slot], parity, poison, 1)) goto producer_done;
                const int sbf = sb0 + ks * SBS;
                const int seg = min(SBS, sb1 - sbf) * SB;
                uint32_t total = 0;
#pragma unroll
                for (int r = lane; r < TILE_ROWS; r += 32) {
                    int grow = min(tile * TILE_ROWS + r, p.N - 1);
                    uintptr_t g = reinterpret_cast<uintptr_t>(p.w) + (uintptr_t)grow * p.rb + (uintptr_t)sbf * SB;
                    uintptr_t a = g & ~(uintptr_t)15;
                    total += (uint32_t)(((g + seg + 15) & ~(uintptr_t)15) - a);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                if (lane == 0) mbar_expect_tx(&full[slot], total);
                __syncwarp();
#pragma unroll
                for (int r = lane; r < TILE_ROWS; r += 32) {
                    int grow = min(tile * TILE_ROWS + r, p.N - 1);
                    uintptr_t g = reinterpret_cast<uintptr_t>(p.w) + (uintptr_t)grow * p.rb + (uintptr_t)sbf * SB;
                    uintptr_t a = g & ~(uintptr_t)15;
                    uint32_t len = (uint32_t)(((g + seg + 15) & ~(uintptr_t)15) - a);
                    bulk_copy_g2s(ring + (size_t)slot * STAGE_BYTES + (size_t)r * SLOT, reinterpret_cast<const void *>(a),
                                  len, &full[slot]);
                }
            }
        }
    producer_done:
        // Leave only when every copy this warp issued has landed.
        if (lane == 0) {
            int poisoned_dummy = 0;
            uint32_t first = it > (uint32_t)stages ? it - stages : 0;
            for (uint32_t j = first; j < it; j++) mbar_wait(&full[j % stages], (j / stages) & 1, &poisoned_dummy, 3);
        }
        return;
    }

    // ---- consumer warps ----
    // Stage the activations of this K part as fp16 in MMA order.
    {
        const int ctid = threadIdx.x, cthreads = NW * 32;
        const XT * X = reinterpret_cast<const XT *>(p.x);
        const int groups = kp >> 2;
        for (int i = ctid; i < p.M * groups; i += cthreads) {
            int m = i / groups, e = (i - m * groups) * 4;
            const XT * src = X + (int64_t)m * p.ldx + (int64_t)sb0 * 256 + e;
            float v0 = x_to_f32<XT>(src[0]), v1 = x_to_f32<XT>(src[1]), v2 = x_to_f32<XT>(src[2]),
                  v3 = x_to_f32<XT>(src[3]);
            __half2 a = __floats2half2_rn(v0, v2), b = __floats2half2_rn(v1, v3);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t *>(&a);
            pk.y = *reinterpret_cast<uint32_t *>(&b);
            int unit = e >> 6;
            *reinterpret_cast<uint2 *>(xs + (size_t)m * xstride + unit * 128 + unit_pos_of_group4(e & 63) * 2) = pk;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
    }

    const int g = lane >> 2, t = lane & 3;
    uint8_t * tab = tabs + warp * TAB_BYTES;
    const uint8_t * xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) xrow[j] = xs + (size_t)min(8 * j + g, p.M - 1) * xstride + t * 32;

    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[j][c] = 0.0f;
        const int row0 = tile * TILE_ROWS + warp * 16;
        bool ok = true;
        for (int ks = 0; ks < kstages; ks++, it++) {
            const int slot = it % stages;
            if (!mbar_wait(&full[slot], (it / stages) & 1, poison, 2)) { ok = false; break; }
            const int sbf = sb0 + ks * SBS;
            const int nsb_stage = min(SBS, sb1 - sbf);
            const uint8_t * stage = ring + (size_t)slot * STAGE_BYTES + (size_t)(warp * 16) * SLOT;
            auto row_ptr = [&](int r) {
                int grow = min(row0 + r, p.N - 1);
                uintptr_t gaddr = reinterpret_cast<uintptr_t>(p.w) + (uintptr_t)grow * p.rb + (uintptr_t)sbf * SB;
                return stage + (size_t)r * SLOT + (gaddr & 15);
            };
            {
                int r = lane & 15, sbi = lane >> 4;
                if (sbi < nsb_stage) decode_header<DT>(row_ptr(r) + sbi * SB, tab + (r * SBS + sbi) * TAB_STRIDE);
                if (SBS > 2) {
                    for (int s2 = 2 + sbi; s2 < nsb_stage; s2 += 2)
                        decode_header<DT>(row_ptr(r) + s2 * SB, tab + (r * SBS + s2) * TAB_STRIDE);
                }
            }
            __syncwarp();
            const uint8_t * rg = row_ptr(g);
            const uint8_t * rh = row_ptr(g + 8);
            for (int sbi = 0; sbi < nsb_stage; sbi++) {
                const uint8_t * blk_g = rg + sbi * SB;
                const uint8_t * blk_h = rh + sbi * SB;
                const uint8_t * tab_g = tab + (g * SBS + sbi) * TAB_STRIDE;
                const uint8_t * tab_h = tab + ((g + 8) * SBS + sbi) * TAB_STRIDE;
                const int unit0 = ((sbf - sb0) + sbi) * 4;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    uint32_t a[4][4];
                    decode_unit<DT>(blk_g, blk_h, tab_g, tab_h, u, t, a);
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        const uint4 b0 = *reinterpret_cast<const uint4 *>(xrow[j] + (unit0 + u) * 128);
                        const uint4 b1 = *reinterpret_cast<const uint4 *>(xrow[j] + (unit0 + u) * 128 + 16);
                        mma16816(acc[j], a[0], b0.x, b0.y);
                        mma16816(acc[j], a[1], b0.z, b0.w);
                        mma16816(acc[j], a[2], b1.x, b1.y);
                        mma16816(acc[j], a[3], b1.z, b1.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        if (!ok) break;

        // ---- epilogue ----
        const int n_g = row0 + g, n_h = n_g + 8;
        if (p.ksplit == 1) {
#pragma unroll
            for (int j = 0; j < NT; j++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    int tok = 8 * j + 2 * t + (c & 1), n = (c & 2) ? n_h : n_g;
                    if (tok < p.M && n < p.N) {
                        float * dst = p.out + (int64_t)tok * p.ldo + n;
                        *dst = p.accumulate ? *dst + acc[j][c] : acc[j][c];
                    }
                }
            }
        } else {
            float * part = p.partial + (size_t)blockIdx.y * p.M * p.N;
#pragma unroll
            for (int j = 0; j < NT; j++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    int tok = 8 * j + 2 * t + (c & 1), n = (c & 2) ? n_h : n_g;
                    if (tok < p.M && n < p.N) __stcg(part + (size_t)tok * p.N + n, acc[j][c]);
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            if (threadIdx.x == 0) {
                int old = atomicAdd(&p.counters[tile], 1);
                *last_flag = (old == p.ksplit - 1);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            if (*last_flag) {
                __threadfence();
                const int tile_row0 = tile * TILE_ROWS;
                for (int i = threadIdx.x; i < p.M * TILE_ROWS; i += NW * 32) {
                    int tok = i / TILE_ROWS, n = tile_row0 + (i - tok * TILE_ROWS);
                    if (n >= p.N) continue;
                    float s = 0.0f;
                    for (int q = 0; q < p.ksplit; q++) s += __ldcg(p.partial + ((size_t)q * p.M + tok) * p.N + n);
                    float * dst = p.out + (int64_t)tok * p.ldo + n;
                    *dst = p.accumulate ? *dst + s : s;
                }
                if (threadIdx.x == 0) p.counters[tile] = 0;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
        }
    }
}

struct MmaPlan {
    int nw, sbs, ksplit, nsb_part, stages, gx;
    size_t smem;
};

static int dtype_sb_bytes(uint32_t dt) {
    switch (dt) {
    case YUUKA_DTYPE_Q4_K: return 144;
    case YUUKA_DTYPE_Q5_K: return 176;
    case YUUKA_DTYPE_Q6_K: return 210;
    case YUUKA_DTYPE_Q8_0: return 272;
    default: return 0;
    }
}

// Tile and split choice for one launch of m (<= 32) activation rows.
static bool plan_mma(const yuuka_device * dev, uint32_t dtype, int n_out, int n_in, int m, MmaPlan & pl) {
    const int nw = n_out >= 4096 ? 8 : 4;
    const int sbs = (dtype == YUUKA_DTYPE_Q4_K || dtype == YUUKA_DTYPE_Q5_K) ? 2 : 1;
    const int slot = ((dtype_sb_bytes(dtype) * sbs + 30) / 16) * 16 + 16;
    const int tile_rows = nw * 16;
    const int nsb = n_in / 256;
    const int n_tiles = (n_out + tile_rows - 1) / tile_rows;
    const size_t limit = dev->prop.sharedMemPerBlockOptin;
    int want = (2 * dev->sm_count + n_tiles - 1) / n_tiles;
    int max_split = nsb / (sbs * 2) > 0 ? nsb / (sbs * 2) : 1;  // at least two stages per part
    int ksplit = want < 1 ? 1 : (want > max_split ? max_split : want);
    for (;; ksplit++) {
        int nsb_part = (nsb + ksplit - 1) / ksplit;
        int eff = (nsb + nsb_part - 1) / nsb_part;
        for (int stages = 4; stages >= 2; stages--) {
            size_t x = (((size_t)m * (nsb_part * 512 + 16) + 127) / 128) * 128;
            size_t sm = 256 + (size_t)nw * 16 * sbs * TAB_STRIDE + x + (size_t)stages * tile_rows * slot;
            if (sm <= limit) {
                pl.nw = nw; pl.sbs = sbs; pl.ksplit = eff; pl.nsb_part = nsb_part; pl.stages = stages; pl.smem = sm;
                int per = (dev->sm_count * (sm * 2 <= limit ? 2 : 1)) / eff;
                pl.gx = per < 1 ? 1 : (per > n_tiles ? n_tiles : per);
                return true;
            }
        }
        if (nsb_part == 1) return false;
    }
}

template <int DT, int NW, int SBS, int NT, typename XT>
static void launch_mma_inst(cudaStream_t stream, const GemmArgs & a, int m0, int m, const MmaPlan & pl) {
    static_assert(SlotBytes<DT, SBS>::value == ((BlockTraits<DT>::sb_bytes * SBS + 30) / 16) * 16 + 16, "slot size");
    auto kern = gemm_q_mma_kernel<DT, NW, SBS, NT, XT>;
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    MmaParams p;
    p.w = a.w;
    p.rb = (int64_t)row_bytes(a.w_dtype, a.n_in);
    p.N = a.n_out;
    p.K = a.n_in;
    p.x = (const XT *)a.x + (int64_t)m0 * a.ldx;
    p.ldx = a.ldx;
    p.M = m;
    p.out = a.out + (int64_t)m0 * a.ldo;
    p.ldo = a.ldo;
    p.accumulate = (a.flags & YUUKA_GEMM_ACCUMULATE) ? 1 : 0;
    p.ksplit = pl.ksplit;
    p.nsb_part = pl.nsb_part;
    p.stages = pl.stages;
    p.partial = a.scratch ? a.scratch->partial : nullptr;
    p.counters = a.scratch ? a.scratch->counters : nullptr;
    dim3 grid(pl.gx, pl.ksplit);
    kern<<<grid, (NW + 1) * 32, pl.smem, stream>>>(p);
    YK_CUDA(cudaGetLastError());
}

template <int DT, int NW, int SBS, typename XT>
static void launch_mma_nt(cudaStream_t stream, const GemmArgs & a, int m0, int m, const MmaPlan & pl) {
    if (m <= 8) launch_mma_inst<DT, NW, SBS, 1, XT>(stream, a, m0, m, pl);
    else if (m <= 16) launch_mma_inst<DT, NW, SBS, 2, XT>(stream, a, m0, m, pl);
    else launch_mma_inst<DT, NW, SBS, 4, XT>(stream, a, m0, m, pl);
}

template <int DT, int SBS, typename XT>
static int launch_mma_dt(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a) {
    int launches = 0;
    for (int m0 = 0; m0 < a.rows; m0 += 32) {
        int m = a.rows - m0 < 32 ? a.rows - m0 : 32;
        MmaPlan pl;
        YK_REQUIRE(plan_mma(dev, a.w_dtype, a.n_out, a.n_in, m, pl), YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant mma route: shape does not fit shared memory");
        if (pl.ksplit > 1) {
            YK_REQUIRE(a.scratch && a.scratch->partial_floats >= (uint64_t)pl.ksplit * m * a.n_out &&
                           a.scratch->counter_count >= (a.n_out + pl.nw * 16 - 1) / (pl.nw * 16),
                       YUUKA_ERR_INTERNAL, "gemm_quant: split-K scratch is too small");
        }
        if (pl.nw == 8) launch_mma_nt<DT, 8, SBS, XT>(stream, a, m0, m, pl);
        else launch_mma_nt<DT, 4, SBS, XT>(stream, a, m0, m, pl);
        launches++;
    }
    return launches;
}

template <typename XT>
static int launch_mma(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a) {
    switch (a.w_dtype) {
    case YUUKA_DTYPE_Q4_K: return launch_mma_dt<YUUKA_DTYPE_Q4_K, 2, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q5_K: return launch_mma_dt<YUUKA_DTYPE_Q5_K, 2, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q6_K: return launch_mma_dt<YUUKA_DTYPE_Q6_K, 1, XT>(dev, stream, a);
    case YUUKA_DTYPE_Q8_0: return launch_mma_dt<YUUKA_DTYPE_Q8_0, 1, XT>(dev, stream, a);
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "gemm_quant mma route: unsupported weight dtype %u", a.w_dtype);
    }
    return 0;
}

static bool mma_supported(const GemmArgs & a) {
    if (a.n_in % 256 != 0) return false;
    switch (a.w_dtype) {
    case YUUKA_DTYPE_Q4_K:
    case YUUKA_DTYPE_Q5_K:
        if (reinterpret_cast<uintptr_t>(a.w) % 16 != 0) return false;  // 16-byte table and header loads
        break;
    case YUUKA_DTYPE_Q6_K:
    case YUUKA_DTYPE_Q8_0:
        if (reinterpret_cast<uintptr_t>(a.w) % 2 != 0) return false;
        break;
    default: return false;
    }
    // the ring copies whole 16-byte lines: the line holding the last weight byte must be readable
    uintptr_t end = reinterpret_cast<uintptr_t>(a.w) + (uintptr_t)a.n_out * row_bytes(a.w_dtype, a.n_in);
    uintptr_t line_end = (end + 15) & ~(uintptr_t)15;
    return line_end <= reinterpret_cast<uintptr_t>(a.w) + a.w_readable;
}

uint32_t gemm_auto_path(uint32_t w_dtype, int rows, int n_in) {
    bool mma_dtype = w_dtype == YUUKA_DTYPE_Q4_K || w_dtype == YUUKA_DTYPE_Q5_K || w_dtype == YUUKA_DTYPE_Q6_K ||
                     w_dtype == YUUKA_DTYPE_Q8_0;
    if (!mma_dtype || n_in % 256 != 0) return YUUKA_GEMM_PATH_FP32;
    return rows <= 2 ? YUUKA_GEMM_PATH_FP32 : YUUKA_GEMM_PATH_MMA;
}

void gemm_scratch_reserve(const yuuka_device * dev, GemmScratch & s, uint32_t w_dtype, int rows, int n_out, int n_in) {
    set_device(dev);
    uint64_t want = 0;
    int tiles = 0;
    if (dtype_sb_bytes(w_dtype) != 0 && n_in % 256 == 0) {
        int m = rows < 32 ? rows : 32;
        MmaPlan pl;
        if (plan_mma(dev, w_dtype, n_out, n_in, m, pl) && pl.ksplit > 1) {
            want = (uint64_t)pl.ksplit * m * n_out;
            tiles = (n_out + pl.nw * 16 - 1) / (pl.nw * 16);
        }
    }
    if (want > s.partial_floats) {
        if (s.partial) cudaFree(s.partial);
        s.partial = nullptr;
        s.partial_floats = 0;
        cudaError_t err = cudaMalloc(&s.partial, want * sizeof(float));
        YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "gemm scratch allocation of %llu bytes failed",
                   (unsigned long long)(want * 4));
        s.partial_floats = want;
    }
    if (tiles > s.counter_count) {
        if (s.counters) cudaFree(s.counters);
        s.counters = nullptr;
        s.counter_count = 0;
        cudaError_t err = cudaMalloc(&s.counters, (size_t)tiles * sizeof(int));
        YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "gemm counter allocation failed");
        YK_CUDA(cudaMemset(s.counters, 0, (size_t)tiles * sizeof(int)));
        s.counter_count = tiles;
    }
}

void gemm_scratch_free(GemmScratch & s) {
    if (s.partial) cudaFree(s.partial);
    if (s.counters) cudaFree(s.counters);
    s = GemmScratch();
}

int launch_gemm_quant(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a) {
    YK_REQUIRE(a.w && a.x && a.out, YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: null operand");
    YK_REQUIRE(a.rows > 0 && a.n_out > 0 && a.n_in > 0, YUUKA_ERR_INVALID_ARGUMENT,
               "gemm_quant: invalid shape rows=%d n_out=%d n_in=%d", a.rows, a.n_out, a.n_in);
    uint64_t rb = row_bytes(a.w_dtype, a.n_in);
    YK_REQUIRE(rb > 0 && a.w_dtype != YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
               "gemm_quant: weight dtype %u does not fit a row of %d columns", a.w_dtype, a.n_in);
    YK_REQUIRE(a.n_in % 8 == 0, YUUKA_ERR_UNSUPPORTED, "gemm_quant: n_in %d is not a multiple of 8", a.n_in);
    YK_REQUIRE(a.x_dtype == YUUKA_DTYPE_F32 || a.x_dtype == YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
               "gemm_quant: activation dtype %u is not F32 or BF16", a.x_dtype);
    YK_REQUIRE(a.ldx >= a.n_in && a.ldo >= a.n_out, YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: leading dimension too small");
    uint32_t path = a.path == YUUKA_GEMM_PATH_AUTO ? gemm_auto_path(a.w_dtype, a.rows, a.n_in) : a.path;
    if (path == YUUKA_GEMM_PATH_MMA && !mma_supported(a)) {
        YK_REQUIRE(a.path == YUUKA_GEMM_PATH_AUTO, YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant: the mma route needs a K-quant or Q8_0 matrix with n_in %% 256 == 0, an aligned base "
                   "and 16 readable bytes after the last row");
        path = YUUKA_GEMM_PATH_FP32;
    }
    set_device(dev);
    if (path == YUUKA_GEMM_PATH_MMA) {
        return a.x_dtype == YUUKA_DTYPE_F32 ? launch_mma<float>(dev, stream, a) : launch_mma<__nv_bfloat16>(dev, stream, a);
    }
    YK_REQUIRE(path == YUUKA_GEMM_PATH_FP32, YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: unknown path %u", path);
    return a.x_dtype == YUUKA_DTYPE_F32 ? launch_fp32<float>(dev, stream, a) : launch_fp32<__nv_bfloat16>(dev, stream, a);
}

}  // namespace yk

// ---------------------------------------------------------------------------
// C ABI

namespace {
// one lazily grown scratch per device index for the kernel-level entry point
yk::GemmScratch g_scratch[16];
}  // namespace

extern "C" yuuka_status yuuka_gemm_quant(yuuka_stream * stream, yuuka_buffer * out, uint64_t out_offset,
                                         const yuuka_buffer * x, uint64_t x_offset, uint32_t x_dtype,
                                         const yuuka_buffer * w, uint64_t w_offset, uint32_t w_dtype, uint64_t n_in,
                                         uint64_t n_out, uint64_t rows, uint32_t path, uint32_t flags,
                                         yuuka_event * completion) {
    using namespace yk;
    return guard([&] {
        YK_REQUIRE(stream && out && x && w, YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: null argument");
        YK_REQUIRE(n_in > 0 && n_out > 0 && rows > 0 && n_in < (1u << 20) && n_out < (1u << 28) && rows <= 65536,
                   YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: invalid shape");
        uint64_t rb = row_bytes(w_dtype, n_in);
        YK_REQUIRE(rb > 0 && w_dtype != YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant: weight dtype %u does not fit a row of %llu columns", w_dtype, (unsigned long long)n_in);
        YK_REQUIRE(x_dtype == YUUKA_DTYPE_F32 || x_dtype == YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant: activation dtype %u is not F32 or BF16", x_dtype);
        uint64_t xb = rows * n_in * (x_dtype == YUUKA_DTYPE_F32 ? 4 : 2);
        YK_REQUIRE(w_offset <= w->bytes && n_out * rb <= w->bytes - w_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant: weight range exceeds the buffer");
        YK_REQUIRE(x_offset <= x->bytes && xb <= x->bytes - x_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant: activation range exceeds the buffer");
        YK_REQUIRE(out_offset <= out->bytes && rows * n_out * 4 <= out->bytes - out_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant: output range exceeds the buffer");
        YK_REQUIRE(x_offset % 16 == 0 && out_offset % 16 == 0, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant: activation and output offsets must be multiples of 16");
        yuuka_device * dev = stream->dev;
        YK_REQUIRE(dev->index >= 0 && dev->index < 16, YUUKA_ERR_UNSUPPORTED, "gemm_quant: device index out of range");
        GemmScratch & sc = g_scratch[dev->index];
        gemm_scratch_reserve(dev, sc, w_dtype, (int)rows, (int)n_out, (int)n_in);
        GemmArgs a;
        a.w = (const uint8_t *)w->ptr + w_offset;
        a.w_readable = w->bytes - w_offset;
        a.w_dtype = w_dtype;
        a.x = (const uint8_t *)x->ptr + x_offset;
        a.x_dtype = x_dtype;
        a.ldx = (int64_t)n_in;
        a.out = (float *)((uint8_t *)out->ptr + out_offset);
        a.ldo = (int64_t)n_out;
        a.rows = (int)rows;
        a.n_out = (int)n_out;
        a.n_in = (int)n_in;
        a.path = path;
        a.flags = flags;
        a.scratch = &sc;
        launch_gemm_quant(dev, stream->s, a);
        record_completion(stream, completion);
    });
}
