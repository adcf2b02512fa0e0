// Paged attention of the verify rows: every row attends to the committed
// positions of its sequence and to its own ancestors among the rows of the
// step (chain or tree), flash-decoding style: key ranges are split over CTAs,
// partial (max, sum, output) triples are merged, and the sigmoid output gate of
// the Qwen3.5 layout is applied (model/qwen35/forward.go:188-220; replaces
// attention_prefill_paged_f32_kernel, kernels/hip/prefill/prefill.hip:683).
//
// fp32 arithmetic on CUDA cores; K and V rows are decoded from the pool format.
#include <cuda_fp16.h>

#include <cfloat>
#include <cstdlib>

#include "layers.cuh"
#include "quant.cuh"
#include "xprep.cuh"

namespace yk {

constexpr int ATT_WARPS = 8;
constexpr int ATT_R = 5;                     // query rows per warp
constexpr int ATT_QT = ATT_WARPS * ATT_R;    // query rows per CTA
constexpr int ATT_KT = 32;                   // keys per tile (one per lane)

struct AttnParams {
    float * partial;
    const float * q;
    int ldq;
    int heads, kv_heads, splits, key_split;
    RowMeta rows;
    KvPool pool;
};

__device__ __forceinline__ void kv_decode8(const uint8_t * row, int format, int e8, float w[8]) {
    if (format == YUUKA_KV_F16) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(row + e8 * 16);
        const __half2 * h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            w[2 * i] = f.x;
            w[2 * i + 1] = f.y;
        }
    } else if (format == YUUKA_KV_F32) {
        const float4 * p = reinterpret_cast<const float4 *>(row + e8 * 32);
        float4 a = p[0], b = p[1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
        decode8<YUUKA_DTYPE_Q8_0>(row, e8, w);
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_partial_kernel(const AttnParams p) {
    pdl_entry();
    constexpr int KSTR = HD + 4;
    extern __shared__ __align__(16) float sm[];
    float * qs = sm;                       // [ATT_QT][HD]
    float * ks = qs + ATT_QT * HD;         // [ATT_KT][KSTR]
    float * vs = ks + ATT_KT * KSTR;       // [ATT_KT][HD]
    float * ps = vs + ATT_KT * HD;         // [ATT_QT][ATT_KT]

    const int seq = blockIdx.z;
    const int kvh = blockIdx.y % p.kv_heads, qt = blockIdx.y / p.kv_heads;
    const int split = blockIdx.x;
    const int G = p.heads / p.kv_heads, N = p.rows.nodes;
    const int sq = seq_of(p.rows, seq);
    const int pos0 = p.rows.pos0[sq];
    const int total = pos0 + N;
    const int k_begin = split * p.key_split;
    const int k_end = min(total, k_begin + p.key_split);
    const int nq = min(ATT_QT, G * N - qt * ATT_QT);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = (float)(1.0 / sqrt((double)HD));

    // query rows of this tile: local index qi -> (node, head)
    for (int i = threadIdx.x; i < nq * (HD / 4); i += blockDim.x) {
        int qi = i / (HD / 4), c = i - qi * (HD / 4);
        int gq = qt * ATT_QT + qi, node = gq / G, head = kvh * G + gq % G;
        const float4 * src = reinterpret_cast<const float4 *>(p.q + (int64_t)(seq * N + node) * p.ldq + (int64_t)head * 2 * HD);
        reinterpret_cast<float4 *>(qs + qi * HD)[c] = src[c];
    }

    float m[ATT_R], l[ATT_R], acc[ATT_R][HD / 32];
    uint64_t mask[ATT_R];
#pragma unroll
    for (int r = 0; r < ATT_R; r++) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int j = 0; j < HD / 32; j++) acc[r][j] = 0.0f;
        int qi = warp * ATT_R + r;
        int node = qi < nq ? (qt * ATT_QT + qi) / G : 0;
        mask[r] = qi < nq ? p.rows.anc_mask[seq * N + node] : 0;
    }

    for (int k0 = k_begin; k0 < k_end; k0 += ATT_KT) {
        __syncthreads();
        for (int i = threadIdx.x; i < ATT_KT * (HD / 8); i += blockDim.x) {
            int j = i / (HD / 8), c8 = i - j * (HD / 8);
            int pos = k0 + j;
            float kw[8], vw[8];
            if (pos < k_end) {
                int block = p.pool.tables[(int64_t)sq * p.pool.table_stride + pos / p.pool.block_size];
                int64_t off = ((int64_t)block * p.pool.block_size + pos % p.pool.block_size) * p.pool.row_bytes;
                kv_decode8(p.pool.k + off, p.pool.format, kvh * (HD / 8) + c8, kw);
                kv_decode8(p.pool.v + off, p.pool.format, kvh * (HD / 8) + c8, vw);
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) kw[e] = vw[e] = 0.0f;
            }
            float4 * kd = reinterpret_cast<float4 *>(ks + j * KSTR + c8 * 8);
            float4 * vd = reinterpret_cast<float4 *>(vs + j * HD + c8 * 8);
            kd[0] = make_float4(kw[0], kw[1], kw[2], kw[3]);
            kd[1] = make_float4(kw[4], kw[5], kw[6], kw[7]);
            vd[0] = make_float4(vw[0], vw[1], vw[2], vw[3]);
            vd[1] = make_float4(vw[4], vw[5], vw[6], vw[7]);
        }
        __syncthreads();

        // scores: lane = key
        float s[ATT_R];
#pragma unroll
        for (int r = 0; r < ATT_R; r++) s[r] = 0.0f;
        const float4 * kr = reinterpret_cast<const float4 *>(ks + lane * KSTR);
#pragma unroll 4
        for (int d4 = 0; d4 < HD / 4; d4++) {
            float4 kv = kr[d4];
#pragma unroll
            for (int r = 0; r < ATT_R; r++) {
                float4 qv = reinterpret_cast<const float4 *>(qs + (warp * ATT_R + r) * HD)[d4];
                s[r] = fmaf(qv.x, kv.x, s[r]);
                s[r] = fmaf(qv.y, kv.y, s[r]);
                s[r] = fmaf(qv.z, kv.z, s[r]);
                s[r] = fmaf(qv.w, kv.w, s[r]);
            }
        }
        const int pos = k0 + lane;
#pragma unroll
        for (int r = 0; r < ATT_R; r++) {
            const int qi = warp * ATT_R + r;
            bool vis = pos < k_end && qi < nq && (pos < pos0 || ((mask[r] >> (pos - pos0)) & 1ull));
            float sv = vis ? s[r] * scale : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float m_new = fmaxf(m[r], mx);
            float pr = 0.0f, corr = 1.0f;
            if (m_new != -INFINITY) {
                corr = expf(m[r] - m_new);
                pr = vis ? expf(sv - m_new) : 0.0f;
            }
            float ps_sum = pr;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ps_sum += __shfl_xor_sync(0xffffffffu, ps_sum, o);
            l[r] = l[r] * corr + ps_sum;
            m[r] = m_new;
#pragma unroll
            for (int j = 0; j < HD / 32; j++) acc[r][j] *= corr;
            ps[qi * ATT_KT + lane] = pr;
        }
        __syncwarp();
        // weighted values: lane owns dims lane + 32 j
#pragma unroll 4
        for (int kk = 0; kk < ATT_KT; kk++) {
            float vv[HD / 32];
#pragma unroll
            for (int j = 0; j < HD / 32; j++) vv[j] = vs[kk * HD + lane + 32 * j];
#pragma unroll
            for (int r = 0; r < ATT_R; r++) {
                float pr = ps[(warp * ATT_R + r) * ATT_KT + kk];
#pragma unroll
                for (int j = 0; j < HD / 32; j++) acc[r][j] = fmaf(pr, vv[j], acc[r][j]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < ATT_R; r++) {
        int qi = warp * ATT_R + r;
        if (qi >= nq) continue;
        int gq = qt * ATT_QT + qi, node = gq / G, head = kvh * G + gq % G;
        float * dst = p.partial + (((int64_t)(seq * N + node) * p.heads + head) * p.splits + split) * (HD + 2);
#pragma unroll
        for (int j = 0; j < HD / 32; j++) dst[lane + 32 * j] = acc[r][j];
        if (lane == 0) {
            dst[HD] = m[r];
            dst[HD + 1] = l[r];
        }
    }
}

// ---------------------------------------------------------------------------
// Tensor-core form of the partial kernel (mma.sync m16n8k16, fp16 operands, fp32 accumulate).
// A CTA of twelve warps covers up to 48 query rows (three blocks of 16) of one KV head and one key
// range; warp (rb, dq) owns row block rb and a quarter dq of the head dimension. The warps of a row
// block build the 16 x 32 score tile together, each over its quarter of the head dimension (queries
// as an fp16 hi + lo pair, so scores keep fp32-level accuracy; keys are exact when the pool stores
// F16 rows, otherwise they are split the same way), add the four partial tiles in one order, hence
// hold the same softmax statistics, and each multiplies the probabilities (fp16) with its own
// 16 x 32 x HD/4 slice of V, fetched with ldmatrix.trans.
constexpr int AM_KT = 32;
// Query rows per CTA: 16 per row block of four warps; three row blocks (a 9-row tree of four query heads per KV head
// fits), four when a sequence has more than 48 query rows per KV head (64 cover a 16-row tree in one pass over the keys).
constexpr int AM_RB_SMALL = 3, AM_RB_LARGE = 4;

// Row blocks per CTA for q_rows query rows of one KV head: whichever of the two sizes walks the keys with fewer
// row blocks in all (tiles x blocks per tile; the larger on a tie). 64 rows: one tile of four blocks; 68 rows (a
// 17-row tree of four query heads): two tiles of three blocks rather than two of four.
static int attention_row_blocks(int q_rows) {
    const int small = (q_rows + 16 * AM_RB_SMALL - 1) / (16 * AM_RB_SMALL) * AM_RB_SMALL;
    const int large = (q_rows + 16 * AM_RB_LARGE - 1) / (16 * AM_RB_LARGE) * AM_RB_LARGE;
    return small < large ? AM_RB_SMALL : AM_RB_LARGE;
}
int attention_query_tiles(int q_rows) {
    const int per = 16 * attention_row_blocks(q_rows);
    return (q_rows + per - 1) / per;
}

__device__ __forceinline__ void mma16816h(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// v as fp16 hi (returned) and the fp16 of the remainder
__device__ __forceinline__ __half split_half(float v, __half & lo) {
    const __half hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
    return hi;
}

template <int HD, bool KSPLIT, int RB>
__global__ void __launch_bounds__(RB * 128) attention_mma_kernel(const AttnParams p) {
    pdl_entry();
    constexpr int AM_ROWS = 16 * RB, AM_WARPS = 4 * RB;
    constexpr int STR = HD + 8;   // halves per shared-memory row: 16 bytes of padding spread the banks
    constexpr int DW = HD / 4;    // head dimensions per warp
    constexpr int NT_O = DW / 8;  // 8-column output tiles per warp
    extern __shared__ __align__(16) uint8_t smraw[];
    __half * qhi = reinterpret_cast<__half *>(smraw);
    __half * qlo = qhi + AM_ROWS * STR;
    __half * ks = qlo + AM_ROWS * STR;
    __half * kl = ks + AM_KT * STR;  // low parts of K (KSPLIT only)
    __half * vs = KSPLIT ? kl + AM_KT * STR : kl;
    float * sx = reinterpret_cast<float *>(vs + AM_KT * STR);  // [AM_WARPS][16][32] partial scores, see below

    const int seq = blockIdx.z;
    const int kvh = blockIdx.y % p.kv_heads, qt = blockIdx.y / p.kv_heads;
    const int split = blockIdx.x;
    const int G = p.heads / p.kv_heads, N = p.rows.nodes;
    const int sq = seq_of(p.rows, seq);
    const int pos0 = p.rows.pos0[sq];
    const int total = pos0 + N;
    const int k_begin = split * p.key_split;
    const int k_end = min(total, k_begin + p.key_split);
    const int nq = min(AM_ROWS, G * N - qt * AM_ROWS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rb = warp >> 2, dq = warp & 3;
    const float scale = (float)(1.0 / sqrt((double)HD));

    // queries of this tile as fp16 hi / lo; rows beyond nq are zero
    for (int i = threadIdx.x; i < AM_ROWS * (HD / 4); i += AM_WARPS * 32) {
        const int qi = i / (HD / 4), c = i - qi * (HD / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qi < nq) {
            const int gq = qt * AM_ROWS + qi, node = gq / G, head = kvh * G + gq % G;
            v = reinterpret_cast<const float4 *>(p.q + (int64_t)(seq * N + node) * p.ldq + (int64_t)head * 2 * HD)[c];
        }
        __half l0, l1, l2, l3;
        const __half h0 = split_half(v.x, l0), h1 = split_half(v.y, l1), h2 = split_half(v.z, l2), h3 = split_half(v.w, l3);
        __half2 * dh = reinterpret_cast<__half2 *>(qhi + qi * STR + c * 4);
        __half2 * dl = reinterpret_cast<__half2 *>(qlo + qi * STR + c * 4);
        dh[0] = __halves2half2(h0, h1);
        dh[1] = __halves2half2(h2, h3);
        dl[0] = __halves2half2(l0, l1);
        dl[1] = __halves2half2(l2, l3);
    }

    // the two query rows this lane holds in the accumulator layout: local rows rb*16 + g and + 8
    uint64_t mask[2];
    int row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = rb * 16 + g + 8 * h;
        row_ok[h] = qi < nq;
        const int node = row_ok[h] ? (qt * AM_ROWS + qi) / G : 0;
        mask[h] = row_ok[h] ? p.rows.anc_mask[seq * N + node] : 0ull;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int nt = 0; nt < NT_O; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) o[nt][c] = 0.0f;

    // F16 pool: the 16-byte pieces of the next key tile are fetched into registers while this one is multiplied
    constexpr int PIECES = AM_KT * (HD / 8);
    constexpr int PER = (PIECES + AM_WARPS * 32 - 1) / (AM_WARPS * 32);
    uint4 nk[PER], nv[PER];
    // (block sizes are powers of two in practice: a shift and a mask instead of two integer divisions per piece)
    const int bsz = p.pool.block_size, bshift = (bsz & (bsz - 1)) == 0 ? __ffs(bsz) - 1 : -1;
    auto fetch = [&](int k0) {
#pragma unroll
        for (int u = 0; u < PER; u++) {
            const int i = threadIdx.x + u * AM_WARPS * 32;
            const int j = i / (HD / 8), c8 = i - j * (HD / 8);
            const int pos = k0 + j;
            nk[u] = make_uint4(0, 0, 0, 0);
            nv[u] = nk[u];
            if (i < PIECES && pos < k_end) {
                const int bi = bshift >= 0 ? pos >> bshift : pos / bsz, within = bshift >= 0 ? pos & (bsz - 1) : pos - bi * bsz;
                const int block = p.pool.tables[(int64_t)sq * p.pool.table_stride + bi];
                const int64_t off = ((int64_t)block * bsz + within) * p.pool.row_bytes;
                nk[u] = *reinterpret_cast<const uint4 *>(p.pool.k + off + (size_t)(kvh * HD + c8 * 8) * 2);
                nv[u] = *reinterpret_cast<const uint4 *>(p.pool.v + off + (size_t)(kvh * HD + c8 * 8) * 2);
            }
        }
    };
    if (!KSPLIT && k_begin < k_end) fetch(k_begin);

    for (int k0 = k_begin; k0 < k_end; k0 += AM_KT) {
        __syncthreads();  // the previous tile has been consumed (and, first time, the queries are in place)
        if (!KSPLIT) {
#pragma unroll
            for (int u = 0; u < PER; u++) {
                const int i = threadIdx.x + u * AM_WARPS * 32;
                const int j = i / (HD / 8), c8 = i - j * (HD / 8);
                if (i < PIECES) {
                    *reinterpret_cast<uint4 *>(ks + j * STR + c8 * 8) = nk[u];
                    *reinterpret_cast<uint4 *>(vs + j * STR + c8 * 8) = nv[u];
                }
            }
            if (k0 + AM_KT < k_end) fetch(k0 + AM_KT);
        } else {
            for (int i = threadIdx.x; i < PIECES; i += AM_WARPS * 32) {
                const int j = i / (HD / 8), c8 = i - j * (HD / 8);
                const int pos = k0 + j;
                uint4 kh4 = make_uint4(0, 0, 0, 0), kl4 = kh4, vh4 = kh4;
                if (pos < k_end) {
                    const int block = p.pool.tables[(int64_t)sq * p.pool.table_stride + pos / p.pool.block_size];
                    const int64_t off = ((int64_t)block * p.pool.block_size + pos % p.pool.block_size) * p.pool.row_bytes;
                    float kw[8], vw[8];
                    kv_decode8(p.pool.k + off, p.pool.format, kvh * (HD / 8) + c8, kw);
                    kv_decode8(p.pool.v + off, p.pool.format, kvh * (HD / 8) + c8, vw);
                    __half hh[8], ll[8], vv[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        hh[e] = split_half(kw[e], ll[e]);
                        vv[e] = __float2half_rn(vw[e]);
                    }
                    kh4 = *reinterpret_cast<const uint4 *>(hh);
                    kl4 = *reinterpret_cast<const uint4 *>(ll);
                    vh4 = *reinterpret_cast<const uint4 *>(vv);
                }
                *reinterpret_cast<uint4 *>(ks + j * STR + c8 * 8) = kh4;
                *reinterpret_cast<uint4 *>(kl + j * STR + c8 * 8) = kl4;
                *reinterpret_cast<uint4 *>(vs + j * STR + c8 * 8) = vh4;
            }
        }
        __syncthreads();

        // scores of this warp's 16 rows against the 32 keys
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int c = 0; c < 4; c++) s[nt][c] = 0.0f;
        const __half * qh_row = qhi + (rb * 16 + g) * STR + 2 * t;
        const __half * ql_row = qlo + (rb * 16 + g) * STR + 2 * t;
        // the four warps of a row block share the head dimensions of the score product: each multiplies its
        // quarter, the partial tiles meet in shared memory and every warp adds them in the same order (each
        // warp redoing the whole product kept the tensor pipe busy four times as long)
        constexpr int KQ = HD / 16 / 4;
#pragma unroll
        for (int kq = 0; kq < KQ; kq++) {
            const int kk = dq * KQ + kq;
            uint32_t ah[4], al[4];
            ah[0] = *reinterpret_cast<const uint32_t *>(qh_row + 16 * kk);
            ah[1] = *reinterpret_cast<const uint32_t *>(qh_row + 8 * STR + 16 * kk);
            ah[2] = *reinterpret_cast<const uint32_t *>(qh_row + 16 * kk + 8);
            ah[3] = *reinterpret_cast<const uint32_t *>(qh_row + 8 * STR + 16 * kk + 8);
            al[0] = *reinterpret_cast<const uint32_t *>(ql_row + 16 * kk);
            al[1] = *reinterpret_cast<const uint32_t *>(ql_row + 8 * STR + 16 * kk);
            al[2] = *reinterpret_cast<const uint32_t *>(ql_row + 16 * kk + 8);
            al[3] = *reinterpret_cast<const uint32_t *>(ql_row + 8 * STR + 16 * kk + 8);
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const __half * kr = ks + (8 * nt + g) * STR + 16 * kk + 2 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(kr), b1 = *reinterpret_cast<const uint32_t *>(kr + 8);
                mma16816h(s[nt], ah, b0, b1);
                mma16816h(s[nt], al, b0, b1);
                if (KSPLIT) {
                    const __half * lr = kl + (8 * nt + g) * STR + 16 * kk + 2 * t;
                    mma16816h(s[nt], ah, *reinterpret_cast<const uint32_t *>(lr), *reinterpret_cast<const uint32_t *>(lr + 8));
                }
            }
        }
        {
            float * mine = sx + warp * 512;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int c = 0; c < 4; c++) mine[(nt * 4 + c) * 32 + lane] = s[nt][c];
            asm volatile("bar.sync %0, 128;" ::"r"(rb + 1) : "memory");
            const float * blk = sx + rb * 4 * 512;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int at = (nt * 4 + c) * 32 + lane;
                    s[nt][c] = ((blk[at] + blk[512 + at]) + blk[1024 + at]) + blk[1536 + at];
                }
        }
        // mask, online softmax; s[nt][0,1] -> row g, keys 8 nt + 2 t + {0,1}; s[nt][2,3] -> row g + 8
        uint32_t pa[2][4];  // probabilities as A fragments of the two 16-key steps
        // a tile that lies entirely in the committed context is visible to every row: no mask, no range test
        const bool plain_tile = k0 + AM_KT <= min(pos0, k_end);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float sv[4][2];
            float mx = -INFINITY;
            if (plain_tile) {
#pragma unroll
                for (int nt = 0; nt < 4; nt++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        sv[nt][e] = row_ok[h] ? s[nt][2 * h + e] * scale : -INFINITY;
                        mx = fmaxf(mx, sv[nt][e]);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < 4; nt++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int pos = k0 + 8 * nt + 2 * t + e;
                        const bool vis = pos < k_end && row_ok[h] && (pos < pos0 || ((mask[h] >> (pos - pos0)) & 1ull));
                        sv[nt][e] = vis ? s[nt][2 * h + e] * scale : -INFINITY;
                        mx = fmaxf(mx, sv[nt][e]);
                    }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[h], mx);
            float corr = 1.0f, sum = 0.0f;
            float pr[4][2];
            if (m_new != -INFINITY) corr = __expf(m[h] - m_new);
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    // (ex2.approx: the value is rounded to fp16 on the next line, 2^-11 against the approximation's 2^-22)
                    const float pv = (m_new != -INFINITY && sv[nt][e] != -INFINITY) ? __expf(sv[nt][e] - m_new) : 0.0f;
                    pr[nt][e] = __half2float(__float2half_rn(pv));  // the value the tensor core will see
                    sum += pr[nt][e];
                }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[h] = l[h] * corr + sum;
            m[h] = m_new;
#pragma unroll
            for (int nt = 0; nt < NT_O; nt++) {
                o[nt][2 * h] *= corr;
                o[nt][2 * h + 1] *= corr;
            }
            // A fragment registers: [0] row g / [1] row g+8 for keys 2t..; [2], [3] the same rows, keys 2t+8..
            pa[0][h] = pack_h2(pr[0][0], pr[0][1]);
            pa[0][2 + h] = pack_h2(pr[1][0], pr[1][1]);
            pa[1][h] = pack_h2(pr[2][0], pr[2][1]);
            pa[1][2 + h] = pack_h2(pr[3][0], pr[3][1]);
        }
        // O += P V on this warp's DW dimensions
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const __half * vrow = vs + (16 * kk + (lane & 15)) * STR + dq * DW;
#pragma unroll
            for (int nt = 0; nt < NT_O; nt++) {
                uint32_t b0, b1;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + 8 * nt);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma16816h(o[nt], pa[kk], b0, b1);
            }
        }
    }

#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (!row_ok[h]) continue;
        const int gq = qt * AM_ROWS + rb * 16 + g + 8 * h, node = gq / G, head = kvh * G + gq % G;
        float * dst = p.partial + (((int64_t)(seq * N + node) * p.heads + head) * p.splits + split) * (HD + 2);
#pragma unroll
        for (int nt = 0; nt < NT_O; nt++) {
            float2 v = make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
            *reinterpret_cast<float2 *>(dst + dq * DW + 8 * nt + 2 * t) = v;
        }
        if (dq == 0 && t == 0) {
            dst[HD] = m[h];
            dst[HD + 1] = l[h];
        }
    }
}

// float exp: the CPU reference evaluates exp in f64 and rounds; the difference is below 2e-7 relative
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }

// One CTA per (row, head): the split statistics are combined once in shared memory, then every thread
// sums its four output dims over the splits that saw a key (independent, coalesced loads), applies the
// sigmoid gate, and a 16-dim group leader writes the prepared form.
constexpr int MERGE_MAX_SPLITS = 1024;

template <int HD>
__global__ void __launch_bounds__(HD / 4 < 32 ? 32 : HD / 4) attention_merge_kernel(float * __restrict__ out, int ldo, const float * __restrict__ partial,
                                                                 const float * __restrict__ q, int ldq, int heads, int splits,
                                                                 XPrepOut prep) {
    pdl_entry();
    __shared__ float w_s[MERGE_MAX_SPLITS], l_s[MERGE_MAX_SPLITS];
    __shared__ float inv_l;
    const int r = blockIdx.x / heads, head = blockIdx.x - r * heads;
    const int tid = threadIdx.x;
    const float * base = partial + ((int64_t)r * heads + head) * splits * (HD + 2);
    constexpr int THREADS = HD / 4 < 32 ? 32 : HD / 4;  // whole warps; threads beyond HD / 4 only help with the statistics
    const bool has_dims = tid < HD / 4;
    // the split's running maximum and sum, all splits in flight at once (one lane summing them straight from
    // global memory was a chain of dependent L2 round trips: 12 us of this kernel at 23 splits)
    for (int s = tid; s < splits; s += THREADS) {
        const float2 ml = *reinterpret_cast<const float2 *>(base + (size_t)s * (HD + 2) + HD);
        w_s[s] = ml.x;
        l_s[s] = ml.y;
    }
    __syncthreads();
    if (tid < 32) {
        float M = -INFINITY;
        for (int s = tid; s < splits; s += 32) M = fmaxf(M, w_s[s]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        // weights exp(m_s - M); the normaliser is summed in split order by one lane, as the serial form did
        for (int s = tid; s < splits; s += 32) {
            const float ms = w_s[s];
            w_s[s] = ms == -INFINITY ? 0.0f : expf(ms - M);
        }
        __syncwarp();
        if (tid == 0) {
            float L = 0.0f;
            for (int s = 0; s < splits; s++)
                if (w_s[s] != 0.0f) L += l_s[s] * w_s[s];
            inv_l = L > 0.0f ? 1.0f / L : 0.0f;
        }
    }
    __syncthreads();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float * col = base + (has_dims ? tid : 0) * 4;
#pragma unroll 8
    for (int s = 0; s < splits; s++) {
        const float w = w_s[s];
        if (w == 0.0f) continue;
        const float2 lo = *reinterpret_cast<const float2 *>(col + (size_t)s * (HD + 2));
        const float2 hi = *reinterpret_cast<const float2 *>(col + (size_t)s * (HD + 2) + 2);
        acc.x = fmaf(lo.x, w, acc.x);
        acc.y = fmaf(lo.y, w, acc.y);
        acc.z = fmaf(hi.x, w, acc.z);
        acc.w = fmaf(hi.y, w, acc.w);
    }
    const float inv = inv_l;
    const float4 gate =
        *reinterpret_cast<const float4 *>(q + (int64_t)r * ldq + (int64_t)head * 2 * HD + HD + (has_dims ? tid : 0) * 4);
    float4 o;
    o.x = acc.x * inv * sigmoid_ref(gate.x);
    o.y = acc.y * inv * sigmoid_ref(gate.y);
    o.z = acc.z * inv * sigmoid_ref(gate.z);
    o.w = acc.w * inv * sigmoid_ref(gate.w);
    if (has_dims) *reinterpret_cast<float4 *>(out + (int64_t)r * ldo + head * HD + tid * 4) = o;
    if (prep.xh) {
        // gather the 16-dim group in its first lane (four neighbouring threads hold it)
        float v[16];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            v[4 * k] = __shfl_sync(0xffffffffu, o.x, (tid & 28) + k);
            v[4 * k + 1] = __shfl_sync(0xffffffffu, o.y, (tid & 28) + k);
            v[4 * k + 2] = __shfl_sync(0xffffffffu, o.z, (tid & 28) + k);
            v[4 * k + 3] = __shfl_sync(0xffffffffu, o.w, (tid & 28) + k);
        }
        if ((tid & 3) == 0 && has_dims) {
            const int cols = heads * HD, gq = head * (HD / 16) + (tid >> 2);
            xprep_store16(prep.xh + (int64_t)r * cols + gq * 16, prep.xl + (int64_t)r * cols + gq * 16, prep.xs16 + (int64_t)r * (cols >> 4) + gq, v);
        }
    }
}

size_t attention_scratch_floats(int rows, int heads, int head_dim, int splits) {
    return (size_t)rows * heads * splits * (head_dim + 2);
}

template <int HD>
static int launch_attention_hd(cudaStream_t s, float * out, int ldo, const float * q, int ldq, int heads, int kv_heads,
                               const RowMeta & rows, const KvPool & pool, const AttnScratch & sc, XPrepOut prep) {
    AttnParams p;
    p.partial = sc.partial;
    p.q = q;
    p.ldq = ldq;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.splits = sc.splits;
    p.key_split = sc.key_split;
    p.rows = rows;
    p.pool = pool;
    const int G = heads / kv_heads;
    static const bool use_mma = [] { const char * e = getenv("YUUKA_CUDA_ATTN_FP32"); return !(e && e[0] == '1'); }();
    if (use_mma) {
        // tensor-core partials; keys are taken as they are from an F16 pool and split into hi + lo otherwise
        const bool ksplit = pool.format != YUUKA_KV_F16;
        const int qtiles = attention_query_tiles(G * rows.nodes);
        const int rb = attention_row_blocks(G * rows.nodes);
        const size_t smem = sizeof(__half) * (size_t)(HD + 8) * (2 * 16 * rb + (ksplit ? 3 : 2) * AM_KT) +
                            sizeof(float) * 4 * rb * 512;
        auto kern = rb == AM_RB_LARGE ? (ksplit ? attention_mma_kernel<HD, true, AM_RB_LARGE> : attention_mma_kernel<HD, false, AM_RB_LARGE>)
                                      : (ksplit ? attention_mma_kernel<HD, true, AM_RB_SMALL> : attention_mma_kernel<HD, false, AM_RB_SMALL>);
        YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid(sc.splits, kv_heads * qtiles, rows.batch);
        launch_k(kern, grid, rb * 128, smem, s, p);
        YK_CUDA(cudaGetLastError());
    } else {
        const int qtiles = (G * rows.nodes + ATT_QT - 1) / ATT_QT;
        size_t smem = sizeof(float) * ((size_t)ATT_QT * HD + ATT_KT * (HD + 4) + ATT_KT * HD + ATT_QT * ATT_KT);
        auto kern = attention_partial_kernel<HD>;
        YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid(sc.splits, kv_heads * qtiles, rows.batch);
        launch_k(kern, grid, ATT_WARPS * 32, smem, s, p);
        YK_CUDA(cudaGetLastError());
    }
    YK_REQUIRE(sc.splits <= MERGE_MAX_SPLITS, YUUKA_ERR_UNSUPPORTED, "attention: %d key splits exceed the merge kernel's %d",
               sc.splits, MERGE_MAX_SPLITS);
    launch_k(attention_merge_kernel<HD>, rows.batch * rows.nodes * heads, HD / 4 < 32 ? 32 : HD / 4, 0, s, out, ldo, sc.partial, q, ldq, heads,
             sc.splits, prep);
    YK_CUDA(cudaGetLastError());
    return 2;
}

int launch_attention(cudaStream_t s, float * out, int ldo, const float * q, int ldq, int heads, int kv_heads,
                     int head_dim, const RowMeta & rows, const KvPool & pool, int max_total_keys,
                     const AttnScratch & scratch, XPrepOut prep) {
    YK_REQUIRE(rows.nodes <= 64, YUUKA_ERR_UNSUPPORTED, "attention: at most 64 rows per sequence");
    YK_REQUIRE((int64_t)scratch.splits * scratch.key_split >= max_total_keys, YUUKA_ERR_INTERNAL,
               "attention: key splits do not cover %d keys", max_total_keys);
    switch (head_dim) {
    case 64: return launch_attention_hd<64>(s, out, ldo, q, ldq, heads, kv_heads, rows, pool, scratch, prep);
    case 128: return launch_attention_hd<128>(s, out, ldo, q, ldq, heads, kv_heads, rows, pool, scratch, prep);
    case 256: return launch_attention_hd<256>(s, out, ldo, q, ldq, heads, kv_heads, rows, pool, scratch, prep);
    default: YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "attention: head_dim %d is not 64, 128 or 256", head_dim);
    }
    return 0;
}

}  // namespace yk
