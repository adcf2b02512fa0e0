// Paged attention of the verify rows: every row attends to the committed
// positions of its sequence and to its own ancestors among the rows of the
// step (chain or tree), flash-decoding style: key ranges are split over CTAs,
// partial (max, sum, output) triples are merged, and the sigmoid output gate of
// the Qwen3.5 layout is applied (model/qwen35/forward.go:188-220; replaces
// attention_prefill_paged_f32_kernel, kernels/hip/prefill/prefill.hip:683).
//
// fp32 arithmetic on CUDA cores; K and V rows are decoded from the pool format.
#include <cfloat>

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
    const int pos0 = p.rows.pos0[seq];
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
                int block = p.pool.tables[(int64_t)seq * p.pool.table_stride + pos / p.pool.block_size];
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

// float exp: the CPU reference evaluates exp in f64 and rounds; the difference is below 2e-7 relative
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }

// one thread per 16 consecutive output dims of one (row, head)
template <int HD>
__global__ void attention_merge_kernel(float * __restrict__ out, int ldo, const float * __restrict__ partial,
                                       const float * __restrict__ q, int ldq, int heads, int splits, XPrepOut prep) {
    pdl_entry();
    const int r = blockIdx.x;
    const int gq = threadIdx.x;  // 16-group within the row: head * (HD/16) + part
    if (gq >= heads * (HD / 16)) return;
    const int head = gq / (HD / 16), part = gq - head * (HD / 16);
    const float * base = partial + ((int64_t)r * heads + head) * splits * (HD + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) M = fmaxf(M, base[s * (HD + 2) + HD]);
    float L = 0.0f;
    float o[16];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i] = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float ms = base[s * (HD + 2) + HD];
        if (ms == -INFINITY) continue;
        const float w = expf(ms - M);
        L += base[s * (HD + 2) + HD + 1] * w;
        const float4 * src = reinterpret_cast<const float4 *>(base + s * (HD + 2) + part * 16);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 lo = reinterpret_cast<const float2 *>(src)[2 * i], hi = reinterpret_cast<const float2 *>(src)[2 * i + 1];
            o[4 * i] = fmaf(lo.x, w, o[4 * i]);
            o[4 * i + 1] = fmaf(lo.y, w, o[4 * i + 1]);
            o[4 * i + 2] = fmaf(hi.x, w, o[4 * i + 2]);
            o[4 * i + 3] = fmaf(hi.y, w, o[4 * i + 3]);
        }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    const float * gate = q + (int64_t)r * ldq + (int64_t)head * 2 * HD + HD + part * 16;
#pragma unroll
    for (int i = 0; i < 16; i++) o[i] = o[i] * inv * sigmoid_ref(gate[i]);
    float4 * d = reinterpret_cast<float4 *>(out + (int64_t)r * ldo + head * HD + part * 16);
#pragma unroll
    for (int i = 0; i < 4; i++) d[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
    const int cols = heads * HD;
    if (prep.xh) xprep_store16(prep.xh + (int64_t)r * cols + gq * 16, prep.xs16 + (int64_t)r * (cols >> 4) + gq, o);
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
    const int qtiles = (G * rows.nodes + ATT_QT - 1) / ATT_QT;
    size_t smem = sizeof(float) * ((size_t)ATT_QT * HD + ATT_KT * (HD + 4) + ATT_KT * HD + ATT_QT * ATT_KT);
    auto kern = attention_partial_kernel<HD>;
    YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(sc.splits, kv_heads * qtiles, rows.batch);
    launch_k(kern, grid, ATT_WARPS * 32, smem, s, p);
    YK_CUDA(cudaGetLastError());
    const int mthreads = ((heads * (HD / 16) + 31) / 32) * 32;
    YK_REQUIRE(mthreads <= 1024, YUUKA_ERR_UNSUPPORTED, "attention: too many heads for the merge kernel");
    launch_k(attention_merge_kernel<HD>, rows.batch * rows.nodes, mthreads, 0, s, out, ldo, sc.partial, q, ldq, heads, sc.splits, prep);
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
