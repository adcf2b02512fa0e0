// Row-wise kernels of the verify step: embedding gather, RMSNorm, SwiGLU
// product, and the attention front end (per-head norm, RoPE, paged KV write).
#include "layers.cuh"
#include "quant.cuh"
#include "xprep.cuh"

namespace yk {

// 16 consecutive floats of a row; four 16-byte loads when the address allows it.
__device__ __forceinline__ void load16(const float * __restrict__ p, float (&v)[16]) {
    if (((uintptr_t)p & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 q = reinterpret_cast<const float4 *>(p)[i];
            v[4 * i] = q.x;
            v[4 * i + 1] = q.y;
            v[4 * i + 2] = q.z;
            v[4 * i + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = p[i];
    }
}

// ---------------------------------------------------------------------------
// block-wide double sum

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ double block_sum_d(double v, double * red) {
    v = warp_sum_d(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = 0;
    for (int i = 0; i < nw; i++) t += red[i];
    __syncthreads();
    return t;
}

// rmsNorm (model/qwen35/forward.go:460-470) of one row by the whole CTA: f64 sum of squares, f32 mean,
// scale = f32(1/sqrt(f64(mean + eps))), dst = x * scale * weight, with the prepared (fp16 + group sums)
// form of dst for the GEMM that consumes it and, for GEMMs that fold the next norm in, the row's sum of
// squares in 2^-24 units.
__device__ void rmsnorm_row(float * __restrict__ dst_row, const float * __restrict__ x, const float * __restrict__ weight, int cols,
                            float eps, XPrepOut prep, unsigned long long * __restrict__ sumsq_out, int r, double * red) {
    double sum = 0;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) sum += (double)x[i] * (double)x[i];
    sum = block_sum_d(sum, red);
    if (sumsq_out && threadIdx.x == 0) sumsq_out[r] = (unsigned long long)(sum * 16777216.0);
    float mean = (float)(sum / (double)cols);
    float scale = (float)(1.0 / sqrt((double)(mean + eps)));
    if ((cols & 15) == 0) {
        for (int gq = threadIdx.x; gq < (cols >> 4); gq += blockDim.x) {
            float v[16], w[16];
            load16(x + gq * 16, v);
            load16(weight + gq * 16, w);
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = v[i] * scale * w[i];
            float4 * d = reinterpret_cast<float4 *>(dst_row + gq * 16);
#pragma unroll
            for (int i = 0; i < 4; i++) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            if (prep.xh) xprep_store16(prep.xh + (int64_t)r * cols + gq * 16, prep.xl + (int64_t)r * cols + gq * 16, prep.xs16 + (int64_t)r * (cols >> 4) + gq, v);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) dst_row[i] = x[i] * scale * weight[i];
    }
}

// ---------------------------------------------------------------------------
// embedding (replaces embedding_batch_f32_kernel, kernels/hip/prefill/prefill.hip:146)

// One CTA per row. With `first` set the CTA also does what the step's next two small kernels would do for
// the row: the first layer's input RMSNorm and the row's RoPE angles (forward.go:503-505, f64).
struct EmbedFirst {
    const float * norm_w = nullptr;  // null: embedding only
    float * xn = nullptr;
    int ldxn = 0;
    float eps = 0.0f;
    XPrepOut prep;
    unsigned long long * sumsq_out = nullptr;
    float2 * rope_cs = nullptr;      // null: no table
    RowMeta rows;
    int rope_dim = 0;
    double rope_base = 0.0;
};

__global__ void __launch_bounds__(256) embedding_kernel(float * __restrict__ x, int ldx, const uint8_t * __restrict__ table,
                                                        uint32_t dtype, int64_t rb, int hidden, int vocab,
                                                        const int32_t * __restrict__ tokens, const EmbedFirst first) {
    pdl_entry();
    __shared__ double red[32];
    const int r = blockIdx.x;
    int tok = tokens[r];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // ids are validated on the host
    const uint8_t * row = table + (int64_t)tok * rb;
    for (int e8 = threadIdx.x; e8 < hidden / 8; e8 += blockDim.x) {
        float w[8];
        switch (dtype) {
        case YUUKA_DTYPE_F32: decode8<YUUKA_DTYPE_F32>(row, e8, w); break;
        case YUUKA_DTYPE_F16: decode8<YUUKA_DTYPE_F16>(row, e8, w); break;
        case YUUKA_DTYPE_Q8_0: decode8<YUUKA_DTYPE_Q8_0>(row, e8, w); break;
        case YUUKA_DTYPE_Q4_K: decode8<YUUKA_DTYPE_Q4_K>(row, e8, w); break;
        case YUUKA_DTYPE_Q5_K: decode8<YUUKA_DTYPE_Q5_K>(row, e8, w); break;
        default: decode8<YUUKA_DTYPE_Q6_K>(row, e8, w); break;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) x[(int64_t)r * ldx + e8 * 8 + i] = w[i];
    }
    if (first.rope_cs) {
        const int seq = r / first.rows.nodes;
        const int pos = first.rows.pos0[seq_of(first.rows, seq)] + first.rows.depth[r];
        const int half = first.rope_dim / 2;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            double theta = (double)pos * pow(first.rope_base, -2.0 * (double)i / (double)first.rope_dim);
            first.rope_cs[(int64_t)r * half + i] = make_float2((float)cos(theta), (float)sin(theta));
        }
    }
    if (first.norm_w) {
        __syncthreads();  // the row just written is read back by other threads of this CTA
        rmsnorm_row(first.xn + (int64_t)r * first.ldxn, x + (int64_t)r * ldx, first.norm_w, hidden, first.eps, first.prep,
                    first.sumsq_out, r, red);
    }
}

void launch_embedding(cudaStream_t s, float * x, int ldx, const uint8_t * table, uint32_t dtype, int hidden, int vocab,
                      const int32_t * tokens, int rows) {
    launch_k(embedding_kernel, rows, 256, 0, s, x, ldx, table, dtype, (int64_t)row_bytes(dtype, hidden), hidden, vocab, tokens,
             EmbedFirst());
    YK_CUDA(cudaGetLastError());
}

// Embedding, the first layer's input norm and (rope_cs non-null) the rows' RoPE table in one launch. `table_rows` is the
// row layout the RoPE positions are counted in (for a wide prompt pass: its sub-chunks as sequences).
void launch_embedding_first(cudaStream_t s, float * x, int ldx, const uint8_t * table, uint32_t dtype, int hidden, int vocab,
                            const int32_t * tokens, int rows, const float * norm_w, float * xn, int ldxn, float eps, XPrepOut prep,
                            unsigned long long * sumsq_out, float2 * rope_cs, const RowMeta & table_rows, int rope_dim,
                            double rope_base) {
    YK_REQUIRE(!prep.xh || ((hidden & 15) == 0 && (ldxn & 3) == 0), YUUKA_ERR_UNSUPPORTED,
               "rmsnorm: prepared output needs a width that is a multiple of 16");
    EmbedFirst f;
    f.norm_w = norm_w;
    f.xn = xn;
    f.ldxn = ldxn;
    f.eps = eps;
    f.prep = prep;
    f.sumsq_out = sumsq_out;
    f.rope_cs = rope_cs;
    f.rows = table_rows;
    f.rope_dim = rope_dim;
    f.rope_base = rope_base;
    launch_k(embedding_kernel, rows, 256, 0, s, x, ldx, table, dtype, (int64_t)row_bytes(dtype, hidden), hidden, vocab, tokens, f);
    YK_CUDA(cudaGetLastError());
}

__global__ void rmsnorm_kernel(float * __restrict__ dst, int ldd, const float * __restrict__ src, int lds,
                               const float * __restrict__ weight, int cols, float eps, XPrepOut prep,
                               unsigned long long * __restrict__ sumsq_out) {
    pdl_entry();
    __shared__ double red[32];
    const int r = blockIdx.x;
    rmsnorm_row(dst + (int64_t)r * ldd, src + (int64_t)r * lds, weight, cols, eps, prep, sumsq_out, r, red);
}

void launch_rmsnorm(cudaStream_t s, float * dst, int ldd, const float * src, int lds, const float * weight, int cols,
                    int rows, float eps, XPrepOut prep, unsigned long long * sumsq_out) {
    YK_REQUIRE(!prep.xh || ((cols & 15) == 0 && (ldd & 3) == 0), YUUKA_ERR_UNSUPPORTED,
               "rmsnorm: prepared output needs a width that is a multiple of 16");
    launch_k(rmsnorm_kernel, rows, 256, 0, s, dst, ldd, src, lds, weight, cols, eps, prep, sumsq_out);
    YK_CUDA(cudaGetLastError());
}

// sigmoid / silu as the reference computes them: exp in f64 (forward.go:552-558)
// float exp: the CPU reference evaluates exp in f64 and rounds; the difference is below 2e-7 relative
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_ref(float x) { return x * sigmoid_ref(x); }

__global__ void silu_mul_kernel(float * __restrict__ act, int lda, const float * __restrict__ gate,
                                const float * __restrict__ up, int ld, int cols, XPrepOut prep, int gstride) {
    pdl_entry();
    const int r = blockIdx.y;
    for (int gq = blockIdx.x * blockDim.x + threadIdx.x; gq < (cols >> 4); gq += gridDim.x * blockDim.x) {
        float v[16], u[16];
        load16(gate + (int64_t)r * ld + gq * gstride, v);
        load16(up + (int64_t)r * ld + gq * gstride, u);
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = silu_ref(v[i]) * u[i];
        float4 * d = reinterpret_cast<float4 *>(act + (int64_t)r * lda + gq * 16);
#pragma unroll
        for (int i = 0; i < 4; i++) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        if (prep.xh) xprep_store16(prep.xh + (int64_t)r * cols + gq * 16, prep.xl + (int64_t)r * cols + gq * 16, prep.xs16 + (int64_t)r * (cols >> 4) + gq, v);
    }
}

// gstride: distance between consecutive 16-column groups of gate (and of up): 16 for plain rows, 32 when
// gate and up alternate 16 columns at a time in one row.
void launch_silu_mul(cudaStream_t s, float * act, int lda, const float * gate, const float * up, int ld, int cols,
                     int rows, XPrepOut prep, int gstride) {
    YK_REQUIRE((cols & 15) == 0 && (lda & 3) == 0, YUUKA_ERR_UNSUPPORTED, "silu_mul: width must be a multiple of 16");
    dim3 grid(((cols >> 4) + 127) / 128, rows);
    launch_k(silu_mul_kernel, grid, 128, 0, s, act, lda, gate, up, ld, cols, prep, gstride);
    YK_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// attention front end

struct PrepParams {
    float * q; int ldq;
    float * k; int ldk;
    const float * v; int ldv;
    const float * q_norm; const float * k_norm;
    int heads, kv_heads, hd, rope_dim;
    const float2 * rope_cs;  // [rows][rope_dim / 2] (cos, sin), see rope_table_kernel
    float eps;
    RowMeta rows;
    KvPool pool;
};

// rmsNormInPlace (forward.go:472-482) on hd values handled by one warp, then
// RoPE over the first rope_dim dims (forward.go:495-514) with the row's
// (cos, sin) table.
__device__ void norm_rope_head(float * x, const float * w, int hd, int rope_dim, const float2 * cs, float eps) {
    const int lane = threadIdx.x & 31;
    double sum = 0;
    for (int i = lane; i < hd; i += 32) sum += (double)x[i] * (double)x[i];
    sum = warp_sum_d(sum);
    float mean = (float)(sum / (double)hd);
    float scale = (float)(1.0 / sqrt((double)(mean + eps)));
    for (int i = lane; i < hd; i += 32) x[i] *= scale * w[i];
    __syncwarp();
    const int half = rope_dim / 2;
    for (int i = lane; i < half; i += 32) {
        const float c = cs[i].x, s = cs[i].y;
        float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x0 * s + x1 * c;
    }
    __syncwarp();
}

__device__ __forceinline__ int64_t kv_row_offset(const KvPool & pool, int seq, int slot) {
    int block = pool.tables[(int64_t)seq * pool.table_stride + slot / pool.block_size];
    return ((int64_t)block * pool.block_size + slot % pool.block_size) * pool.row_bytes;
}

// (cos, sin) of every row's RoPE angles, once per step: the rows keep their positions through all the
// attention layers. Angles in f64 as the reference computes them (forward.go:503-505).
__global__ void rope_table_kernel(float2 * __restrict__ cs, RowMeta rows, int rope_dim, double rope_base) {
    pdl_entry();
    const int r = blockIdx.x;
    const int seq = r / rows.nodes;
    const int pos = rows.pos0[seq_of(rows, seq)] + rows.depth[r];
    const int half = rope_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double theta = (double)pos * pow(rope_base, -2.0 * (double)i / (double)rope_dim);
        cs[(int64_t)r * half + i] = make_float2((float)cos(theta), (float)sin(theta));
    }
}

void launch_rope_table(cudaStream_t s, float2 * cs, const RowMeta & rows, int rope_dim, double rope_base) {
    launch_k(rope_table_kernel, rows.batch * rows.nodes, 64, 0, s, cs, rows, rope_dim, rope_base);
    YK_CUDA(cudaGetLastError());
}

// KVFormat.EncodeRow (model/qwen35/kv_format.go:75-131) for the n values of one head (n a multiple of
// 32), by one warp; dst is the row in the pool, first the head's first element. Q8_0 blocks are 32
// values, so a head's blocks are its own.
__device__ void kv_encode_head(uint8_t * row, int format, const float * src, int first, int n) {
    const int lane = threadIdx.x & 31;
    if (format == YUUKA_KV_F32) {
        float * d = reinterpret_cast<float *>(row) + first;
        for (int i = lane; i < n; i += 32) d[i] = src[i];
    } else if (format == YUUKA_KV_F16) {
        uint16_t * d = reinterpret_cast<uint16_t *>(row) + first;
        for (int i = lane; i < n; i += 32) d[i] = f32_to_f16_ref(src[i]);
    } else {
        for (int blk = 0; blk < n / 32; blk++) {
            const float v = src[blk * 32 + lane];
            float amax = fabsf(v);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float scale = amax / 127.0f;
            uint8_t * o = row + (first / 32 + blk) * 34;
            if (lane == 0) *reinterpret_cast<uint16_t *>(o) = f32_to_f16_ref(scale);
            int8_t q = 0;
            if (scale != 0.0f) q = (int8_t)(int)round((double)(v / scale));
            o[2 + lane] = (uint8_t)q;
        }
    }
}

// grid (rows, ceil((heads + 2 kv_heads) / 4)), one warp per unit of work: a query head (norm + RoPE in
// place), a key head (norm + RoPE, then its slice of the pool row) or a value head (its slice of the pool row).
__global__ void __launch_bounds__(128) attn_prep_kernel(const PrepParams p) {
    pdl_entry();
    const int r = blockIdx.x;
    const int seq = r / p.rows.nodes, node = r - seq * p.rows.nodes;
    const int sq = seq_of(p.rows, seq);
    const int unit = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= p.heads + 2 * p.kv_heads) return;
    const float2 * cs = p.rope_cs + (int64_t)r * (p.rope_dim / 2);
    // every row is stored at slot pos0 + node; the commit moves accepted rows of
    // a tree to their final positions
    if (unit < p.heads) {
        norm_rope_head(p.q + (int64_t)r * p.ldq + (int64_t)unit * 2 * p.hd, p.q_norm, p.hd, p.rope_dim, cs, p.eps);
    } else if (unit < p.heads + p.kv_heads) {
        const int h = unit - p.heads;
        float * k = p.k + (int64_t)r * p.ldk + (int64_t)h * p.hd;
        norm_rope_head(k, p.k_norm, p.hd, p.rope_dim, cs, p.eps);
        const int64_t off = kv_row_offset(p.pool, sq, p.rows.pos0[sq] + node);
        kv_encode_head(p.pool.k + off, p.pool.format, k, h * p.hd, p.hd);
    } else {
        const int h = unit - p.heads - p.kv_heads;
        const int64_t off = kv_row_offset(p.pool, sq, p.rows.pos0[sq] + node);
        kv_encode_head(p.pool.v + off, p.pool.format, p.v + (int64_t)r * p.ldv + (int64_t)h * p.hd, h * p.hd, p.hd);
    }
}

void launch_attn_prep(cudaStream_t s, float * q, int ldq, float * k, int ldk, const float * v, int ldv,
                      const float * q_norm, const float * k_norm, int heads, int kv_heads, int head_dim, int rope_dim,
                      const float2 * rope_cs, float eps, const RowMeta & rows, const KvPool & pool) {
    YK_REQUIRE(head_dim % 32 == 0 && rope_cs, YUUKA_ERR_UNSUPPORTED, "attn_prep: head width %d is not a multiple of 32", head_dim);
    PrepParams p{q, ldq, k, ldk, v, ldv, q_norm, k_norm, heads, kv_heads, head_dim, rope_dim, rope_cs, eps, rows, pool};
    dim3 grid(rows.batch * rows.nodes, (heads + 2 * kv_heads + 3) / 4);
    launch_k(attn_prep_kernel, grid, 128, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

}  // namespace yk
