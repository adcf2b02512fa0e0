/* CPU oracle for the yuuka speculative-decoding verify path. TEST
 * INFRASTRUCTURE ONLY: see yuuka_oracle.h for scope and parity status.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (oracle/Makefile).
 * -ffp-contract=off keeps every multiply and add separately rounded, which is
 * how the reference's float32 loops are written.
 *
 * Each function cites the reference file:line it restates.
 */
#include "yuuka_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;
void yo_set_threads(int n) { g_threads = n; }
int yo_get_threads(void) {
#ifdef _OPENMP
    return g_threads > 0 ? g_threads : omp_get_num_procs();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* binary16 codec: tensor/half.go:6-68                                       */

float yo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t mant = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            uint32_t e = 127 - 15 + 1;
            while ((mant & 0x400u) == 0) { mant <<= 1; e--; }
            bits = sign | (e << 23) | ((mant & 0x3ffu) << 13);
        }
    } else if (exp == 0x1f) {
        bits = sign | 0x7f800000u | (mant << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Rounds half-up on the 13 dropped mantissa bits (half.go:59), not ties-to-even. */
uint16_t yo_f32_to_f16(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xff) - 127;
    uint32_t mant = b & 0x7fffffu;
    if (exp == 128) return (uint16_t)(sign | (mant ? 0x7e00 : 0x7c00));
    if (exp > 15) return (uint16_t)(sign | 0x7c00);
    if (exp < -24) return sign;
    if (exp < -14) {
        uint32_t shift = (uint32_t)(-exp - 14);
        uint32_t full = mant | 0x800000u;
        uint32_t rounded = full + (1u << (shift + 12));
        return (uint16_t)(sign | (uint16_t)(rounded >> (shift + 13)));
    }
    uint32_t rounded = mant + 0x1000u;
    if (rounded & 0x800000u) {
        exp++;
        rounded = 0;
        if (exp > 15) return (uint16_t)(sign | 0x7c00);
    }
    return (uint16_t)(sign | (uint16_t)((exp + 15) << 10) | (uint16_t)(rounded >> 13));
}

static inline float rd_f16(const uint8_t *p) {
    return yo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
}
static inline float rd_f32(const uint8_t *p) {
    float f;
    memcpy(&f, p, 4);
    return f;
}

/* ------------------------------------------------------------------------- */
/* block layouts: tensor/dtype.go:102-171                                     */

static int block_layout(int dtype, int *elems, int *bytes) {
    switch (dtype) {
    case YO_F32: *elems = 1; *bytes = 4; return 0;
    case YO_F16: *elems = 1; *bytes = 2; return 0;
    case YO_Q4_0: *elems = 32; *bytes = 18; return 0;
    case YO_Q5_0: *elems = 32; *bytes = 22; return 0;
    case YO_Q8_0: *elems = 32; *bytes = 34; return 0;
    case YO_Q4_K: *elems = 256; *bytes = 144; return 0;
    case YO_Q5_K: *elems = 256; *bytes = 176; return 0;
    case YO_Q6_K: *elems = 256; *bytes = 210; return 0;
    default: return -1;
    }
}

int64_t yo_row_bytes(int dtype, int64_t cols) {
    int e, b;
    if (block_layout(dtype, &e, &b) != 0 || cols <= 0) return -1;
    if (e > 1 && cols % e != 0) return -1;
    return cols / e * b;
}

/* ------------------------------------------------------------------------- */
/* dequantizers: tensor/quant.go:64-158,261-285                               */

static void dq_q4_0(float *dst, const uint8_t *s) {
    float d = rd_f16(s);
    for (int j = 0; j < 16; j++) {
        dst[j] = d * (float)((int)(s[2 + j] & 0x0f) - 8);
        dst[j + 16] = d * (float)((int)(s[2 + j] >> 4) - 8);
    }
}

static void dq_q5_0(float *dst, const uint8_t *s) {
    float d = rd_f16(s);
    uint32_t qh = (uint32_t)s[2] | ((uint32_t)s[3] << 8) | ((uint32_t)s[4] << 16) | ((uint32_t)s[5] << 24);
    for (int j = 0; j < 16; j++) {
        uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10);
        uint8_t xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
        dst[j] = d * (float)((int)((s[6 + j] & 0x0f) | xh0) - 16);
        dst[j + 16] = d * (float)((int)((s[6 + j] >> 4) | xh1) - 16);
    }
}

static void dq_q8_0(float *dst, const uint8_t *s) {
    float d = rd_f16(s);
    for (int i = 0; i < 32; i++) dst[i] = d * (float)(int8_t)s[2 + i];
}

/* 6-bit scale/min unpack: quant.go:96-103 */
static void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

static void dq_q4_k(float *dst, const uint8_t *s) {
    float d = rd_f16(s), dm = rd_f16(s + 2);
    const uint8_t *scales = s + 4, *qs = s + 16;
    int is = 0;
    for (int j = 0; j < 256; j += 64) {
        uint8_t s0, m0, s1, m1;
        scale_min_k4(is, scales, &s0, &m0);
        scale_min_k4(is + 1, scales, &s1, &m1);
        float d1 = d * (float)s0, min1 = dm * (float)m0;
        float d2 = d * (float)s1, min2 = dm * (float)m1;
        for (int l = 0; l < 32; l++) {
            dst[j + l] = d1 * (float)(qs[l] & 0x0f) - min1;
            dst[j + 32 + l] = d2 * (float)(qs[l] >> 4) - min2;
        }
        qs += 32;
        is += 2;
    }
}

static void dq_q5_k(float *dst, const uint8_t *s) {
    float d = rd_f16(s), dm = rd_f16(s + 2);
    const uint8_t *scales = s + 4, *qh = s + 16, *ql = s + 48;
    int is = 0;
    for (int j = 0; j < 256; j += 64) {
        uint8_t s0, m0, s1, m1;
        scale_min_k4(is, scales, &s0, &m0);
        scale_min_k4(is + 1, scales, &s1, &m1);
        float d1 = d * (float)s0, min1 = dm * (float)m0;
        float d2 = d * (float)s1, min2 = dm * (float)m1;
        uint8_t bit0 = (uint8_t)(1u << (2 * (j / 64)));
        uint8_t bit1 = (uint8_t)(bit0 << 1);
        for (int l = 0; l < 32; l++) {
            int q0 = ql[l] & 0x0f;
            if (qh[l] & bit0) q0 += 16;
            int q1 = ql[l] >> 4;
            if (qh[l] & bit1) q1 += 16;
            dst[j + l] = d1 * (float)q0 - min1;
            dst[j + 32 + l] = d2 * (float)q1 - min2;
        }
        ql += 32;
        is += 2;
    }
}

static void dq_q6_k(float *dst, const uint8_t *s) {
    const uint8_t *ql = s, *qh = s + 128;
    const int8_t *sc = (const int8_t *)(s + 192);
    float d = rd_f16(s + 208);
    for (int n = 0; n < 2; n++) {
        const uint8_t *qln = ql + n * 64, *qhn = qh + n * 32;
        const int8_t *scn = sc + n * 8;
        float *o = dst + n * 128;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int8_t q1 = (int8_t)((qln[l] & 0x0f) | (((qhn[l] >> 0) & 3) << 4)) - 32;
            int8_t q2 = (int8_t)((qln[l + 32] & 0x0f) | (((qhn[l] >> 2) & 3) << 4)) - 32;
            int8_t q3 = (int8_t)((qln[l] >> 4) | (((qhn[l] >> 4) & 3) << 4)) - 32;
            int8_t q4 = (int8_t)((qln[l + 32] >> 4) | (((qhn[l] >> 6) & 3) << 4)) - 32;
            o[l] = d * (float)scn[is + 0] * (float)q1;
            o[l + 32] = d * (float)scn[is + 2] * (float)q2;
            o[l + 64] = d * (float)scn[is + 4] * (float)q3;
            o[l + 96] = d * (float)scn[is + 6] * (float)q4;
        }
    }
}

/* tensor/quant.go:15-62 */
int yo_dequantize_row(float *dst, int64_t dst_len, int dtype, const uint8_t *src, int64_t src_len) {
    int e, b;
    if (block_layout(dtype, &e, &b) != 0) return -1;
    if (src_len % b != 0) return -2;
    int64_t blocks = src_len / b;
    if (dst_len != blocks * e) return -3;
    for (int64_t i = 0; i < blocks; i++) {
        const uint8_t *s = src + i * b;
        float *o = dst + i * e;
        switch (dtype) {
        case YO_F32: *o = rd_f32(s); break;
        case YO_F16: *o = rd_f16(s); break;
        case YO_Q4_0: dq_q4_0(o, s); break;
        case YO_Q5_0: dq_q5_0(o, s); break;
        case YO_Q8_0: dq_q8_0(o, s); break;
        case YO_Q4_K: dq_q4_k(o, s); break;
        case YO_Q5_K: dq_q5_k(o, s); break;
        case YO_Q6_K: dq_q6_k(o, s); break;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* packed matvec: tensor/quant.go:341-466. Rows are split over threads the way
 * the reference splits them over goroutines; each output's summation order is
 * the sequential column order regardless of the thread count.               */

static void matmul_row(float *dst, const float *x, int batch, const uint8_t *src, int dtype,
                       int64_t rows, int64_t cols, int64_t row) {
    switch (dtype) {
    case YO_F32:
        for (int b = 0; b < batch; b++) {
            const float *xb = x + (int64_t)b * cols;
            float sum = 0;
            for (int64_t i = 0; i < cols; i++) sum += xb[i] * rd_f32(src + i * 4);
            dst[(int64_t)b * rows + row] = sum;
        }
        break;
    case YO_F16:
        for (int b = 0; b < batch; b++) {
            const float *xb = x + (int64_t)b * cols;
            float sum = 0;
            for (int64_t i = 0; i < cols; i++) sum += xb[i] * rd_f16(src + i * 2);
            dst[(int64_t)b * rows + row] = sum;
        }
        break;
    case YO_Q8_0:
        /* quant.go:404-415: sum += x * d * q, left to right */
        for (int b = 0; b < batch; b++) {
            const float *xb = x + (int64_t)b * cols;
            float sum = 0;
            for (int64_t blk = 0; blk < cols / 32; blk++) {
                const uint8_t *s = src + blk * 34;
                float d = rd_f16(s);
                for (int i = 0; i < 32; i++) sum += xb[blk * 32 + i] * d * (float)(int8_t)s[2 + i];
            }
            dst[(int64_t)b * rows + row] = sum;
        }
        break;
    case YO_Q4_0:
    case YO_Q5_0: {
        float values[32];
        int bb = dtype == YO_Q4_0 ? 18 : 22;
        for (int b = 0; b < batch; b++) {
            const float *xb = x + (int64_t)b * cols;
            float sum = 0;
            for (int64_t blk = 0; blk < cols / 32; blk++) {
                if (dtype == YO_Q4_0) dq_q4_0(values, src + blk * bb);
                else dq_q5_0(values, src + blk * bb);
                for (int i = 0; i < 32; i++) sum += xb[blk * 32 + i] * values[i];
            }
            dst[(int64_t)b * rows + row] = sum;
        }
        break;
    }
    default: {
        float values[256];
        int e, bb;
        block_layout(dtype, &e, &bb);
        for (int b = 0; b < batch; b++) {
            const float *xb = x + (int64_t)b * cols;
            float sum = 0;
            for (int64_t off = 0, si = 0; off < cols; off += 256, si += bb) {
                if (dtype == YO_Q4_K) dq_q4_k(values, src + si);
                else if (dtype == YO_Q5_K) dq_q5_k(values, src + si);
                else dq_q6_k(values, src + si);
                for (int i = 0; i < 256; i++) sum += xb[off + i] * values[i];
            }
            dst[(int64_t)b * rows + row] = sum;
        }
    }
    }
}

int yo_matmul(float *dst, const float *x, int batch, const uint8_t *w, int dtype, int64_t rows,
              int64_t cols) {
    int64_t rb = yo_row_bytes(dtype, cols);
    if (rb < 0 || rows <= 0 || batch <= 0) return -1;
    int threads = yo_get_threads();
    if (rows * rb < 64 * 1024) threads = 1; /* quant.go:347 */
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
    for (int64_t r = 0; r < rows; r++) matmul_row(dst, x, batch, w + r * rb, dtype, rows, cols, r);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* KV row codec: model/qwen35/kv_format.go:75-168                             */

int64_t yo_kv_row_bytes(int format, int kv_dim) {
    if (kv_dim <= 0) return -1;
    switch (format) {
    case YO_KV_F32: return (int64_t)kv_dim * 4;
    case YO_KV_F16: return (int64_t)kv_dim * 2;
    case YO_KV_Q8_0: return (int64_t)(kv_dim + 31) / 32 * 34;
    default: return -1;
    }
}

int yo_kv_encode_row(uint8_t *dst, int format, const float *src, int n) {
    switch (format) {
    case YO_KV_F32: memcpy(dst, src, (size_t)n * 4); return 0;
    case YO_KV_F16:
        for (int i = 0; i < n; i++) {
            uint16_t h = yo_f32_to_f16(src[i]);
            dst[i * 2] = (uint8_t)h;
            dst[i * 2 + 1] = (uint8_t)(h >> 8);
        }
        return 0;
    case YO_KV_Q8_0:
        for (int blk = 0; blk < (n + 31) / 32; blk++) {
            int start = blk * 32, end = start + 32 < n ? start + 32 : n;
            float max_abs = 0;
            for (int i = start; i < end; i++) {
                float a = (float)fabs((double)src[i]);
                if (a > max_abs) max_abs = a;
            }
            float scale = max_abs / 127;
            uint8_t *o = dst + blk * 34;
            uint16_t h = yo_f32_to_f16(scale);
            o[0] = (uint8_t)h;
            o[1] = (uint8_t)(h >> 8);
            for (int i = 0; i < 32; i++) {
                int8_t q = 0;
                /* Go's math.Round rounds half away from zero, as round() does. */
                if (start + i < end && scale != 0) q = (int8_t)round((double)(src[start + i] / scale));
                o[2 + i] = (uint8_t)q;
            }
        }
        return 0;
    default: return -1;
    }
}

int yo_kv_decode_row(float *dst, int format, const uint8_t *src, int n) {
    switch (format) {
    case YO_KV_F32: memcpy(dst, src, (size_t)n * 4); return 0;
    case YO_KV_F16:
        for (int i = 0; i < n; i++) dst[i] = rd_f16(src + i * 2);
        return 0;
    case YO_KV_Q8_0:
        for (int i = 0; i < n; i++) {
            const uint8_t *o = src + i / 32 * 34;
            dst[i] = rd_f16(o) * (float)(int8_t)o[2 + i % 32];
        }
        return 0;
    default: return -1;
    }
}

/* memory/memory.go:253-266 */
int yo_table_map(const int32_t *blocks, int n_blocks, int block_size, int pos, int32_t *block,
                 int32_t *offset) {
    if (pos < 0 || block_size <= 0) return -1;
    int index = pos / block_size;
    if (index >= n_blocks) return -2;
    *block = blocks[index];
    *offset = pos % block_size;
    return 0;
}

/* ------------------------------------------------------------------------- */
/* scalar helpers: model/qwen35/forward.go:460-565                            */

float yo_sigmoid(float x) { return 1.0f / (1.0f + (float)exp((double)-x)); }
float yo_silu(float x) { return x * yo_sigmoid(x); }
float yo_softplus(float x) {
    if (x > 20) return x;
    return (float)log1p(exp((double)x));
}

void yo_rms_norm(float *dst, const float *src, const float *weight, int n, float eps) {
    double sum = 0;
    for (int i = 0; i < n; i++) sum += (double)src[i] * (double)src[i];
    float mean = (float)(sum / (double)n);
    float scale = (float)(1.0 / sqrt((double)(mean + eps)));
    for (int i = 0; i < n; i++) dst[i] = src[i] * scale * weight[i];
}

static void rms_norm_inplace(float *x, const float *weight, int n, float eps) {
    double sum = 0;
    for (int i = 0; i < n; i++) sum += (double)x[i] * (double)x[i];
    float mean = (float)(sum / (double)n);
    float scale = (float)(1.0 / sqrt((double)(mean + eps)));
    /* forward.go:480 multiplies by (scale*weight), not scale then weight */
    for (int i = 0; i < n; i++) x[i] *= scale * weight[i];
}

void yo_l2_norm_head(float *x, int n, float eps, float extra) {
    double sum = 0;
    for (int i = 0; i < n; i++) sum += (double)x[i] * (double)x[i];
    float scale = (float)(1.0 / sqrt(sum + (double)eps)) * extra;
    for (int i = 0; i < n; i++) x[i] *= scale;
}

void yo_apply_rope(float *vec, int heads, int stride, int head_dim, int rot_dim, int pos, double base) {
    (void)head_dim;
    int half = rot_dim / 2;
    for (int i = 0; i < half; i++) {
        double theta = (double)pos * pow(base, -2 * (double)i / (double)rot_dim);
        float c = (float)cos(theta), s = (float)sin(theta);
        for (int h = 0; h < heads; h++) {
            int off = h * stride + i;
            float x0 = vec[off], x1 = vec[off + half];
            vec[off] = x0 * c - x1 * s;
            vec[off + half] = x0 * s + x1 * c;
        }
    }
}

void yo_softmax_inplace(float *x, int n) {
    if (n == 0) return;
    float mx = x[0];
    for (int i = 1; i < n; i++)
        if (x[i] > mx) mx = x[i];
    float sum = 0;
    for (int i = 0; i < n; i++) {
        float e = (float)exp((double)(x[i] - mx));
        x[i] = e;
        sum += e;
    }
    float inv = 1.0f / sum;
    for (int i = 0; i < n; i++) x[i] *= inv;
}

static float dotf(const float *a, const float *b, int n) {
    float sum = 0;
    for (int i = 0; i < n; i++) sum += a[i] * b[i];
    return sum;
}

/* model/qwen35/recurrent.go:56-105 */
void yo_gdn_per_token_scan(float *state, const float *conv, const float *alpha, const float *beta,
                           float *out, int rows, int groups, int rank, int S, int conv_dim) {
    int key_dim = groups * S;
    float *sk = (float *)malloc(sizeof(float) * (size_t)S * 2);
    float *d = sk + S;
    for (int r = 0; r < rows; r++) {
        const float *row = conv + (int64_t)r * conv_dim;
        for (int h = 0; h < rank; h++) {
            int kh = h % groups;
            const float *q = row + kh * S;
            const float *k = row + key_dim + kh * S;
            const float *v = row + 2 * key_dim + h * S;
            float *mat = state + (int64_t)h * S * S;
            float decay = (float)exp((double)alpha[r * rank + h]);
            for (int i = 0; i < S * S; i++) mat[i] *= decay;
            for (int j = 0; j < S; j++) sk[j] = 0;
            for (int i = 0; i < S; i++) {
                float ki = k[i];
                const float *mrow = mat + i * S;
                for (int j = 0; j < S; j++) sk[j] += mrow[j] * ki;
            }
            float b = beta[r * rank + h];
            for (int j = 0; j < S; j++) d[j] = (v[j] - sk[j]) * b;
            for (int i = 0; i < S; i++) {
                float ki = k[i];
                float *mrow = mat + i * S;
                for (int j = 0; j < S; j++) mrow[j] += ki * d[j];
            }
            float *head = out + ((int64_t)r * rank + h) * S;
            for (int j = 0; j < S; j++) head[j] = 0;
            for (int i = 0; i < S; i++) {
                float qi = q[i];
                const float *mrow = mat + i * S;
                for (int j = 0; j < S; j++) head[j] += mrow[j] * qi;
            }
        }
    }
    free(sk);
}

/* gdnChunkedScan, model/qwen35/recurrent.go:107-351: the same recurrence in the chunkwise WY form, chunks of
 * YO_GDN_CHUNK = 32 rows (recurrent.go:8). Within a chunk, relative to the state S_0 at its start, with g the
 * cumulative log decay from the chunk start and g_c its last entry:
 *   M = I + B, B[r][s] = beta_r (k_r . k_s) for s < r;  Z = (Q K^T on the lower triangle) M^-1
 *   S_C = exp(g_c) S_0 + K^T (M^-1 diag(beta) (exp(g_c - g) V - exp(g_c) K S_0))
 *   o_r = exp(g_r) (q_r S_0 + z_r (diag(beta exp(-g)) V - M^-1 diag(beta) K S_0))
 * The summation orders of the reference are kept (inverse by rows, recurrent.go:307-331; triangular products,
 * recurrent.go:335-351). */
#define YO_GDN_CHUNK 32
static void gdn_chunk_head(float *matrix, const float *conv, const float *alpha, const float *beta, float *out,
                           int c0, int n, int h, int groups, int rank, int S, int conv_dim, float *scratch) {
    const int C = YO_GDN_CHUNK;
    const int kh = h % groups, key_dim = groups * S;
    const float *qbase = conv + (int64_t)c0 * conv_dim + kh * S;
    const float *kbase = conv + (int64_t)c0 * conv_dim + key_dim + kh * S;
    const float *vbase = conv + (int64_t)c0 * conv_dim + 2 * key_dim + h * S;
#define QROW(r) (qbase + (int64_t)(r) * conv_dim)
#define KROW(r) (kbase + (int64_t)(r) * conv_dim)
#define VROW(r) (vbase + (int64_t)(r) * conv_dim)
#define BETA(r) (beta[(int64_t)(c0 + (r)) * rank + h])
    float *lower = scratch;            /* [C][C], later Z */
    float *minv = lower + C * C;       /* [C][C] */
    float *logd = minv + C * C;        /* [C] */
    float *prow = logd + C;            /* [C] */
    float *kp = prow + C;              /* [C][S]  K S_0 */
    float *qp = kp + C * S;            /* [C][S]  Q S_0 */
    float *work = qp + C * S;          /* [C][S] */
    float *ref = work + C * S;         /* [C][S] */
    float *tmp = ref + C * S;          /* [S] */

    float acc = 0;
    for (int r = 0; r < n; r++) {
        acc += alpha[(int64_t)(c0 + r) * rank + h];
        logd[r] = acc;
    }
    const float gc = acc;
    const float decay = (float)exp((double)gc);

    for (int i = 0; i < C * C; i++) lower[i] = 0;
    for (int r = 0; r < n; r++) {
        const float br = BETA(r);
        for (int s = 0; s < r; s++) lower[r * C + s] = br * dotf(KROW(r), KROW(s), S);
    }
    /* (I + lower)^-1, recurrent.go:307-331 */
    for (int r = 0; r < n; r++) {
        for (int s = 0; s < n; s++) minv[r * C + s] = 0;
        minv[r * C + r] = 1;
    }
    for (int r = 1; r < n; r++)
        for (int u = 0; u < r; u++) {
            const float lu = lower[r * C + u];
            if (lu == 0) continue;
            for (int s = 0; s <= u; s++) minv[r * C + s] -= lu * minv[u * C + s];
        }
    /* Z over the block of lower */
    float *zm = lower;
    for (int r = 0; r < n; r++) {
        for (int s = 0; s <= r; s++) prow[s] = dotf(QROW(r), KROW(s), S);
        for (int s = 0; s <= r; s++) {
            float sum = 0;
            for (int u = s; u <= r; u++) sum += prow[u] * minv[u * C + s];
            zm[r * C + s] = sum;
        }
    }
    for (int r = 0; r < n; r++)
        for (int s = 0; s < n; s++) minv[r * C + s] *= BETA(s);

    for (int r = 0; r < n; r++) {
        float *krow = kp + r * S, *qrow = qp + r * S;
        for (int j = 0; j < S; j++) krow[j] = qrow[j] = 0;
        for (int i = 0; i < S; i++) {
            const float ki = KROW(r)[i], qi = QROW(r)[i];
            const float *srow = matrix + i * S;
            for (int j = 0; j < S; j++) {
                krow[j] += ki * srow[j];
                qrow[j] += qi * srow[j];
            }
        }
    }
    for (int r = 0; r < n; r++) {
        const float scale = (float)exp((double)(gc - logd[r]));
        for (int j = 0; j < S; j++) work[r * S + j] = scale * VROW(r)[j] - decay * kp[r * S + j];
    }
    /* ref = mb work, recurrent.go:335-351 */
    for (int r = 0; r < n; r++) {
        for (int j = 0; j < S; j++) tmp[j] = 0;
        for (int s = 0; s <= r; s++) {
            const float coef = minv[r * C + s];
            if (coef == 0) continue;
            for (int j = 0; j < S; j++) tmp[j] += coef * work[s * S + j];
        }
        memcpy(ref + r * S, tmp, sizeof(float) * (size_t)S);
    }
    for (int i = 0; i < S * S; i++) matrix[i] *= decay;
    for (int r = 0; r < n; r++)
        for (int i = 0; i < S; i++) {
            const float ki = KROW(r)[i];
            float *srow = matrix + i * S;
            for (int j = 0; j < S; j++) srow[j] += ki * ref[r * S + j];
        }
    for (int r = 0; r < n; r++) {
        const float br = BETA(r);
        const float scale = (float)exp((double)(-logd[r]));
        for (int j = 0; j < S; j++) work[r * S + j] = br * (scale * VROW(r)[j] - kp[r * S + j]);
    }
    for (int r = 0; r < n; r++) {
        float *orow = ref + r * S;
        for (int j = 0; j < S; j++) orow[j] = 0;
        for (int s = 0; s <= r; s++) {
            const float zs = zm[r * C + s];
            for (int j = 0; j < S; j++) orow[j] += zs * work[s * S + j];
        }
    }
    for (int r = 0; r < n; r++) {
        const float scale = (float)exp((double)logd[r]);
        float *head = out + ((int64_t)(c0 + r) * rank + h) * S;
        for (int j = 0; j < S; j++) head[j] = scale * (qp[r * S + j] + ref[r * S + j]);
    }
#undef QROW
#undef KROW
#undef VROW
#undef BETA
}

void yo_gdn_chunked_scan(float *state, const float *conv, const float *alpha, const float *beta, float *out,
                         int rows, int groups, int rank, int S, int conv_dim) {
    const int C = YO_GDN_CHUNK;
    float *scratch = (float *)malloc(sizeof(float) * ((size_t)2 * C * C + 2 * C + (size_t)4 * C * S + S));
    for (int c0 = 0; c0 < rows; c0 += C) {
        const int n = rows - c0 < C ? rows - c0 : C;
        for (int h = 0; h < rank; h++)
            gdn_chunk_head(state + (int64_t)h * S * S, conv, alpha, beta, out, c0, n, h, groups, rank, S, conv_dim, scratch);
    }
    free(scratch);
}

/* model/qwen35/recurrent.go:39-50 */
void yo_gdn_norm_gate(float *out, const float *z, const float *norm, int rows, int rank, int S,
                      float eps) {
    for (int r = 0; r < rows; r++)
        for (int h = 0; h < rank; h++) {
            float *row = out + ((int64_t)r * rank + h) * S;
            const float *gate = z + ((int64_t)r * rank + h) * S;
            rms_norm_inplace(row, norm, S, eps);
            for (int d = 0; d < S; d++) row[d] *= yo_silu(gate[d]);
        }
}

/* model/qwen35/forward.go:393-439: repeated argmax, lowest index wins ties,
 * softmax over the selected logits only. */
void yo_select_experts(const float *logits, int n, int32_t *ids, float *weights, int k) {
    for (int slot = 0; slot < k; slot++) {
        int best = -1;
        for (int e = 0; e < n; e++) {
            int used = 0;
            for (int p = 0; p < slot; p++)
                if (ids[p] == e) { used = 1; break; }
            if (used) continue;
            if (best < 0 || logits[e] > logits[best]) best = e;
        }
        if (best < 0) { ids[slot] = 0; weights[slot] = 0; continue; }
        ids[slot] = best;
    }
    if (k == 0) return;
    float mx = logits[ids[0]];
    for (int s = 1; s < k; s++)
        if (logits[ids[s]] > mx) mx = logits[ids[s]];
    float total = 0;
    for (int s = 0; s < k; s++) {
        float w = (float)exp((double)(logits[ids[s]] - mx));
        weights[s] = w;
        total += w;
    }
    if (total > 0)
        for (int s = 0; s < k; s++) weights[s] /= total;
}

/* ------------------------------------------------------------------------- */
/* model: model/qwen35/load.go:60-215                                         */

typedef struct {
    const uint8_t *data;
    int dtype;
    int64_t rows, cols;
} yo_mat;

typedef struct {
    const float *attn_norm, *post_norm;
    /* full attention */
    yo_mat q, k, v, o;
    const float *q_norm, *k_norm;
    /* recurrent */
    yo_mat qkv, gate, out, beta, alpha;
    const float *conv, *dt, *a, *ssm_norm;
    /* dense ffn */
    yo_mat ffn_gate, ffn_up, ffn_down;
    /* moe */
    yo_mat router, sh_gate, sh_up, sh_down, gate_exps, up_exps, down_exps;
    const float *sh_gate_inp;
} yo_layer;

struct yo_model {
    yo_config cfg;
    yo_mat embedding, output;
    int has_output;
    const float *output_norm;
    yo_layer *layers;
};

int yo_is_recurrent(const yo_config *c, int layer) { return (layer + 1) % c->full_attention_interval != 0; }

/* model/qwen35/config.go:231-276 */
int yo_config_validate(const yo_config *c, char *msg, size_t n) {
#define FAIL(...) do { if (msg) snprintf(msg, n, __VA_ARGS__); return -1; } while (0)
    if (c->kv_heads <= 0 || c->heads % c->kv_heads != 0)
        FAIL("head count %d is not a multiple of KV head count %d", c->heads, c->kv_heads);
    if (c->rope_dim % 2 != 0 || c->rope_dim > c->head_dim)
        FAIL("invalid RoPE dimension %d for head dim %d", c->rope_dim, c->head_dim);
    if (c->full_attention_interval <= 0) FAIL("full attention interval must be positive");
    if (c->inner_size != c->time_step_rank * c->state_size)
        FAIL("ssm inner size %d != time_step_rank %d * state_size %d", c->inner_size,
             c->time_step_rank, c->state_size);
    if (c->conv_kernel < 2) FAIL("invalid ssm conv kernel %d", c->conv_kernel);
    if (c->expert_count > 0) {
        if (c->expert_used <= 0 || c->expert_used > c->expert_count)
            FAIL("expert used count %d is outside 1..%d", c->expert_used, c->expert_count);
        if (c->expert_ffn <= 0) FAIL("invalid expert feed-forward size %d", c->expert_ffn);
        if (c->shared_ffn <= 0) FAIL("invalid shared expert feed-forward size %d", c->shared_ffn);
    } else if (c->ffn <= 0) {
        FAIL("invalid feed-forward size %d", c->ffn);
    }
    if (c->context_length <= 0 || c->vocab <= 0) FAIL("invalid context or vocabulary size");
    if (c->block_count <= 0 || c->hidden <= 0 || c->head_dim <= 0) FAIL("invalid model size");
    return 0;
#undef FAIL
}

yo_model *yo_model_create(const yo_config *cfg) {
    if (yo_config_validate(cfg, NULL, 0) != 0) return NULL;
    yo_model *m = (yo_model *)calloc(1, sizeof(*m));
    m->cfg = *cfg;
    m->layers = (yo_layer *)calloc((size_t)cfg->block_count, sizeof(yo_layer));
    return m;
}

void yo_model_destroy(yo_model *m) {
    if (!m) return;
    free(m->layers);
    free(m);
}

static yo_mat mk(int dtype, const void *data, int64_t rows, int64_t cols) {
    yo_mat a = {(const uint8_t *)data, dtype, rows, cols};
    return a;
}

int yo_model_set_tensor(yo_model *m, const char *name, int dtype, const void *data, int64_t rows,
                        int64_t cols) {
    if (!m || !name || !data) return -1;
    if (yo_row_bytes(dtype, cols) < 0) return -2;
    yo_mat a = mk(dtype, data, rows, cols);
    const float *f = (const float *)data;
    if (!strcmp(name, "token_embd.weight")) { m->embedding = a; return 0; }
    if (!strcmp(name, "output.weight")) { m->output = a; m->has_output = 1; return 0; }
    if (!strcmp(name, "output_norm.weight")) { m->output_norm = f; return 0; }
    int li;
    char rest[96];
    if (sscanf(name, "blk.%d.%95s", &li, rest) != 2) return -3;
    if (li < 0 || li >= m->cfg.block_count) return -4;
    yo_layer *L = &m->layers[li];
#define V(n, fld) if (!strcmp(rest, n)) { if (dtype != YO_F32) return -5; L->fld = f; return 0; }
#define M(n, fld) if (!strcmp(rest, n)) { L->fld = a; return 0; }
    V("attn_norm.weight", attn_norm)
    V("post_attention_norm.weight", post_norm)
    M("attn_q.weight", q) M("attn_k.weight", k) M("attn_v.weight", v) M("attn_output.weight", o)
    V("attn_q_norm.weight", q_norm) V("attn_k_norm.weight", k_norm)
    M("attn_qkv.weight", qkv) M("attn_gate.weight", gate) M("ssm_out.weight", out)
    M("ssm_beta.weight", beta) M("ssm_alpha.weight", alpha)
    V("ssm_conv1d.weight", conv) V("ssm_dt.bias", dt) V("ssm_a", a) V("ssm_norm.weight", ssm_norm)
    M("ffn_gate.weight", ffn_gate) M("ffn_up.weight", ffn_up) M("ffn_down.weight", ffn_down)
    M("ffn_gate_inp.weight", router) V("ffn_gate_inp_shexp.weight", sh_gate_inp)
    M("ffn_gate_shexp.weight", sh_gate) M("ffn_up_shexp.weight", sh_up) M("ffn_down_shexp.weight", sh_down)
    M("ffn_gate_exps.weight", gate_exps) M("ffn_up_exps.weight", up_exps) M("ffn_down_exps.weight", down_exps)
#undef V
#undef M
    return -6;
}

static int want_mat(const yo_mat *a, int64_t rows, int64_t cols) {
    return a->data && a->rows == rows && a->cols == cols;
}

int yo_model_check(const yo_model *m, char *msg, size_t n) {
#define FAIL(...) do { if (msg) snprintf(msg, n, __VA_ARGS__); return -1; } while (0)
    const yo_config *c = &m->cfg;
    if (!want_mat(&m->embedding, c->vocab, c->hidden)) FAIL("token_embd.weight missing or misshaped");
    if (m->has_output && !want_mat(&m->output, c->vocab, c->hidden)) FAIL("output.weight misshaped");
    if (!m->output_norm) FAIL("output_norm.weight missing");
    int q_dim = c->heads * c->head_dim * 2, kv_dim = c->kv_heads * c->head_dim;
    int o_dim = c->heads * c->head_dim;
    int conv_dim = 2 * c->group_count * c->state_size + c->inner_size;
    for (int i = 0; i < c->block_count; i++) {
        const yo_layer *L = &m->layers[i];
        if (!L->attn_norm || !L->post_norm) FAIL("blk.%d norms missing", i);
        if (yo_is_recurrent(c, i)) {
            if (!want_mat(&L->qkv, conv_dim, c->hidden) || !want_mat(&L->gate, c->inner_size, c->hidden) ||
                !want_mat(&L->out, c->hidden, c->inner_size) ||
                !want_mat(&L->beta, c->time_step_rank, c->hidden) ||
                !want_mat(&L->alpha, c->time_step_rank, c->hidden) || !L->conv || !L->dt || !L->a ||
                !L->ssm_norm)
                FAIL("blk.%d recurrent tensors missing or misshaped", i);
        } else {
            if (!want_mat(&L->q, q_dim, c->hidden) || !want_mat(&L->k, kv_dim, c->hidden) ||
                !want_mat(&L->v, kv_dim, c->hidden) || !want_mat(&L->o, c->hidden, o_dim) ||
                !L->q_norm || !L->k_norm)
                FAIL("blk.%d attention tensors missing or misshaped", i);
        }
        if (c->expert_count > 0) {
            if (!want_mat(&L->router, c->expert_count, c->hidden) || !L->sh_gate_inp ||
                !want_mat(&L->sh_gate, c->shared_ffn, c->hidden) ||
                !want_mat(&L->sh_up, c->shared_ffn, c->hidden) ||
                !want_mat(&L->sh_down, c->hidden, c->shared_ffn) ||
                !want_mat(&L->gate_exps, (int64_t)c->expert_ffn * c->expert_count, c->hidden) ||
                !want_mat(&L->up_exps, (int64_t)c->expert_ffn * c->expert_count, c->hidden) ||
                !want_mat(&L->down_exps, (int64_t)c->hidden * c->expert_count, c->expert_ffn))
                FAIL("blk.%d MoE tensors missing or misshaped", i);
        } else if (!want_mat(&L->ffn_gate, c->ffn, c->hidden) || !want_mat(&L->ffn_up, c->ffn, c->hidden) ||
                   !want_mat(&L->ffn_down, c->hidden, c->ffn)) {
            FAIL("blk.%d FFN tensors missing or misshaped", i);
        }
    }
    return 0;
#undef FAIL
}

/* ------------------------------------------------------------------------- */
/* state: model/qwen35/state.go:46-263, kv_pool.go                            */

struct yo_state {
    const yo_model *m;
    int pos, capacity;
    int kv_format, pool_blocks, block_size, kv_dim;
    int64_t kv_row_bytes;
    int32_t *table;
    int table_len;
    uint8_t **k, **v;     /* per layer, NULL for recurrent layers */
    float **conv, **s;    /* per layer, NULL for attention layers */
    int64_t conv_count, s_count;
    /* scratch */
    float *x, *norm, *q, *kk, *vv, *attn, *tmp, *qkv, *z, *beta, *alpha, *cv, *gdn;
    float *ffn_gate, *ffn_up, *router, *ex_gate, *ex_up, *ex_out, *ex_w, *scores, *kv_row, *logits;
    int32_t *ex_ids;
};

static float *fz(int64_t n) { return (float *)calloc((size_t)(n > 0 ? n : 1), sizeof(float)); }

yo_state *yo_state_create(const yo_model *m, int capacity, int kv_format, int pool_blocks,
                          int block_size, const int32_t *table, int table_len) {
    const yo_config *c = &m->cfg;
    if (capacity <= 0 || capacity > c->context_length) return NULL;
    if (block_size <= 0) { /* state.go:68-72 */
        block_size = 16;
        if (capacity < block_size) block_size = capacity;
    }
    int need = (capacity + block_size - 1) / block_size;
    if (pool_blocks <= 0) pool_blocks = need;
    if (table && table_len < need) return NULL;
    int kv_dim = c->kv_heads * c->head_dim;
    int64_t rb = yo_kv_row_bytes(kv_format, kv_dim);
    if (rb < 0) return NULL;
    yo_state *s = (yo_state *)calloc(1, sizeof(*s));
    s->m = m;
    s->capacity = capacity;
    s->kv_format = kv_format;
    s->pool_blocks = pool_blocks;
    s->block_size = block_size;
    s->kv_dim = kv_dim;
    s->kv_row_bytes = rb;
    s->table_len = table ? table_len : need;
    s->table = (int32_t *)malloc(sizeof(int32_t) * (size_t)s->table_len);
    for (int i = 0; i < s->table_len; i++) {
        s->table[i] = table ? table[i] : i;
        if (s->table[i] < 0 || s->table[i] >= pool_blocks) {
            free(s->table);
            free(s);
            return NULL;
        }
    }
    int L = c->block_count;
    s->k = (uint8_t **)calloc((size_t)L, sizeof(void *));
    s->v = (uint8_t **)calloc((size_t)L, sizeof(void *));
    s->conv = (float **)calloc((size_t)L, sizeof(void *));
    s->s = (float **)calloc((size_t)L, sizeof(void *));
    int conv_dim = 2 * c->group_count * c->state_size + c->inner_size;
    s->conv_count = (int64_t)(c->conv_kernel - 1) * conv_dim;
    s->s_count = (int64_t)c->time_step_rank * c->state_size * c->state_size;
    int64_t pool_bytes = (int64_t)pool_blocks * block_size * rb;
    for (int i = 0; i < L; i++) {
        if (yo_is_recurrent(c, i)) {
            s->conv[i] = fz(s->conv_count);
            s->s[i] = fz(s->s_count);
        } else {
            s->k[i] = (uint8_t *)calloc((size_t)pool_bytes, 1);
            s->v[i] = (uint8_t *)calloc((size_t)pool_bytes, 1);
        }
    }
    int q_dim = c->heads * c->head_dim * 2, o_dim = c->heads * c->head_dim;
    s->x = fz(c->hidden); s->norm = fz(c->hidden); s->q = fz(q_dim); s->kk = fz(kv_dim);
    s->vv = fz(kv_dim); s->attn = fz(o_dim); s->tmp = fz(c->hidden); s->qkv = fz(conv_dim);
    s->z = fz(c->inner_size); s->beta = fz(c->time_step_rank); s->alpha = fz(c->time_step_rank);
    s->cv = fz(conv_dim); s->gdn = fz(c->inner_size); s->ffn_gate = fz(c->ffn); s->ffn_up = fz(c->ffn);
    s->scores = fz(capacity); s->kv_row = fz(kv_dim); s->logits = fz(c->vocab);
    if (c->expert_count > 0) {
        int width = c->expert_ffn > c->shared_ffn ? c->expert_ffn : c->shared_ffn;
        s->router = fz(c->expert_count); s->ex_gate = fz(width); s->ex_up = fz(width);
        s->ex_out = fz(c->hidden); s->ex_w = fz(c->expert_used);
        s->ex_ids = (int32_t *)calloc((size_t)c->expert_used, sizeof(int32_t));
    }
    return s;
}

void yo_state_destroy(yo_state *s) {
    if (!s) return;
    int L = s->m->cfg.block_count;
    for (int i = 0; i < L; i++) { free(s->k[i]); free(s->v[i]); free(s->conv[i]); free(s->s[i]); }
    free(s->k); free(s->v); free(s->conv); free(s->s); free(s->table);
    free(s->x); free(s->norm); free(s->q); free(s->kk); free(s->vv); free(s->attn); free(s->tmp);
    free(s->qkv); free(s->z); free(s->beta); free(s->alpha); free(s->cv); free(s->gdn);
    free(s->ffn_gate); free(s->ffn_up); free(s->router); free(s->ex_gate); free(s->ex_up);
    free(s->ex_out); free(s->ex_w); free(s->ex_ids); free(s->scores); free(s->kv_row); free(s->logits);
    free(s);
}

/* state.go:174-190 */
void yo_state_reset(yo_state *s) {
    s->pos = 0;
    int L = s->m->cfg.block_count;
    int64_t pool_bytes = (int64_t)s->pool_blocks * s->block_size * s->kv_row_bytes;
    for (int i = 0; i < L; i++) {
        if (s->k[i]) { memset(s->k[i], 0, (size_t)pool_bytes); memset(s->v[i], 0, (size_t)pool_bytes); }
        if (s->conv[i]) {
            memset(s->conv[i], 0, sizeof(float) * (size_t)s->conv_count);
            memset(s->s[i], 0, sizeof(float) * (size_t)s->s_count);
        }
    }
}

int yo_state_pos(const yo_state *s) { return s->pos; }
int yo_state_set_pos(yo_state *s, int pos) {
    if (pos < 0 || pos > s->capacity) return -1;
    s->pos = pos;
    return 0;
}

/* state.go:211-263: little-endian f32, conv then s, recurrent layers in order */
int64_t yo_state_snapshot_bytes(const yo_state *s) {
    int64_t n = 0;
    for (int i = 0; i < s->m->cfg.block_count; i++)
        if (s->conv[i]) n += s->conv_count + s->s_count;
    return n * 4;
}
int yo_state_snapshot(const yo_state *s, uint8_t *dst, int64_t len) {
    if (len != yo_state_snapshot_bytes(s)) return -1;
    for (int i = 0; i < s->m->cfg.block_count; i++) {
        if (!s->conv[i]) continue;
        memcpy(dst, s->conv[i], (size_t)s->conv_count * 4); dst += s->conv_count * 4;
        memcpy(dst, s->s[i], (size_t)s->s_count * 4); dst += s->s_count * 4;
    }
    return 0;
}
int yo_state_restore(yo_state *s, const uint8_t *src, int64_t len) {
    if (len != yo_state_snapshot_bytes(s)) return -1;
    for (int i = 0; i < s->m->cfg.block_count; i++) {
        if (!s->conv[i]) continue;
        memcpy(s->conv[i], src, (size_t)s->conv_count * 4); src += s->conv_count * 4;
        memcpy(s->s[i], src, (size_t)s->s_count * 4); src += s->s_count * 4;
    }
    return 0;
}

uint8_t *yo_state_kv(yo_state *s, int layer, int which, int64_t *bytes) {
    if (bytes) *bytes = (int64_t)s->pool_blocks * s->block_size * s->kv_row_bytes;
    return which ? s->v[layer] : s->k[layer];
}
float *yo_state_conv(yo_state *s, int layer, int64_t *count) {
    if (count) *count = s->conv_count;
    return s->conv[layer];
}
float *yo_state_s(yo_state *s, int layer, int64_t *count) {
    if (count) *count = s->s_count;
    return s->s[layer];
}
const float *yo_state_last_hidden(const yo_state *s) { return s->norm; }
const float *yo_logits(const yo_state *s) { return s->logits; }

/* kv_pool.go:117-170 */
static int64_t kv_row_offset(const yo_state *s, int pos) {
    int32_t block, off;
    if (yo_table_map(s->table, s->table_len, s->block_size, pos, &block, &off) != 0) return -1;
    if (block < 0 || block >= s->pool_blocks) return -1;
    return ((int64_t)block * s->block_size + off) * s->kv_row_bytes;
}

/* ------------------------------------------------------------------------- */
/* forward: model/qwen35/forward.go:116-389                                   */

static int matvec(float *dst, const yo_mat *w, const float *x) {
    return yo_matmul(dst, x, 1, w->data, w->dtype, w->rows, w->cols);
}

static int forward_ffn(const yo_model *m, const yo_layer *L, yo_state *s) {
    const yo_config *c = &m->cfg;
    if (c->expert_count > 0) {
        /* forward.go:320-389 */
        yo_rms_norm(s->norm, s->x, L->post_norm, c->hidden, c->rms_eps);
        matvec(s->router, &L->router, s->norm);
        yo_select_experts(s->router, c->expert_count, s->ex_ids, s->ex_w, c->expert_used);
        memset(s->tmp, 0, sizeof(float) * (size_t)c->hidden);
        int64_t rb_in = yo_row_bytes(L->gate_exps.dtype, c->hidden);
        int64_t rb_dn = yo_row_bytes(L->down_exps.dtype, c->expert_ffn);
        for (int slot = 0; slot < c->expert_used; slot++) {
            int id = s->ex_ids[slot];
            yo_mat g = mk(L->gate_exps.dtype, L->gate_exps.data + (int64_t)id * c->expert_ffn * rb_in,
                          c->expert_ffn, c->hidden);
            yo_mat u = mk(L->up_exps.dtype, L->up_exps.data + (int64_t)id * c->expert_ffn * rb_in,
                          c->expert_ffn, c->hidden);
            yo_mat d = mk(L->down_exps.dtype, L->down_exps.data + (int64_t)id * c->hidden * rb_dn,
                          c->hidden, c->expert_ffn);
            matvec(s->ex_gate, &g, s->norm);
            matvec(s->ex_up, &u, s->norm);
            for (int i = 0; i < c->expert_ffn; i++) s->ex_gate[i] = yo_silu(s->ex_gate[i]) * s->ex_up[i];
            matvec(s->ex_out, &d, s->ex_gate);
            float w = s->ex_w[slot];
            for (int i = 0; i < c->hidden; i++) s->tmp[i] += w * s->ex_out[i];
        }
        matvec(s->ex_gate, &L->sh_gate, s->norm);
        matvec(s->ex_up, &L->sh_up, s->norm);
        for (int i = 0; i < c->shared_ffn; i++) s->ex_gate[i] = yo_silu(s->ex_gate[i]) * s->ex_up[i];
        matvec(s->ex_out, &L->sh_down, s->ex_gate);
        float sg = yo_sigmoid(dotf(L->sh_gate_inp, s->norm, c->hidden));
        for (int i = 0; i < c->hidden; i++) s->tmp[i] += sg * s->ex_out[i];
        for (int i = 0; i < c->hidden; i++) s->x[i] += s->tmp[i];
        return 0;
    }
    /* forward.go:295-315 */
    yo_rms_norm(s->norm, s->x, L->post_norm, c->hidden, c->rms_eps);
    matvec(s->ffn_gate, &L->ffn_gate, s->norm);
    matvec(s->ffn_up, &L->ffn_up, s->norm);
    for (int i = 0; i < c->ffn; i++) s->ffn_gate[i] = yo_silu(s->ffn_gate[i]) * s->ffn_up[i];
    matvec(s->tmp, &L->ffn_down, s->ffn_gate);
    for (int i = 0; i < c->hidden; i++) s->x[i] += s->tmp[i];
    return 0;
}

/* forward.go:157-226 */
static int forward_full_attention(const yo_model *m, int index, const yo_layer *L, yo_state *s) {
    const yo_config *c = &m->cfg;
    int hd = c->head_dim;
    yo_rms_norm(s->norm, s->x, L->attn_norm, c->hidden, c->rms_eps);
    matvec(s->q, &L->q, s->norm);
    matvec(s->kk, &L->k, s->norm);
    matvec(s->vv, &L->v, s->norm);
    for (int h = 0; h < c->heads; h++) rms_norm_inplace(s->q + h * 2 * hd, L->q_norm, hd, c->rms_eps);
    for (int h = 0; h < c->kv_heads; h++) rms_norm_inplace(s->kk + h * hd, L->k_norm, hd, c->rms_eps);
    yo_apply_rope(s->q, c->heads, 2 * hd, hd, c->rope_dim, s->pos, c->rope_freq_base);
    yo_apply_rope(s->kk, c->kv_heads, hd, hd, c->rope_dim, s->pos, c->rope_freq_base);
    int64_t off = kv_row_offset(s, s->pos);
    if (off < 0) return -1;
    yo_kv_encode_row(s->k[index] + off, s->kv_format, s->kk, s->kv_dim);
    yo_kv_encode_row(s->v[index] + off, s->kv_format, s->vv, s->kv_dim);

    int group = c->heads / c->kv_heads;
    float scale = (float)(1.0 / sqrt((double)hd));
    int length = s->pos + 1;
    for (int h = 0; h < c->heads; h++) {
        int kvh = h / group;
        const float *q = s->q + h * 2 * hd;
        for (int p = 0; p < length; p++) {
            int64_t o = kv_row_offset(s, p);
            if (o < 0) return -1;
            yo_kv_decode_row(s->kv_row, s->kv_format, s->k[index] + o, s->kv_dim);
            s->scores[p] = dotf(q, s->kv_row + kvh * hd, hd) * scale;
        }
        yo_softmax_inplace(s->scores, length);
        float *out = s->attn + h * hd;
        memset(out, 0, sizeof(float) * (size_t)hd);
        for (int p = 0; p < length; p++) {
            float w = s->scores[p];
            int64_t o = kv_row_offset(s, p);
            yo_kv_decode_row(s->kv_row, s->kv_format, s->v[index] + o, s->kv_dim);
            const float *v = s->kv_row + kvh * hd;
            for (int d = 0; d < hd; d++) out[d] += w * v[d];
        }
        const float *gate = s->q + h * 2 * hd + hd;
        for (int d = 0; d < hd; d++) out[d] *= yo_sigmoid(gate[d]);
    }
    matvec(s->tmp, &L->o, s->attn);
    for (int i = 0; i < c->hidden; i++) s->x[i] += s->tmp[i];
    return forward_ffn(m, L, s);
}

/* forward.go:228-293 */
static int forward_recurrent(const yo_model *m, int index, const yo_layer *L, yo_state *s) {
    const yo_config *c = &m->cfg;
    yo_rms_norm(s->norm, s->x, L->attn_norm, c->hidden, c->rms_eps);
    matvec(s->qkv, &L->qkv, s->norm);
    matvec(s->z, &L->gate, s->norm);
    matvec(s->beta, &L->beta, s->norm);
    matvec(s->alpha, &L->alpha, s->norm);
    for (int h = 0; h < c->time_step_rank; h++) {
        s->beta[h] = yo_sigmoid(s->beta[h]);
        s->alpha[h] = yo_softplus(s->alpha[h] + L->dt[h]) * L->a[h];
    }
    float *cs = s->conv[index];
    int S = c->state_size;
    int conv_dim = 2 * c->group_count * S + c->inner_size;
    int kernel = c->conv_kernel;
    for (int ch = 0; ch < conv_dim; ch++) {
        float sum = 0;
        int base = ch * kernel, sb = ch * (kernel - 1);
        for (int t = 0; t < kernel - 1; t++) sum += L->conv[base + t] * cs[sb + t];
        sum += L->conv[base + kernel - 1] * s->qkv[ch];
        s->cv[ch] = yo_silu(sum);
        for (int t = 0; t < kernel - 2; t++) cs[sb + t] = cs[sb + t + 1];
        if (kernel > 1) cs[sb + kernel - 2] = s->qkv[ch];
    }
    int key_dim = c->group_count * S;
    float q_scale = (float)(1.0 / sqrt((double)S));
    for (int h = 0; h < c->group_count; h++) {
        yo_l2_norm_head(s->cv + h * S, S, c->rms_eps, q_scale);
        yo_l2_norm_head(s->cv + key_dim + h * S, S, c->rms_eps, 1);
    }
    yo_gdn_per_token_scan(s->s[index], s->cv, s->alpha, s->beta, s->gdn, 1, c->group_count,
                          c->time_step_rank, S, conv_dim);
    yo_gdn_norm_gate(s->gdn, s->z, L->ssm_norm, 1, c->time_step_rank, S, c->rms_eps);
    matvec(s->tmp, &L->out, s->gdn);
    for (int i = 0; i < c->hidden; i++) s->x[i] += s->tmp[i];
    return forward_ffn(m, L, s);
}

/* forward.go:116-155 */
int yo_forward_one(const yo_model *m, yo_state *s, int32_t token, int want_logits) {
    const yo_config *c = &m->cfg;
    if (s->pos >= s->capacity) return -1;
    if (token < 0 || token >= c->vocab) return -2;
    int64_t rb = yo_row_bytes(m->embedding.dtype, c->hidden);
    if (yo_dequantize_row(s->x, c->hidden, m->embedding.dtype, m->embedding.data + (int64_t)token * rb, rb) != 0)
        return -3;
    for (int i = 0; i < c->block_count; i++) {
        const yo_layer *L = &m->layers[i];
        int rc = yo_is_recurrent(c, i) ? forward_recurrent(m, i, L, s) : forward_full_attention(m, i, L, s);
        if (rc != 0) return rc;
    }
    yo_rms_norm(s->norm, s->x, m->output_norm, c->hidden, c->rms_eps);
    if (want_logits) {
        const yo_mat *out = m->has_output ? &m->output : &m->embedding;
        matvec(s->logits, out, s->norm);
    }
    s->pos++;
    return 0;
}

/* forward.go:12-38 */
int yo_forward(const yo_model *m, yo_state *s, const int32_t *tokens, int n, float *last_logits) {
    if (n <= 0) return -1;
    if (s->pos + n > s->capacity) return -2;
    for (int i = 0; i < n; i++) {
        int rc = yo_forward_one(m, s, tokens[i], i == n - 1);
        if (rc != 0) return rc;
    }
    if (last_logits) memcpy(last_logits, s->logits, sizeof(float) * (size_t)m->cfg.vocab);
    return 0;
}

/* forward.go:77-99 */
int yo_prefill_logits(const yo_model *m, yo_state *s, const int32_t *tokens, int n, float *out) {
    if (n <= 0) return -1;
    if (s->pos + n > s->capacity) return -2;
    for (int i = 0; i < n; i++) {
        int rc = yo_forward_one(m, s, tokens[i], 1);
        if (rc != 0) return rc;
        memcpy(out + (int64_t)i * m->cfg.vocab, s->logits, sizeof(float) * (size_t)m->cfg.vocab);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* speculative loop pieces: engine/speculative.go                             */

/* speculative.go:263-271: first maximum wins (strict >) */
int32_t yo_argmax(const float *logits, int n) {
    int best = 0;
    for (int i = 1; i < n; i++)
        if (logits[i] > logits[best]) best = i;
    return best;
}

/* speculative.go:39-66 */
int yo_lookup_draft(const int32_t *h, int n, int max_draft, int min_match, int32_t *out) {
    if (max_draft <= 0 || min_match <= 0 || n <= min_match) return 0;
    int max_n = n - 1 < 8 ? n - 1 : 8;
    for (int len = max_n; len >= min_match; len--) {
        const int32_t *suffix = h + n - len;
        for (int start = n - len - 1; start >= 0; start--) {
            int match = 1;
            for (int i = 0; i < len; i++)
                if (h[start + i] != suffix[i]) { match = 0; break; }
            if (!match) continue;
            int follow = start + len;
            int take = n - follow < max_draft ? n - follow : max_draft;
            if (take <= 0) continue;
            memcpy(out, h + follow, sizeof(int32_t) * (size_t)take);
            return take;
        }
    }
    return 0;
}

/* speculative.go:181-239 */
int yo_spec_verify_reference(const yo_model *m, yo_state *s, float *logits, const int32_t *draft,
                             int k, int32_t *accepted_out, int32_t *emitted, int32_t *n_emitted) {
    int V = m->cfg.vocab;
    int64_t snap_len = yo_state_snapshot_bytes(s);
    uint8_t *snap = (uint8_t *)malloc((size_t)(snap_len > 0 ? snap_len : 1));
    yo_state_snapshot(s, snap, snap_len);
    int position = s->pos;
    float *cand = (float *)malloc(sizeof(float) * (size_t)k * V);
    int rc = yo_prefill_logits(m, s, draft, k, cand);
    if (rc != 0) { free(snap); free(cand); return rc; }
    int accepted = 0;
    const float *before = logits;
    int32_t correction = -1;
    for (int i = 0; i < k; i++) {
        int32_t want = yo_argmax(before, V);
        if (want == draft[i]) { accepted++; before = cand + (int64_t)i * V; continue; }
        correction = want;
        break;
    }
    if (accepted == k) {
        memcpy(emitted, draft, sizeof(int32_t) * (size_t)k);
        *n_emitted = k;
        memcpy(logits, cand + (int64_t)(k - 1) * V, sizeof(float) * (size_t)V);
    } else {
        yo_state_restore(s, snap, snap_len);
        yo_state_set_pos(s, position);
        memcpy(emitted, draft, sizeof(int32_t) * (size_t)accepted);
        emitted[accepted] = correction;
        *n_emitted = accepted + 1;
        rc = yo_forward(m, s, emitted, accepted + 1, logits);
    }
    *accepted_out = accepted;
    free(snap);
    free(cand);
    return rc;
}

int yo_verify_chain(const yo_model *m, yo_state *s, int32_t pending, const int32_t *draft, int k,
                    int32_t *accepted, int32_t *emitted, float *all_logits) {
    int n = k + 1;
    int32_t *tokens = (int32_t *)malloc(sizeof(int32_t) * (size_t)n * 2);
    int32_t *parent = tokens + n;
    tokens[0] = pending;
    parent[0] = -1;
    for (int i = 0; i < k; i++) { tokens[i + 1] = draft[i]; parent[i + 1] = i; }
    int rc = yo_verify_tree_greedy(m, s, tokens, parent, n, accepted, NULL, emitted, all_logits);
    free(tokens);
    return rc;
}

int yo_accept_greedy_tree(const float *logits, int V, const int32_t *tokens, const int32_t *parent,
                          int n, int32_t *accepted, int32_t *path_out, int32_t *emitted) {
    int cur = 0, a = 0;
    for (;;) {
        int32_t want = yo_argmax(logits + (int64_t)cur * V, V);
        int next = -1;
        for (int c = cur + 1; c < n; c++)
            if (parent[c] == cur && tokens[c] == want) { next = c; break; }
        emitted[a] = want;
        if (next < 0) break;
        if (path_out) path_out[a] = next;
        a++;
        cur = next;
    }
    *accepted = a;
    return cur;
}

/* Per-node logits by running every root-to-node path as a chain from the
 * entry state; the committed state is the one after the accepted path. */
int yo_verify_tree_greedy(const yo_model *m, yo_state *s, const int32_t *tokens,
                          const int32_t *parent, int n, int32_t *accepted, int32_t *path_out,
                          int32_t *emitted, float *all_logits) {
    int V = m->cfg.vocab;
    if (n <= 0 || parent[0] != -1) return -1;
    for (int i = 1; i < n; i++)
        if (parent[i] < 0 || parent[i] >= i) return -1;
    int64_t snap_len = yo_state_snapshot_bytes(s);
    uint8_t *snap = (uint8_t *)malloc((size_t)(snap_len > 0 ? snap_len : 1));
    yo_state_snapshot(s, snap, snap_len);
    int pos0 = s->pos;
    float *logits = all_logits ? all_logits : (float *)malloc(sizeof(float) * (size_t)n * V);
    int32_t *path = (int32_t *)malloc(sizeof(int32_t) * (size_t)n * 3);
    int32_t *toks = path + n, *own_path = path + 2 * n;
    int rc = 0;
    char *done = (char *)calloc((size_t)n, 1);
    /* run leaves' paths; every node lies on some leaf path */
    for (int leaf = n - 1; leaf >= 0 && rc == 0; leaf--) {
        if (done[leaf]) continue;
        int len = 0;
        for (int c = leaf; c >= 0; c = parent[c]) path[len++] = c;
        yo_state_restore(s, snap, snap_len);
        yo_state_set_pos(s, pos0);
        for (int i = len - 1; i >= 0 && rc == 0; i--) {
            int node = path[i];
            rc = yo_forward_one(m, s, tokens[node], !done[node]);
            if (rc == 0 && !done[node]) {
                memcpy(logits + (int64_t)node * V, s->logits, sizeof(float) * (size_t)V);
                done[node] = 1;
            }
        }
    }
    if (rc == 0) {
        if (!path_out) path_out = own_path;
        yo_accept_greedy_tree(logits, V, tokens, parent, n, accepted, path_out, emitted);
        /* commit: replay the accepted path from the entry state */
        yo_state_restore(s, snap, snap_len);
        yo_state_set_pos(s, pos0);
        toks[0] = tokens[0];
        for (int i = 0; i < *accepted; i++) toks[i + 1] = tokens[path_out[i]];
        for (int i = 0; i <= *accepted && rc == 0; i++) rc = yo_forward_one(m, s, toks[i], 0);
    }
    free(done);
    free(path);
    free(snap);
    if (!all_logits) free(logits);
    return rc;
}

/* ------------------------------------------------------------------------- */
/* Rejection-sampling acceptance. The reference has none (it requires greedy
 * sampling, engine/speculative.go:73-75); this rule is defined here and the
 * CUDA kernel implements the same one. Every quantity that decides a token is
 * either an elementwise IEEE operation or an integer sum, so the result does
 * not depend on summation order and the two sides agree bit for bit.
 *
 * ACCEPT_RULE, at node cur (start: root 0), with children in node order:
 *   mx   = max_i L[cur][i]
 *   e_i  = exp_det((L[cur][i] - mx) * (1/T))              (fp32, yo_exp_det)
 *   w_i  = (uint64) (e_i * 2^40)                           (truncation)
 *   r = w, R = sum_i w_i
 *   for child c (token x, draft distribution Q[c][.], uniform u = U[2c]):
 *     accept iff (double)(u * Q[c][x]) * (double)R <= (double) r_x
 *       -> cur = c, restart at the top with node c
 *     else r_i = max(0, r_i - (uint64)((double)Q[c][i] * (double)R)); R = sum r_i;
 *          if R == 0: r = w, R = sum w
 *   no child accepted: t = min((uint64)((double)U[2cur+1] * (double)R), R-1);
 *     emit the smallest j with sum_{i<=j} r_i > t, stop.
 */

float yo_exp_det(float x) {
    if (x < -87.0f) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float n = rintf(x * 1.44269504f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float e = fmaf(p, r2, r) + 1.0f;
    uint32_t bits = (uint32_t)((int)n + 127) << 23;
    float scale;
    memcpy(&scale, &bits, 4);
    return e * scale;
}

int yo_accept_rejection_tree(const float *logits, const float *Q, int V, const int32_t *tokens,
                             const int32_t *parent, int n, float T, const float *U,
                             int32_t *accepted, int32_t *path_out, int32_t *emitted) {
    uint64_t *w = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)V * 2);
    uint64_t *r = w + V;
    float inv_t = 1.0f / T;
    int cur = 0, a = 0;
    for (;;) {
        const float *L = logits + (int64_t)cur * V;
        float mx = L[0];
        for (int i = 1; i < V; i++)
            if (L[i] > mx) mx = L[i];
        uint64_t Z = 0;
        for (int i = 0; i < V; i++) {
            float e = yo_exp_det((L[i] - mx) * inv_t);
            w[i] = (uint64_t)(e * 1099511627776.0f);
            Z += w[i];
        }
        memcpy(r, w, sizeof(uint64_t) * (size_t)V);
        uint64_t R = Z;
        int next = -1;
        for (int c = cur + 1; c < n && next < 0; c++) {
            if (parent[c] != cur) continue;
            const float *q = Q + (int64_t)c * V;
            int32_t x = tokens[c];
            float lhs = U[2 * c] * q[x];
            if ((double)lhs * (double)R <= (double)r[x]) { next = c; break; }
            uint64_t sum = 0;
            for (int i = 0; i < V; i++) {
                uint64_t qr = (uint64_t)((double)q[i] * (double)R);
                r[i] = r[i] > qr ? r[i] - qr : 0;
                sum += r[i];
            }
            R = sum;
            if (R == 0) { memcpy(r, w, sizeof(uint64_t) * (size_t)V); R = Z; }
        }
        if (next >= 0) {
            emitted[a] = tokens[next];
            if (path_out) path_out[a] = next;
            a++;
            cur = next;
            continue;
        }
        uint64_t t = (uint64_t)((double)U[2 * cur + 1] * (double)R);
        if (t >= R) t = R - 1;
        uint64_t acc = 0;
        int32_t tok = V - 1;
        for (int i = 0; i < V; i++) {
            acc += r[i];
            if (acc > t) { tok = i; break; }
        }
        emitted[a] = tok;
        break;
    }
    *accepted = a;
    free(w);
    return cur;
}
