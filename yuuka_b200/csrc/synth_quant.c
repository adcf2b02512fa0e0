/* Synthetic-weight tooling: a seeded normal generator and F32 -> Q8_0 / Q4_K /
 * Q5_K / Q6_K weight quantizers (host only, OpenMP over rows).
 *
 * The reference ships dequantizers only (tensor/quant.go:87-158,261-285); its
 * tests fill packed rows with arbitrary bytes. These quantizers are written
 * from the block layouts in tensor/dtype.go:102-151 so that "weights N(0, s)
 * quantized to Q4_K" can be produced for the benchmark configurations. Any
 * packing is valid as long as the same bytes feed the CPU oracle and the GPU.
 *
 * The generator is counter based (value i depends on seed and i only), so the
 * bytes do not depend on the thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define YS_API __attribute__((visibility("default")))

enum { YS_F32 = 0, YS_F16 = 1, YS_Q8_0 = 8, YS_Q4_K = 12, YS_Q5_K = 13, YS_Q6_K = 14 };

static inline uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

/* Two standard normals from counter c (Box-Muller in double). */
static inline void normal_pair(uint64_t seed, uint64_t c, float *a, float *b) {
    uint64_t h = mix64(seed * 0xd1342543de82ef95ull + c);
    uint64_t g = mix64(h ^ 0x2545f4914f6cdd1dull);
    double u1 = ((double)(h >> 11) + 1.0) * (1.0 / 9007199254740993.0); /* (0,1) */
    double u2 = (double)(g >> 11) * (1.0 / 9007199254740992.0);
    double r = sqrt(-2.0 * log(u1));
    double t = 6.283185307179586476925 * u2;
    *a = (float)(r * cos(t));
    *b = (float)(r * sin(t));
}

/* element i of stream seed: pair i/2, member i%2 */
static void fill_normal_range(float *dst, int64_t start, int64_t n, float mean, float std, uint64_t seed) {
    int64_t i = 0;
    if (start & 1) {
        float a, b;
        normal_pair(seed, (uint64_t)(start >> 1), &a, &b);
        dst[0] = mean + std * b;
        i = 1;
    }
    for (; i + 1 < n; i += 2) {
        float a, b;
        normal_pair(seed, (uint64_t)((start + i) >> 1), &a, &b);
        dst[i] = mean + std * a;
        dst[i + 1] = mean + std * b;
    }
    if (i < n) {
        float a, b;
        normal_pair(seed, (uint64_t)((start + i) >> 1), &a, &b);
        dst[i] = mean + std * a;
    }
}

YS_API void ys_fill_normal_f32(float *dst, int64_t n, float mean, float std, uint64_t seed) {
    const int64_t chunk = 1 << 16;
    int64_t chunks = (n + chunk - 1) / chunk;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < chunks; c++) {
        int64_t s = c * chunk, len = n - s < chunk ? n - s : chunk;
        fill_normal_range(dst + s, s, len, mean, std, seed);
    }
}

YS_API void ys_fill_uniform_i32(int32_t *dst, int64_t n, int32_t lo, int32_t hi, uint64_t seed) {
    uint64_t span = (uint64_t)(hi - lo);
    for (int64_t i = 0; i < n; i++) dst[i] = lo + (int32_t)(mix64(seed * 0x9e3779b97f4a7c15ull + (uint64_t)i) % span);
}

YS_API void ys_fill_uniform_f32(float *dst, int64_t n, uint64_t seed) {
    for (int64_t i = 0; i < n; i++)
        dst[i] = (float)(mix64(seed * 0xd6e8feb86659fd93ull + (uint64_t)i) >> 40) * (1.0f / 16777216.0f);
}

/* round-to-nearest-even binary16 encode (storage of block scales) */
static uint16_t f32_to_f16(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    uint32_t sign = (b >> 16) & 0x8000u;
    int32_t e = (int32_t)((b >> 23) & 0xff) - 127 + 15;
    uint32_t m = b & 0x7fffffu;
    if (((b >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00 | (m ? 0x200 : 0));
    if (e >= 31) return (uint16_t)(sign | 0x7c00);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000u;
        int shift = 14 - e;
        uint32_t half = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (m >> 13);
    uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff, bits;
    if (e == 0) {
        if (m == 0) bits = sign;
        else {
            uint32_t ee = 113;
            while (!(m & 0x400)) { m <<= 1; ee--; }
            bits = sign | (ee << 23) | ((m & 0x3ff) << 13);
        }
    } else if (e == 31) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline void put16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void q_q8_0(uint8_t *dst, const float *x) {
    float amax = 0;
    for (int i = 0; i < 32; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    uint16_t dh = f32_to_f16(amax / 127.0f);
    float d = f16_to_f32(dh);
    float id = d != 0 ? 1.0f / d : 0.0f;
    put16(dst, dh);
    for (int i = 0; i < 32; i++) dst[2 + i] = (uint8_t)(int8_t)clampi((int)lrintf(x[i] * id), -127, 127);
}

/* shared Q4_K / Q5_K: qmax = 15 or 31 */
static void kquant_scales(const float *x, int qmax, uint8_t *sc, uint8_t *mn, float *d_out, float *dm_out,
                          uint16_t *dh, uint16_t *dmh) {
    float scale[8], minv[8], smax = 0, mmax = 0;
    for (int b = 0; b < 8; b++) {
        float lo = 0, hi = 0;
        for (int i = 0; i < 32; i++) {
            float v = x[b * 32 + i];
            if (v < lo) lo = v;
            if (v > hi) hi = v;
        }
        scale[b] = (hi - lo) / (float)qmax;
        minv[b] = -lo;
        if (scale[b] > smax) smax = scale[b];
        if (minv[b] > mmax) mmax = minv[b];
    }
    *dh = f32_to_f16(smax / 63.0f);
    *dmh = f32_to_f16(mmax / 63.0f);
    float d = f16_to_f32(*dh), dm = f16_to_f32(*dmh);
    for (int b = 0; b < 8; b++) {
        sc[b] = (uint8_t)(d != 0 ? clampi((int)lrintf(scale[b] / d), 0, 63) : 0);
        mn[b] = (uint8_t)(dm != 0 ? clampi((int)lrintf(minv[b] / dm), 0, 63) : 0);
    }
    *d_out = d;
    *dm_out = dm;
}

static void pack_scales_k4(uint8_t *out, const uint8_t *sc, const uint8_t *mn) {
    for (int j = 0; j < 4; j++) {
        out[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        out[j + 4] = (uint8_t)((mn[j] & 63) | ((mn[j + 4] >> 4) << 6));
        out[j + 8] = (uint8_t)((sc[j + 4] & 0x0f) | ((mn[j + 4] & 0x0f) << 4));
    }
}

static void q_q4_k(uint8_t *dst, const float *x) {
    uint8_t sc[8], mn[8], q[256];
    float d, dm;
    uint16_t dh, dmh;
    kquant_scales(x, 15, sc, mn, &d, &dm, &dh, &dmh);
    put16(dst, dh);
    put16(dst + 2, dmh);
    pack_scales_k4(dst + 4, sc, mn);
    for (int b = 0; b < 8; b++) {
        float s = d * (float)sc[b], m = dm * (float)mn[b];
        float is = s != 0 ? 1.0f / s : 0.0f;
        for (int i = 0; i < 32; i++) q[b * 32 + i] = (uint8_t)clampi((int)lrintf((x[b * 32 + i] + m) * is), 0, 15);
    }
    uint8_t *qs = dst + 16;
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) qs[j * 32 + l] = (uint8_t)(q[j * 64 + l] | (q[j * 64 + 32 + l] << 4));
}

static void q_q5_k(uint8_t *dst, const float *x) {
    uint8_t sc[8], mn[8], q[256];
    float d, dm;
    uint16_t dh, dmh;
    kquant_scales(x, 31, sc, mn, &d, &dm, &dh, &dmh);
    put16(dst, dh);
    put16(dst + 2, dmh);
    pack_scales_k4(dst + 4, sc, mn);
    for (int b = 0; b < 8; b++) {
        float s = d * (float)sc[b], m = dm * (float)mn[b];
        float is = s != 0 ? 1.0f / s : 0.0f;
        for (int i = 0; i < 32; i++) q[b * 32 + i] = (uint8_t)clampi((int)lrintf((x[b * 32 + i] + m) * is), 0, 31);
    }
    uint8_t *qh = dst + 16, *ql = dst + 48;
    memset(qh, 0, 32);
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) {
            uint8_t a = q[j * 64 + l], b = q[j * 64 + 32 + l];
            ql[j * 32 + l] = (uint8_t)((a & 15) | ((b & 15) << 4));
            if (a & 16) qh[l] |= (uint8_t)(1u << (2 * j));
            if (b & 16) qh[l] |= (uint8_t)(2u << (2 * j));
        }
}

static void q_q6_k(uint8_t *dst, const float *x) {
    float scale[16], smax = 0;
    for (int b = 0; b < 16; b++) {
        float amax = 0;
        for (int i = 0; i < 16; i++) { float a = fabsf(x[b * 16 + i]); if (a > amax) amax = a; }
        scale[b] = amax / 31.0f;
        if (scale[b] > smax) smax = scale[b];
    }
    uint16_t dh = f32_to_f16(smax / 127.0f);
    float d = f16_to_f32(dh);
    int8_t sc[16];
    uint8_t q[256];
    for (int b = 0; b < 16; b++) {
        sc[b] = (int8_t)(d != 0 ? clampi((int)lrintf(scale[b] / d), 0, 127) : 0);
        float s = d * (float)sc[b];
        float is = s != 0 ? 1.0f / s : 0.0f;
        for (int i = 0; i < 16; i++) q[b * 16 + i] = (uint8_t)(clampi((int)lrintf(x[b * 16 + i] * is), -32, 31) + 32);
    }
    uint8_t *ql = dst, *qh = dst + 128;
    memset(dst, 0, 192);
    /* element n*128 + g*32 + l: ql[n*64 + (g&1)*32 + l] nibble (g>>1), qh[n*32 + l] bits 2g..2g+1 */
    for (int n = 0; n < 2; n++)
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++) {
                uint8_t v = q[n * 128 + g * 32 + l];
                ql[n * 64 + (g & 1) * 32 + l] |= (uint8_t)((v & 15) << ((g >> 1) * 4));
                qh[n * 32 + l] |= (uint8_t)((v >> 4) << (2 * g));
            }
    memcpy(dst + 192, sc, 16);
    put16(dst + 208, dh);
}

static int layout(int dtype, int *elems, int *bytes) {
    switch (dtype) {
    case YS_F32: *elems = 1; *bytes = 4; return 0;
    case YS_F16: *elems = 1; *bytes = 2; return 0;
    case YS_Q8_0: *elems = 32; *bytes = 34; return 0;
    case YS_Q4_K: *elems = 256; *bytes = 144; return 0;
    case YS_Q5_K: *elems = 256; *bytes = 176; return 0;
    case YS_Q6_K: *elems = 256; *bytes = 210; return 0;
    default: return -1;
    }
}

YS_API int64_t ys_row_bytes(int dtype, int64_t cols) {
    int e, b;
    if (layout(dtype, &e, &b) != 0 || cols <= 0 || cols % e != 0) return -1;
    return cols / e * b;
}

static void quantize_row(uint8_t *dst, int dtype, const float *x, int64_t cols) {
    switch (dtype) {
    case YS_F32: memcpy(dst, x, (size_t)cols * 4); break;
    case YS_F16: for (int64_t i = 0; i < cols; i++) put16(dst + i * 2, f32_to_f16(x[i])); break;
    case YS_Q8_0: for (int64_t b = 0; b < cols / 32; b++) q_q8_0(dst + b * 34, x + b * 32); break;
    case YS_Q4_K: for (int64_t b = 0; b < cols / 256; b++) q_q4_k(dst + b * 144, x + b * 256); break;
    case YS_Q5_K: for (int64_t b = 0; b < cols / 256; b++) q_q5_k(dst + b * 176, x + b * 256); break;
    case YS_Q6_K: for (int64_t b = 0; b < cols / 256; b++) q_q6_k(dst + b * 210, x + b * 256); break;
    }
}

/* Quantize a row-major float matrix. */
YS_API int ys_quantize(uint8_t *dst, int dtype, const float *src, int64_t rows, int64_t cols) {
    int64_t rb = ys_row_bytes(dtype, cols);
    if (rb < 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) quantize_row(dst + r * rb, dtype, src + r * cols, cols);
    return 0;
}

/* Draw rows x cols values N(0, std) from stream seed and quantize them. */
YS_API int ys_fill_normal_quant(uint8_t *dst, int dtype, int64_t rows, int64_t cols, float std, uint64_t seed) {
    int64_t rb = ys_row_bytes(dtype, cols);
    if (rb < 0) return -1;
    int fail = 0;
#pragma omp parallel
    {
        float *buf = (float *)malloc(sizeof(float) * (size_t)cols);
        if (!buf) {
#pragma omp atomic write
            fail = 1;
        } else {
#pragma omp for schedule(static)
            for (int64_t r = 0; r < rows; r++) {
                fill_normal_range(buf, r * cols, cols, 0.0f, std, seed);
                quantize_row(dst + r * rb, dtype, buf, cols);
            }
            free(buf);
        }
    }
    return fail ? -2 : 0;
}
