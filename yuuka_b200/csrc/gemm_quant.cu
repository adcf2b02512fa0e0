// Quantized GEMM entry points.
//   out[m][n] = sum_k x[m][k] * W[n][k],  W in packed GGUF rows (Q4_K/Q5_K/Q6_K/Q8_0/F16/F32)
// This file holds the kernel for weights in the GGUF row-major layout (a
// warp-per-row CUDA-core dot product with the reference's fp32 decode,
// tensor/quant.go:378-466; any dtype, any alignment) and the C ABI entry
// points. The fast kernels read a tile-ordered copy of the matrix
// (gemm_tiled.cu).
#include <mutex>

#include "gemm_quant.cuh"
#include "gemm_tiled.cuh"
#include "quant.cuh"

namespace yk {

__device__ int g_device_error = 0;

int read_device_error(const yuuka_device * dev) {
    set_device(dev);
    int v = 0;
    YK_CUDA(cudaMemcpyFromSymbol(&v, g_device_error, sizeof(int)));
    return v | read_gemm_wait_expired();
}

void clear_device_error(const yuuka_device * dev) {
    set_device(dev);
    const int zero = 0;
    cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int));
    clear_gemm_wait_expired();
}

// The same two flags copied behind the work already queued on `stream`, into two page-locked words.
void enqueue_device_error_read(cudaStream_t stream, int * out2) {
    YK_CUDA(cudaMemcpyFromSymbolAsync(out2, g_device_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
    enqueue_gemm_wait_expired_read(stream, out2 + 1);
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

uint32_t gemm_auto_path(uint32_t w_dtype, int rows, int n_in) {
    if (!tiled_supported(w_dtype, n_in)) return YUUKA_GEMM_PATH_FP32;
    // (one and two rows too: the exact register-fed route streams the weights four times faster than the fp32
    // CUDA-core kernel, which stays available as YUUKA_GEMM_PATH_FP32 and serves GGUF-ordered weights)
    (void)rows;
    return YUUKA_GEMM_PATH_MMA;
}

void gemm_scratch_reserve(const yuuka_device * dev, GemmScratch & s, uint32_t w_dtype, int rows, int n_out, int n_in) {
    set_device(dev);
    uint64_t want = 0;
    int tiles = 0;
    gemm_tiled_scratch_need(dev, w_dtype, rows, n_out, n_in, &want, &tiles);
    if (want > s.partial_floats) {
        if (s.partial) cudaFree(s.partial);
        s.partial = nullptr;
        s.partial_floats = 0;
        cudaError_t err = cudaMalloc(&s.partial, want * sizeof(float));
        YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "gemm scratch allocation of %llu bytes failed",
                   (unsigned long long)(want * 4));
        s.partial_floats = want;
    }
    const uint64_t xneed = tiled_supported(w_dtype, n_in) ? (uint64_t)rows * n_in : 0;
    if (xneed > s.xh_elems) {
        if (s.xh) cudaFree(s.xh);
        if (s.xl) cudaFree(s.xl);
        if (s.xs16) cudaFree(s.xs16);
        s.xh = nullptr;
        s.xl = nullptr;
        s.xs16 = nullptr;
        s.xh_elems = 0;
        cudaError_t err = cudaMalloc(&s.xh, xneed * sizeof(__half));
        if (err == cudaSuccess) err = cudaMalloc(&s.xl, xneed * sizeof(__half));
        if (err == cudaSuccess) err = cudaMalloc(&s.xs16, xneed / 16 * sizeof(__half2) + 16);
        YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "gemm activation scratch allocation failed");
        s.xh_elems = xneed;
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
    if (s.xh) cudaFree(s.xh);
    if (s.xl) cudaFree(s.xl);
    if (s.xs16) cudaFree(s.xs16);
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
    YK_REQUIRE(a.path != YUUKA_GEMM_PATH_MMA, YUUKA_ERR_UNSUPPORTED,
               "gemm_quant: the mma route reads tile-ordered weights (yuuka_weights_tile, YUUKA_GEMM_TILED)");
    set_device(dev);
    return a.x_dtype == YUUKA_DTYPE_F32 ? launch_fp32<float>(dev, stream, a) : launch_fp32<__nv_bfloat16>(dev, stream, a);
}

}  // namespace yk

// ---------------------------------------------------------------------------
// C ABI

namespace {
// One lazily grown scratch per device index for the kernel-level entry point. The mutex covers its host
// side (growing it frees and reallocates the buffers) and the launch that captures the pointers; the
// device side is shared by every call on the device, as the header says.
yk::GemmScratch g_scratch[16];
std::mutex g_scratch_mutex;
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
        std::lock_guard<std::mutex> lock(g_scratch_mutex);
        GemmScratch & sc = g_scratch[dev->index];
        if (flags & YUUKA_GEMM_TILED) {
            YK_REQUIRE(tiled_supported(w_dtype, n_in), YUUKA_ERR_UNSUPPORTED,
                       "gemm_quant: dtype %u with %llu columns has no tiled layout", w_dtype, (unsigned long long)n_in);
            YK_REQUIRE(tiled_bytes(w_dtype, n_out, n_in) <= w->bytes - w_offset && w_offset % 16 == 0,
                       YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant: tiled weight range exceeds the buffer or is misaligned");
            gemm_scratch_reserve(dev, sc, w_dtype, (int)rows, (int)n_out, (int)n_in);
            TiledGemmArgs t;
            t.w = (const uint8_t *)w->ptr + w_offset;
            t.w_dtype = w_dtype;
            t.x = (const uint8_t *)x->ptr + x_offset;
            t.x_dtype = x_dtype;
            t.ldx = (int64_t)n_in;
            t.out = (float *)((uint8_t *)out->ptr + out_offset);
            t.ldo = (int64_t)n_out;
            t.rows = (int)rows;
            t.n_out = (int)n_out;
            t.n_in = (int)n_in;
            t.path = path;
            t.flags = flags;
            t.scratch = &sc;
            launch_gemm_tiled(dev, stream->s, t);
            record_completion(stream, completion);
            return;
        }
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

extern "C" uint64_t yuuka_weights_tiled_bytes(uint32_t dtype, uint64_t n_out, uint64_t n_in) {
    return yk::tiled_supported(dtype, n_in) ? yk::tiled_bytes(dtype, n_out, n_in) : 0;
}

extern "C" yuuka_status yuuka_weights_tile(yuuka_stream * stream, yuuka_buffer * dst, uint64_t dst_offset,
                                           const yuuka_buffer * src, uint64_t src_offset, uint32_t dtype, uint64_t n_out,
                                           uint64_t n_in, yuuka_event * completion) {
    using namespace yk;
    return guard([&] {
        YK_REQUIRE(stream && dst && src, YUUKA_ERR_INVALID_ARGUMENT, "weights_tile: null argument");
        YK_REQUIRE(n_out > 0 && n_out < (1u << 28) && n_in > 0 && n_in < (1u << 20), YUUKA_ERR_INVALID_ARGUMENT,
                   "weights_tile: invalid shape");
        YK_REQUIRE(tiled_supported(dtype, n_in), YUUKA_ERR_UNSUPPORTED,
                   "weights_tile: dtype %u with %llu columns has no tiled layout", dtype, (unsigned long long)n_in);
        uint64_t rb = row_bytes(dtype, n_in);
        YK_REQUIRE(src_offset <= src->bytes && n_out * rb <= src->bytes - src_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "weights_tile: source range exceeds the buffer");
        YK_REQUIRE(dst_offset % 16 == 0 && dst_offset <= dst->bytes && tiled_bytes(dtype, n_out, n_in) <= dst->bytes - dst_offset,
                   YUUKA_ERR_INVALID_ARGUMENT, "weights_tile: destination range exceeds the buffer or is misaligned");
        set_device(stream->dev);
        launch_tile_weights(stream->s, (uint8_t *)dst->ptr + dst_offset, (const uint8_t *)src->ptr + src_offset, dtype,
                            (int)n_out, (int)n_in);
        record_completion(stream, completion);
    });
}
