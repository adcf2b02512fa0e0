// Tiled quantized GEMM whose scratch memory is a fixed device array of this
// library, for callers that must not cause a device allocation.
//
// yuuka_gemm_quant keeps a per-device scratch that it grows with cudaMalloc
// when a larger shape arrives. This entry point runs the same kernels with
// the scratch placed in g_static_scratch below: the split-K arrival counters,
// the prepared fp16 activations with their per-16 sums, and the split-K
// partial sums. Nothing here calls cudaMalloc, cudaFree or a library routine
// that allocates.
#include <mutex>

#include "common.cuh"
#include "gemm_tiled.cuh"

namespace {

constexpr uint64_t STATIC_COUNTER_BYTES = 16 * 1024;  // 4096 split-K arrival counters
static_assert(YUUKA_GEMM_STATIC_SCRATCH_BYTES % 256 == 0 && YUUKA_GEMM_STATIC_SCRATCH_BYTES > STATIC_COUNTER_BYTES,
              "static scratch size");

// One array per device (every device that loads the module gets its own copy).
static __device__ __align__(256) unsigned char g_static_scratch[YUUKA_GEMM_STATIC_SCRATCH_BYTES];

struct StaticSetup {
    bool ready = false;
    unsigned char * base = nullptr;
};
StaticSetup g_setup[16];
std::mutex g_setup_mutex;

uint64_t align256(uint64_t v) { return (v + 255) / 256 * 256; }

// Once per device, with that device current: the array's address on this device,
// zeros in the counters (the kernels leave them at zero after every launch), and
// the code of every kernel the entry point can launch brought onto the device.
unsigned char * static_scratch_base(const yuuka_device * dev) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    StaticSetup & st = g_setup[dev->index];
    if (st.ready) return st.base;
    yk::set_device(dev);
    void * ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    YK_REQUIRE(err == cudaSuccess && ptr != nullptr, YUUKA_ERR_DEVICE, "gemm_quant_static: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(err));
    YK_REQUIRE(((uintptr_t)ptr & 255) == 0, YUUKA_ERR_INTERNAL, "gemm_quant_static: scratch array is not 256-byte aligned");
    YK_CUDA(cudaMemset(ptr, 0, STATIC_COUNTER_BYTES));
    // every kernel the routes below can pick is loaded now: with lazy module loading the driver would
    // otherwise place a kernel's code in device memory at its first launch, in the middle of serving
    yk::gemm_tiled_preload_kernels();
    YK_CUDA(cudaDeviceSynchronize());
    st.base = (unsigned char *)ptr;
    st.ready = true;
    return st.base;
}

}  // namespace

extern "C" yuuka_status yuuka_gemm_quant_static(yuuka_stream * stream, yuuka_buffer * out, uint64_t out_offset,
                                                const yuuka_buffer * x, uint64_t x_offset, uint32_t x_dtype,
                                                const yuuka_buffer * w, uint64_t w_offset, uint32_t w_dtype,
                                                uint64_t n_in, uint64_t n_out, uint64_t rows, uint32_t path,
                                                uint32_t flags, yuuka_event * completion) {
    using namespace yk;
    return guard([&] {
        YK_REQUIRE(stream && out && x && w, YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant_static: null argument");
        YK_REQUIRE(flags & YUUKA_GEMM_TILED, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant_static: reads tile-ordered weights only (YUUKA_GEMM_TILED)");
        YK_REQUIRE(n_in > 0 && n_out > 0 && rows > 0 && n_in < (1u << 20) && n_out < (1u << 28) && rows <= 65536,
                   YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant_static: invalid shape");
        YK_REQUIRE(tiled_supported(w_dtype, n_in), YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant_static: dtype %u with %llu columns has no tiled layout", w_dtype, (unsigned long long)n_in);
        YK_REQUIRE(x_dtype == YUUKA_DTYPE_F32 || x_dtype == YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant_static: activation dtype %u is not F32 or BF16", x_dtype);
        const uint64_t xb = rows * n_in * (x_dtype == YUUKA_DTYPE_F32 ? 4 : 2);
        YK_REQUIRE(w_offset % 16 == 0 && w_offset <= w->bytes && tiled_bytes(w_dtype, n_out, n_in) <= w->bytes - w_offset,
                   YUUKA_ERR_INVALID_ARGUMENT, "gemm_quant_static: tiled weight range exceeds the buffer or is misaligned");
        YK_REQUIRE(x_offset <= x->bytes && xb <= x->bytes - x_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant_static: activation range exceeds the buffer");
        YK_REQUIRE(out_offset <= out->bytes && rows * n_out * 4 <= out->bytes - out_offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant_static: output range exceeds the buffer");
        YK_REQUIRE(x_offset % 16 == 0 && out_offset % 16 == 0, YUUKA_ERR_INVALID_ARGUMENT,
                   "gemm_quant_static: activation and output offsets must be multiples of 16");
        yuuka_device * dev = stream->dev;
        YK_REQUIRE(dev->index >= 0 && dev->index < 16, YUUKA_ERR_UNSUPPORTED, "gemm_quant_static: device index out of range");

        // carve the fixed array: counters | xh | xl | xs16 | split-K partial sums
        uint64_t partial_floats = 0;
        int counters = 0;
        gemm_tiled_scratch_need(dev, w_dtype, (int)rows, (int)n_out, (int)n_in, &partial_floats, &counters);
        const uint64_t xh_bytes = align256(rows * n_in * sizeof(__half));
        const uint64_t xs_bytes = align256(rows * n_in / 16 * sizeof(__half2) + 16);
        const uint64_t need = STATIC_COUNTER_BYTES + 2 * xh_bytes + xs_bytes + align256(partial_floats * sizeof(float));
        YK_REQUIRE((uint64_t)counters * sizeof(int) <= STATIC_COUNTER_BYTES && need <= YUUKA_GEMM_STATIC_SCRATCH_BYTES,
                   YUUKA_ERR_UNSUPPORTED,
                   "gemm_quant_static: rows=%llu n_out=%llu n_in=%llu needs %llu bytes of scratch (%d counters), the fixed "
                   "area holds %llu bytes (%llu counters); use yuuka_gemm_quant",
                   (unsigned long long)rows, (unsigned long long)n_out, (unsigned long long)n_in, (unsigned long long)need,
                   counters, (unsigned long long)YUUKA_GEMM_STATIC_SCRATCH_BYTES,
                   (unsigned long long)(STATIC_COUNTER_BYTES / sizeof(int)));

        unsigned char * base = static_scratch_base(dev);
        GemmScratch sc;
        sc.counters = (int *)base;
        sc.counter_count = (int)(STATIC_COUNTER_BYTES / sizeof(int));
        sc.xh = (__half *)(base + STATIC_COUNTER_BYTES);
        sc.xl = (__half *)(base + STATIC_COUNTER_BYTES + xh_bytes);
        sc.xs16 = (__half2 *)(base + STATIC_COUNTER_BYTES + 2 * xh_bytes);
        sc.xh_elems = rows * n_in;
        sc.partial = (float *)(base + STATIC_COUNTER_BYTES + 2 * xh_bytes + xs_bytes);
        sc.partial_floats = (YUUKA_GEMM_STATIC_SCRATCH_BYTES - STATIC_COUNTER_BYTES - 2 * xh_bytes - xs_bytes) / sizeof(float);

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
    });
}
