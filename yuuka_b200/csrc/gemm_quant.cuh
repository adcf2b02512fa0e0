// Host interface of the quantized GEMM kernels (gemm_quant.cu).
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace yk {

struct GemmScratch {
    float * partial = nullptr;   // split-K partial sums [parts][rows][n_out]
    uint64_t partial_floats = 0;
    int * counters = nullptr;    // one arrival counter per tile group, zero between launches
    int counter_count = 0;
    __half * xh = nullptr;       // prepared activations of a launch whose caller passed f32 / bf16
    __half * xl = nullptr;
    __half2 * xs16 = nullptr;
    uint64_t xh_elems = 0;
};

struct GemmArgs {
    const uint8_t * w = nullptr;
    uint64_t w_readable = 0;     // bytes that may be read starting at w
    uint32_t w_dtype = 0;
    const void * x = nullptr;    // [rows][ldx] f32 or bf16
    uint32_t x_dtype = YUUKA_DTYPE_F32;
    int64_t ldx = 0;
    float * out = nullptr;       // [rows][ldo] f32
    int64_t ldo = 0;
    int rows = 0, n_out = 0, n_in = 0;
    uint32_t path = YUUKA_GEMM_PATH_AUTO;
    uint32_t flags = 0;
    GemmScratch * scratch = nullptr;
};

// Enqueues the GEMM on stream. Throws StatusError on invalid arguments.
// Returns the number of kernels launched.
int launch_gemm_quant(const yuuka_device * dev, cudaStream_t stream, const GemmArgs & a);

// Which route AUTO takes for this shape.
uint32_t gemm_auto_path(uint32_t w_dtype, int rows, int n_in);

// Grows (never shrinks) a scratch so it fits a launch of this shape.
void gemm_scratch_reserve(const yuuka_device * dev, GemmScratch & s, uint32_t w_dtype, int rows, int n_out, int n_in);
void gemm_scratch_free(GemmScratch & s);

// Sticky device-side error word: set when a bounded wait inside a kernel gave
// up. Reading it synchronises the device.
int read_device_error(const yuuka_device * dev);
// Back to zero (after the error has been reported): the next steps are judged on their own.
void clear_device_error(const yuuka_device * dev);
void enqueue_device_error_read(cudaStream_t stream, int * out2);

}  // namespace yk
