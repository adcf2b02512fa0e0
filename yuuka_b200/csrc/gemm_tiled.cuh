// Tile-ordered weight layout and the GEMM kernels that read it.
//
// A GGUF matrix [n_out][row_bytes] is re-ordered once, byte for byte, into
// records of 16 rows x 256 columns (one K-quant superblock per row): record
// (rt, sb) holds rows 16*rt .. 16*rt+15, columns 256*sb .. 256*sb+255, with the
// bytes placed in the order the 32 lanes of a warp consume them. A warp then
// streams a 16-row tile along K with fully coalesced 512-byte loads, every
// address 16-byte aligned whatever the GGUF row alignment was (Q6_K rows are
// only 2-byte aligned). The re-ordering is a permutation: dequantized values
// are bit-identical to the GGUF tensor's.
#pragma once

#include "gemm_quant.cuh"
#include "xprep.cuh"

namespace yk {

// Bytes of one 16-row x 256-column record; 0 if the dtype has no tiled form.
inline int tiled_record_bytes(uint32_t dtype) {
    switch (dtype) {
    case YUUKA_DTYPE_Q4_K: return 16 * 144;
    case YUUKA_DTYPE_Q5_K: return 16 * 176;
    case YUUKA_DTYPE_Q6_K: return 16 * 210;
    case YUUKA_DTYPE_Q8_0: return 16 * 272;
    default: return 0;
    }
}
inline bool tiled_supported(uint32_t dtype, uint64_t n_in) { return tiled_record_bytes(dtype) != 0 && n_in % 256 == 0; }
inline uint64_t tiled_bytes(uint32_t dtype, uint64_t n_out, uint64_t n_in) {
    return ((n_out + 15) / 16) * (n_in / 256) * (uint64_t)tiled_record_bytes(dtype);
}

// dst (tiled_bytes long) <- GGUF rows at src. Rows beyond n_out are zero.
void launch_tile_weights(cudaStream_t s, uint8_t * dst, const uint8_t * src, uint32_t dtype, int n_out, int n_in);

// One run of at most 8 consecutive rows bound to one expert matrix (grouped GEMM). count <= 0 marks
// an unused slot: the list has a fixed length so that the launch shape does not depend on the routing.
struct GemmSegment {
    int32_t expert;
    int32_t row0;
    int32_t count;
    int32_t reserved;
};
constexpr int GEMM_SEGMENT_ROWS = 8;

// out[row0 + i][:] = x[row(row0 + i)][:] * W[expert]^T for every segment, W[e] = w + e * expert_stride
// (tile-ordered, n_out x n_in each). row(j) = row_index[j] if given, else j.
struct GroupedGemmArgs {
    const uint8_t * w = nullptr;
    uint32_t w_dtype = 0;
    size_t expert_stride = 0;
    XPrepOut xprep;
    const int32_t * row_index = nullptr;
    float * out = nullptr;
    int64_t ldo = 0;
    int n_out = 0, n_in = 0;
    const GemmSegment * segments = nullptr;  // device
    int max_segments = 0;
};
int launch_gemm_tiled_grouped(const yuuka_device * dev, cudaStream_t stream, const GroupedGemmArgs & a);

// RMSNorm folded into the GEMMs around it (register-fed mma route, up to 32 rows). A GEMM that finishes
// residual rows x (producer) also writes the prepared input of the next GEMM, fp16(x * w * pre) with its
// 16-column sums, and adds every row's sum of squares (fixed point, 2^-24 units, integer atomics: the
// result does not depend on the order of the CTAs) to produce_sumsq, which the caller zeroed. The GEMM
// that reads those rows (consumer) multiplies its output rows by scale / pre, scale = 1 / rms(x) from
// consume_now. pre = the scale of the row at the previous norm (produce_prev / consume_prev, null: 1)
// keeps the unnormalised fp16 values near unit range whatever the magnitude of the residual stream.
struct NormFuse {
    const float * produce_w = nullptr;
    const unsigned long long * produce_prev = nullptr;
    unsigned long long * produce_sumsq = nullptr;
    XPrepOut produce_prep;
    const unsigned long long * consume_now = nullptr;
    const unsigned long long * consume_prev = nullptr;
    float eps = 0.0f;
    int cols = 0;
};

struct TiledGemmArgs {
    const uint8_t * w = nullptr;  // tiled layout
    uint32_t w_dtype = 0;
    const void * x = nullptr;     // f32 / bf16 activations (fp32 route, or to be prepared into the scratch)
    XPrepOut xprep;               // prepared activations [rows][n_in], if a producer already made them
    uint32_t x_dtype = YUUKA_DTYPE_F32;
    int64_t ldx = 0;
    float * out = nullptr;
    int64_t ldo = 0;
    int rows = 0, n_out = 0, n_in = 0;
    uint32_t path = YUUKA_GEMM_PATH_AUTO;
    uint32_t flags = 0;
    bool exact_only = false;          // wide passes too stay on the register-fed route (16 rows per launch)
    bool wide_from_33 = false;        // 33..47 rows take the tensor-memory route as well
    GemmScratch * scratch = nullptr;  // needed when the plan splits K across CTAs
    NormFuse norm;
    // Set: `w` holds ffn_gate and ffn_up interleaved by 16-row tile and the launch writes silu(gate) * up in
    // prepared form, [rows][n_out / 2], instead of `out` (register-fed mma route, up to 32 rows).
    XPrepOut swiglu;
    const uint8_t * next_w = nullptr;  // optional L2 prefetch hint: the next matrix to be streamed (mma route)
    uint64_t next_bytes = 0;
};

int launch_gemm_tiled(const yuuka_device * dev, cudaStream_t stream, const TiledGemmArgs & a);
// Scratch the launch above needs for this shape (0 partial floats when K is not split across CTAs).
void gemm_tiled_scratch_need(const yuuka_device * dev, uint32_t w_dtype, int rows, int n_out, int n_in,
                             uint64_t * partial_floats, int * counters);

// Makes the driver load the code of every kernel launch_gemm_tiled can launch (the current device).
void gemm_tiled_preload_kernels();

// Non-zero once a bounded wait inside a GEMM kernel has expired (sticky).
int read_gemm_wait_expired();
void clear_gemm_wait_expired();
void enqueue_gemm_wait_expired_read(cudaStream_t stream, int * out);

}  // namespace yk
