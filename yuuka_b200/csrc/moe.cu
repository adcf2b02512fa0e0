// qwen35moe feed-forward block on the device (model/qwen35/forward.go:320-458):
// router logits -> top-k experts by repeated argmax (lowest index wins ties) ->
// softmax over the selected logits only -> grouping of the (row, slot) pairs by
// expert -> the combine  x += sum_slot w * expert_out + sigmoid(gate) * shared_out.
// The expert matrices themselves run through the grouped tiled GEMM.
#include <cfloat>

#include "gemm_tiled.cuh"
#include "layers.cuh"

namespace yk {

constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_MAX_EXPERTS = 1024;

struct RouteParams {
    const float * xn;       // [rows][hidden] normalised activations
    const float * router;   // [experts][hidden] f32
    const float * sh_gate;  // [hidden] f32 (shared-expert gate vector)
    int hidden, experts, used;
    int32_t * ids;          // [rows][used]
    float * weights;        // [rows][used]
    float * shared_gate;    // [rows]
};

constexpr int ROUTE_ROWS = 8;      // rows per CTA: a router row is read once per eight activation rows
constexpr int ROUTE_EXPERTS = 32;  // router rows per CTA: four per warp

// grid (row groups, expert groups). A warp takes four router rows and all eight activation rows: 16-byte
// weight loads shared by the rows, 32 accumulators per lane; a dot product is summed by lanes in a fixed
// order (the CPU reference sums sequentially, so logits agree to rounding, not bit for bit). Logits go to
// global memory; the last CTA of a row group to arrive (atomic counter, no waiting) selects the experts
// of its eight rows, one warp per row.
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const RouteParams p, int rows, float * logits, int * counters) {
    pdl_entry();
    extern __shared__ __align__(16) float sm[];
    float * x = sm;  // [ROUTE_ROWS][hidden]
    __shared__ int last_flag;
    const int r0 = blockIdx.x * ROUTE_ROWS, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nr = min(ROUTE_ROWS, rows - r0);
    const int n_vec = p.experts + 1;  // index `experts` is the shared-expert gate vector
    for (int i = threadIdx.x; i < ROUTE_ROWS * (p.hidden / 4); i += ROUTE_THREADS) {
        const int rr = i / (p.hidden / 4), c = i - rr * (p.hidden / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rr < nr) v = reinterpret_cast<const float4 *>(p.xn + (int64_t)(r0 + rr) * p.hidden)[c];
        reinterpret_cast<float4 *>(x + rr * p.hidden)[c] = v;
    }
    __syncthreads();
    const int e0 = blockIdx.y * ROUTE_EXPERTS + warp * 4;
    if (e0 < n_vec) {
        const float * w[4];
        float acc[4][ROUTE_ROWS];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int e = min(e0 + q, n_vec - 1);
            w[q] = e < p.experts ? p.router + (int64_t)e * p.hidden : p.sh_gate;
#pragma unroll
            for (int rr = 0; rr < ROUTE_ROWS; rr++) acc[q][rr] = 0.0f;
        }
#pragma unroll 2
        for (int i = lane * 4; i < p.hidden; i += 128) {
            float4 wv[4];
#pragma unroll
            for (int q = 0; q < 4; q++) wv[q] = __ldg(reinterpret_cast<const float4 *>(w[q] + i));
#pragma unroll
            for (int rr = 0; rr < ROUTE_ROWS; rr++) {
                const float4 xv = *reinterpret_cast<const float4 *>(x + rr * p.hidden + i);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    acc[q][rr] = fmaf(wv[q].x, xv.x, acc[q][rr]);
                    acc[q][rr] = fmaf(wv[q].y, xv.y, acc[q][rr]);
                    acc[q][rr] = fmaf(wv[q].z, xv.z, acc[q][rr]);
                    acc[q][rr] = fmaf(wv[q].w, xv.w, acc[q][rr]);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int e = e0 + q;
#pragma unroll
            for (int rr = 0; rr < ROUTE_ROWS; rr++) {
                float v = acc[q][rr];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && e < n_vec && rr < nr) {
                    if (e < p.experts) __stcg(logits + (int64_t)(r0 + rr) * p.experts + e, v);
                    else p.shared_gate[r0 + rr] = 1.0f / (1.0f + (float)exp((double)-v));
                }
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_flag = atomicAdd(&counters[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;
    if (warp >= nr) return;
    const int r = r0 + warp;
    float * logit = sm + warp * p.experts;  // (the activation rows in shared memory are no longer needed)
    __syncwarp();
    for (int e = lane; e < p.experts; e += 32) logit[e] = __ldcg(logits + (int64_t)r * p.experts + e);
    __syncwarp();
    // selectExperts (forward.go:393-439): `used` rounds of first-maximum argmax over the experts not yet taken
    int32_t * ids = p.ids + (int64_t)r * p.used;
    float * wts = p.weights + (int64_t)r * p.used;
    float my_logit = 0.0f;  // lane s keeps the logit of slot s (used <= 32)
    for (int slot = 0; slot < p.used; slot++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < p.experts; e += 32) {
            const float v = logit[e];
            if (v != v) continue;  // taken (marked NaN below)
            if (bi == 0x7fffffff || v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;
        if (lane == slot) my_logit = bv;
        if (lane == 0) {
            ids[slot] = bi;
            logit[bi] = __int_as_float(0x7fc00000);
        }
        __syncwarp();
    }
    // softmax over the selected logits: exp in double, sum in float in slot order
    float mx = lane < p.used ? my_logit : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float w = lane < p.used ? (float)exp((double)(my_logit - mx)) : 0.0f;
    float total = 0.0f;
    for (int s = 0; s < p.used; s++) total += __shfl_sync(0xffffffffu, w, s);
    if (lane < p.used) wts[lane] = total > 0.0f ? w / total : w;
}

struct GroupParams {
    const int32_t * ids;     // [pairs] expert of pair p = row * used + slot
    int pairs, used, experts, max_segments;
    int32_t * pos_of_pair;   // [pairs] position of the pair in the expert-sorted order
    int32_t * row_of_pos;    // [pairs] source row of the pair at a position
    GemmSegment * segments;  // [max_segments]
};

// One CTA. Stable counting sort of the pairs by expert, cut into segments of at most 8 rows: counts by
// shared-memory atomics, offsets by a warp scan over the experts, then one warp walks the pairs 32 at a
// time in order, __match_any_sync giving every pair its rank among the equal experts of its group and a
// per-expert cursor carrying the ranks from group to group. (A first form had one thread per expert scan
// all pairs twice: 110 us for 1280 pairs and 256 experts, now a few.)
__global__ void __launch_bounds__(ROUTE_THREADS) moe_group_kernel(const GroupParams p) {
    pdl_entry();
    __shared__ int count[ROUTE_MAX_EXPERTS];
    __shared__ int pair_off[ROUTE_MAX_EXPERTS];
    __shared__ int seg_off[ROUTE_MAX_EXPERTS];
    __shared__ int cursor[ROUTE_MAX_EXPERTS];
    __shared__ int total_segments;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < p.experts; e += ROUTE_THREADS) {
        count[e] = 0;
        cursor[e] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.pairs; i += ROUTE_THREADS) atomicAdd(&count[p.ids[i]], 1);
    __syncthreads();
    if (warp == 0) {
        // exclusive scans of the pair counts and of the segment counts: a lane sums its run of experts, the
        // runs are scanned across the warp, then every lane walks its run again
        const int per = (p.experts + 31) / 32, e0 = lane * per, e1 = min(p.experts, e0 + per);
        int pairs_run = 0, segs_run = 0;
        for (int e = e0; e < e1; e++) {
            pairs_run += count[e];
            segs_run += (count[e] + GEMM_SEGMENT_ROWS - 1) / GEMM_SEGMENT_ROWS;
        }
        int pairs_before = pairs_run, segs_before = segs_run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, pairs_before, o), b = __shfl_up_sync(0xffffffffu, segs_before, o);
            if (lane >= o) {
                pairs_before += a;
                segs_before += b;
            }
        }
        if (lane == 31) total_segments = segs_before;
        pairs_before -= pairs_run;
        segs_before -= segs_run;
        for (int e = e0; e < e1; e++) {
            pair_off[e] = pairs_before;
            seg_off[e] = segs_before;
            pairs_before += count[e];
            segs_before += (count[e] + GEMM_SEGMENT_ROWS - 1) / GEMM_SEGMENT_ROWS;
        }
    }
    __syncthreads();
    if (warp == 0) {
        for (int base = 0; base < p.pairs; base += 32) {
            const int i = base + lane;
            const bool valid = i < p.pairs;
            const int e = valid ? p.ids[i] : -1 - lane;  // (lanes past the end match nobody)
            const unsigned same = __match_any_sync(0xffffffffu, e);
            const int leader = __ffs(same) - 1, rank = __popc(same & ((1u << lane) - 1u));
            int start = 0;
            if (valid && lane == leader) {
                start = cursor[e];
                cursor[e] = start + __popc(same);
            }
            start = __shfl_sync(0xffffffffu, start, leader);
            __syncwarp();
            if (valid) {
                const int j = start + rank, c = count[e], pos = pair_off[e] + j;
                p.pos_of_pair[i] = pos;
                p.row_of_pos[pos] = i / p.used;
                if (j % GEMM_SEGMENT_ROWS == 0) {
                    const int z = seg_off[e] + j / GEMM_SEGMENT_ROWS;
                    if (z < p.max_segments) p.segments[z] = GemmSegment{e, pos, min(GEMM_SEGMENT_ROWS, c - j), 0};
                }
            }
        }
    }
    for (int z = total_segments + threadIdx.x; z < p.max_segments; z += ROUTE_THREADS) p.segments[z] = GemmSegment{0, 0, 0, 0};
}

int moe_max_segments(int pairs, int experts) {
    const int by_rows = pairs / GEMM_SEGMENT_ROWS + (experts < pairs ? experts : pairs);
    return by_rows < pairs ? by_rows : pairs;
}

void launch_moe_route(cudaStream_t s, const float * xn, const float * router, const float * sh_gate, int hidden, int experts,
                      int used, int rows, int32_t * ids, float * weights, float * shared_gate, float * logits, int * counters) {
    YK_REQUIRE(hidden % 4 == 0, YUUKA_ERR_UNSUPPORTED, "moe: hidden size %d is not a multiple of 4", hidden);
    YK_REQUIRE(experts <= ROUTE_MAX_EXPERTS && used <= 32 && used <= experts, YUUKA_ERR_UNSUPPORTED,
               "moe: %d experts / %d used exceeds the router kernel's limits (%d / 32)", experts, used, ROUTE_MAX_EXPERTS);
    YK_REQUIRE(experts <= hidden, YUUKA_ERR_UNSUPPORTED, "moe: more experts (%d) than hidden columns (%d)", experts, hidden);
    RouteParams p{xn, router, sh_gate, hidden, experts, used, ids, weights, shared_gate};
    const size_t smem = sizeof(float) * (size_t)ROUTE_ROWS * (size_t)hidden;
    YK_REQUIRE(smem <= 200 * 1024, YUUKA_ERR_UNSUPPORTED, "moe: hidden size %d is too wide for the router kernel", hidden);
    YK_CUDA(cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((rows + ROUTE_ROWS - 1) / ROUTE_ROWS, (experts + 1 + ROUTE_EXPERTS - 1) / ROUTE_EXPERTS);
    launch_k(moe_route_kernel, grid, ROUTE_THREADS, smem, s, p, rows, logits, counters);
    YK_CUDA(cudaGetLastError());
}

void launch_moe_group(cudaStream_t s, const int32_t * ids, int rows, int used, int experts, int32_t * pos_of_pair,
                      int32_t * row_of_pos, GemmSegment * segments, int max_segments) {
    GroupParams p{ids, rows * used, used, experts, max_segments, pos_of_pair, row_of_pos, segments};
    launch_k(moe_group_kernel, 1, ROUTE_THREADS, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

struct CombineParams {
    float * x;                 // [rows][hidden] residual stream, updated in place
    const float * expert_out;  // [pairs][hidden] in expert-sorted order
    const float * shared_out;  // [rows][hidden]
    const int32_t * pos_of_pair;
    const float * weights;     // [rows][used]
    const float * shared_gate; // [rows]
    int hidden, used;
};

// forward.go:370-389, same order of operations: tmp = sum over slots of w * out (slot order), then
// + gate * shared, then x += tmp; products and sums rounded separately as the reference does.
__global__ void moe_combine_kernel(const CombineParams p) {
    pdl_entry();
    const int r = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.hidden) return;
    float tmp = 0.0f;
    for (int s = 0; s < p.used; s++) {
        const int pos = p.pos_of_pair[r * p.used + s];
        tmp = __fadd_rn(tmp, __fmul_rn(p.weights[r * p.used + s], p.expert_out[(int64_t)pos * p.hidden + i]));
    }
    tmp = __fadd_rn(tmp, __fmul_rn(p.shared_gate[r], p.shared_out[(int64_t)r * p.hidden + i]));
    float * dst = p.x + (int64_t)r * p.hidden + i;
    *dst = __fadd_rn(*dst, tmp);
}

void launch_moe_combine(cudaStream_t s, float * x, const float * expert_out, const float * shared_out,
                        const int32_t * pos_of_pair, const float * weights, const float * shared_gate, int hidden, int used,
                        int rows) {
    CombineParams p{x, expert_out, shared_out, pos_of_pair, weights, shared_gate, hidden, used};
    dim3 grid((hidden + 255) / 256, rows);
    launch_k(moe_combine_kernel, grid, 256, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

}  // namespace yk
