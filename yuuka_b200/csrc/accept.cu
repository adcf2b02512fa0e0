// On-device acceptance for a verify step.
//
// Greedy: first-maximum argmax of every logits row (argmaxLogit,
// engine/speculative.go:263-271) and the prefix walk of the accept loop
// (engine/speculative.go:193-202), generalised from a chain to a tree: at node
// cur the wanted token is argmax(logits[cur]); the lowest-numbered child of
// cur that carries it is accepted and becomes cur; otherwise the wanted token
// is emitted as the correction and the walk ends.
#include "layers.cuh"

namespace yk {

constexpr int ARGMAX_CHUNK = 4096;

// (value, index) with the reference's tie rule: larger value wins, equal
// values keep the lower index. NaNs never win against a number.
__device__ __forceinline__ void best_of(float & v, int & i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float * __restrict__ logits, int vocab,
                                                             float * __restrict__ val, int32_t * __restrict__ idx,
                                                             int chunks) {
    pdl_entry();
    const int r = blockIdx.y, c = blockIdx.x;
    const float * row = logits + (int64_t)r * vocab;
    const int begin = c * ARGMAX_CHUNK, end = min(vocab, begin + ARGMAX_CHUNK);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best_of(bv, bi, row[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        best_of(bv, bi, ov, oi);
    }
    __shared__ float sv[8];
    __shared__ int si[8];
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) best_of(bv, bi, sv[w], si[w]);
        val[(int64_t)r * chunks + c] = bv;
        idx[(int64_t)r * chunks + c] = bi;
    }
}

struct WalkParams {
    const float * val;
    const int32_t * idx;
    int chunks;
    RowMeta rows;
    AcceptOut out;
};

// one CTA per sequence: finish the argmax of each of its rows, then walk
__global__ void __launch_bounds__(64) greedy_walk_kernel(const WalkParams p) {
    pdl_entry();
    __shared__ int want[64];
    const int seq = blockIdx.x, N = p.rows.nodes;
    for (int node = threadIdx.x; node < N; node += blockDim.x) {
        const int r = seq * N + node;
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int c = 0; c < p.chunks; c++) best_of(bv, bi, p.val[(int64_t)r * p.chunks + c], p.idx[(int64_t)r * p.chunks + c]);
        want[node] = bi == 0x7fffffff ? 0 : bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int32_t * tokens = p.rows.tokens + (int64_t)seq * N;
        const int32_t * parent = p.rows.parent + (int64_t)seq * N;
        int32_t * path = p.out.path + (int64_t)seq * N;
        int32_t * emitted = p.out.emitted + (int64_t)seq * N;
        int cur = 0, a = 0;
        for (;;) {
            const int w = want[cur];
            int next = -1;
            for (int c = cur + 1; c < N; c++)
                if (parent[c] == cur && tokens[c] == w) { next = c; break; }
            emitted[a] = w;
            if (next < 0) break;
            path[a] = next;
            a++;
            cur = next;
        }
        for (int i = a; i < N; i++) path[i] = -1;
        for (int i = a + 1; i < N; i++) emitted[i] = -1;
        p.out.accepted[seq] = a;
    }
}

int launch_accept_greedy(cudaStream_t s, const float * logits, int vocab, const RowMeta & rows,
                         const ArgmaxScratch & scratch, const AcceptOut & out) {
    const int R = rows.batch * rows.nodes;
    const int chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    YK_REQUIRE(chunks <= scratch.chunks, YUUKA_ERR_INTERNAL, "argmax scratch is too small");
    dim3 grid(chunks, R);
    launch_k(argmax_partial_kernel, grid, 256, 0, s, logits, vocab, scratch.val, scratch.idx, scratch.chunks);
    YK_CUDA(cudaGetLastError());
    WalkParams p{scratch.val, scratch.idx, scratch.chunks, rows, out};
    launch_k(greedy_walk_kernel, rows.batch, 64, 0, s, p);
    YK_CUDA(cudaGetLastError());
    return 2;
}

__global__ void accept_all_kernel(RowMeta rows, AcceptOut out) {
    pdl_entry();
    const int seq = blockIdx.x, N = rows.nodes;
    if (threadIdx.x == 0) out.accepted[seq] = N - 1;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        out.path[(int64_t)seq * N + i] = i + 1 < N ? i + 1 : -1;
        out.emitted[(int64_t)seq * N + i] = i + 1 < N ? rows.tokens[(int64_t)seq * N + i + 1] : -1;
    }
}

void launch_accept_all(cudaStream_t s, const RowMeta & rows, const AcceptOut & out) {
    launch_k(accept_all_kernel, rows.batch, 64, 0, s, rows, out);
    YK_CUDA(cudaGetLastError());
}

int argmax_chunks(int vocab) { return (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK; }

}  // namespace yk
