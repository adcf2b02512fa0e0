// On-device acceptance for a verify step.
//
// Greedy: first-maximum argmax of every logits row (argmaxLogit,
// engine/speculative.go:263-271) and the prefix walk of the accept loop
// (engine/speculative.go:193-202), generalised from a chain to a tree: at node
// cur the wanted token is argmax(logits[cur]); the lowest-numbered child of
// cur that carries it is accepted and becomes cur; otherwise the wanted token
// is emitted as the correction and the walk ends.
#include <vector>

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

// one CTA per sequence: finish the argmax of each of its rows (a warp per row, lanes over the chunk maxima,
// combined with the same tie rule), then one thread walks the tree, whose tokens and parents wait in shared memory
constexpr int WALK_THREADS = 256;
__global__ void __launch_bounds__(WALK_THREADS) greedy_walk_kernel(const WalkParams p) {
    pdl_entry();
    __shared__ int want[64], tok_s[64], par_s[64];
    const int seq = blockIdx.x, N = p.rows.nodes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int node = threadIdx.x; node < N; node += blockDim.x) {
        tok_s[node] = p.rows.tokens[(int64_t)seq * N + node];
        par_s[node] = p.rows.parent[(int64_t)seq * N + node];
    }
    for (int node = warp; node < N; node += WALK_THREADS / 32) {
        const int r = seq * N + node;
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int c = lane; c < p.chunks; c += 32) best_of(bv, bi, p.val[(int64_t)r * p.chunks + c], p.idx[(int64_t)r * p.chunks + c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            best_of(bv, bi, ov, oi);
        }
        if (lane == 0) want[node] = bi == 0x7fffffff ? 0 : bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t * path = p.out.path + (int64_t)seq * N;
        int32_t * emitted = p.out.emitted + (int64_t)seq * N;
        int cur = 0, a = 0;
        for (;;) {
            const int w = want[cur];
            int next = -1;
            for (int c = cur + 1; c < N; c++)
                if (par_s[c] == cur && tok_s[c] == w) { next = c; break; }
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
    launch_k(greedy_walk_kernel, rows.batch, WALK_THREADS, 0, s, p);
    YK_CUDA(cudaGetLastError());
    return 2;
}

// ---------------------------------------------------------------------------
// Rejection-sampling acceptance over a draft tree (not in the reference, which
// verifies greedily only: engine/speculative.go:73-75). The rule is written so
// that every deciding quantity is an elementwise IEEE operation or an integer
// sum; the result does not depend on the order of the parallel reductions.
//
// At node cur (start: the root), with children in row order:
//   mx  = max_i L[cur][i];  e_i = exp_det((L[cur][i] - mx) / T);  w_i = (uint64)(e_i * 2^40)
//   r = w, R = sum w
//   child c (token x, draft distribution Q[c], uniform u = U[2c]):
//     accept iff (double)(u * Q[c][x]) * (double)R <= (double)r_x      -> cur = c, start over at c
//     else r_i = max(0, r_i - (uint64)((double)Q[c][i] * (double)R)), R = sum r  (R == 0: r = w again)
//   no child accepted: t = min((uint64)((double)U[2 cur + 1] * (double)R), R - 1);
//     emit the smallest j with sum_{i <= j} r_i > t.

__device__ __forceinline__ float exp_det(float x) {
    if (x < -87.0f) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    const float n = rintf(x * 1.44269504f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = __fmul_rn(r, r);
    const float e = __fadd_rn(fmaf(p, r2, r), 1.0f);
    const float scale = __uint_as_float((uint32_t)((int)n + 127) << 23);
    return __fmul_rn(e, scale);
}

__device__ __forceinline__ unsigned long long target_weight(float logit, float mx, float inv_t) {
    const float e = exp_det(__fmul_rn(__fsub_rn(logit, mx), inv_t));
    return (unsigned long long)__fmul_rn(e, 1099511627776.0f);
}

constexpr int REJ_THREADS = 1024;
constexpr int REJ_CLUSTER = 8;          // CTAs that share one sequence's vocabulary when it is large
constexpr int REJ_CLUSTER_MIN_VOCAB = 32768;

struct RejectParams {
    const float * logits;   // [batch][nodes][vocab]
    const float * q;        // [batch][nodes][vocab]
    const float * u;        // [batch][nodes][2]
    unsigned long long * r; // [batch][vocab]
    int vocab;
    float inv_t;
    RowMeta rows;
    AcceptOut out;
};

// Sums and maxima over the CL CTAs that walk one sequence together. Every CTA reduces its own slice, leaves the
// result in one of two shared-memory slots (alternating: a CTA can only be one exchange ahead of the slowest,
// because the hardware barrier of exchange k + 1 needs every CTA to have finished reading exchange k), and reads
// all CL slots after the cluster barrier. Integer sums and float maxima do not depend on the order, so every
// CTA holds the same value and takes the same branches. CL = 1 degenerates to the block reduction.
template <int CL> struct RejectExchange {
    unsigned long long * red;   // [REJ_THREADS / 32]
    unsigned long long * slot;  // [2]
    int turn = 0;

    __device__ unsigned long long block_sum(unsigned long long v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        __syncthreads();  // red may still be read from the previous use
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        unsigned long long t = 0;
        for (int w = 0; w < REJ_THREADS / 32; w++) t += red[w];
        return t;
    }
    __device__ float block_max(float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = (unsigned long long)__float_as_uint(v);
        __syncthreads();
        for (int w = 0; w < REJ_THREADS / 32; w++) v = fmaxf(v, __uint_as_float((uint32_t)red[w]));
        return v;
    }
    // total over the cluster; *before (if given) receives the sum over the CTAs of lower rank
    __device__ unsigned long long sum(unsigned long long v, unsigned long long * before = nullptr) {
        const unsigned long long mine = block_sum(v);
        if constexpr (CL == 1) {
            if (before) *before = 0;
            return mine;
        } else {
            if (threadIdx.x == 0) slot[turn] = mine;
            cluster_sync_all();
            unsigned long long tot = 0, low = 0;
            const unsigned me = cluster_cta_rank();
            for (unsigned c = 0; c < (unsigned)CL; c++) {
                const unsigned long long x = ld_cluster_u64(slot + turn, c);
                if (c < me) low += x;
                tot += x;
            }
            if (before) *before = low;
            turn ^= 1;
            return tot;
        }
    }
    __device__ float max(float v) {
        v = block_max(v);
        if constexpr (CL == 1) {
            return v;
        } else {
            if (threadIdx.x == 0) slot[turn] = (unsigned long long)__float_as_uint(v);
            cluster_sync_all();
            for (unsigned c = 0; c < (unsigned)CL; c++) v = fmaxf(v, __uint_as_float((uint32_t)ld_cluster_u64(slot + turn, c)));
            turn ^= 1;
            return v;
        }
    }
    // orders this cluster's global writes (the residual weights) before the reads that follow in other CTAs
    __device__ void sync() {
        if constexpr (CL == 1) __syncthreads();
        else cluster_sync_all();
    }
};

// One sequence per cluster of CL CTAs; CTA c of the cluster owns the vocabulary slice [c * slice, (c + 1) * slice).
// All CTAs of a cluster walk the tree together: the deciding quantities (R, r[x], q[x], the uniforms) are the
// same everywhere, so they take the same turns; only rank 0 writes the path.
template <int CL>
__global__ void __launch_bounds__(REJ_THREADS) rejection_walk_kernel(const RejectParams p) {
    pdl_entry();
    __shared__ unsigned long long red[REJ_THREADS / 32];
    __shared__ unsigned long long slot[2];
    __shared__ int flag;
    RejectExchange<CL> ex{red, slot};
    const unsigned rank = CL == 1 ? 0u : cluster_cta_rank();
    const int seq = blockIdx.x / CL, N = p.rows.nodes, V = p.vocab, tid = threadIdx.x;
    const int slice = CL == 1 ? V : (((V + CL - 1) / CL + 3) & ~3);
    const int v0 = min(V, (int)rank * slice), v1 = min(V, v0 + slice);
    const int32_t * tokens = p.rows.tokens + (int64_t)seq * N;
    const int32_t * parent = p.rows.parent + (int64_t)seq * N;
    const float * U = p.u + (int64_t)seq * N * 2;
    unsigned long long * r = p.r + (int64_t)seq * V;
    int32_t * path = p.out.path + (int64_t)seq * N;
    int32_t * emitted = p.out.emitted + (int64_t)seq * N;
    int cur = 0, a = 0;
    for (;;) {
        const float * L = p.logits + ((int64_t)seq * N + cur) * V;
        // max of the row (order-independent)
        float mx = -INFINITY;
        for (int i = v0 + tid; i < v1; i += REJ_THREADS) mx = fmaxf(mx, L[i]);
        mx = ex.max(mx);
        // target weights
        unsigned long long z = 0;
        for (int i = v0 + tid; i < v1; i += REJ_THREADS) {
            const unsigned long long w = target_weight(L[i], mx, p.inv_t);
            r[i] = w;
            z += w;
        }
        const unsigned long long Z = ex.sum(z);  // (its barrier also publishes r)
        unsigned long long R = Z;
        int next = -1;
        for (int c = cur + 1; c < N && next < 0; c++) {
            if (parent[c] != cur) continue;
            const float * q = p.q + ((int64_t)seq * N + c) * V;
            __syncthreads();  // flag of the previous child has been read
            if (tid == 0) {
                const int32_t x = tokens[c];
                const float lhs = __fmul_rn(U[2 * c], q[x]);
                flag = __dmul_rn((double)lhs, (double)R) <= (double)__ldcg(r + x);
            }
            __syncthreads();
            if (flag) {
                next = c;
                break;
            }
            if constexpr (CL > 1) ex.sync();  // every CTA has read r[x] before its owner rewrites it
            unsigned long long sum = 0;
            for (int i = v0 + tid; i < v1; i += REJ_THREADS) {
                const unsigned long long qr = (unsigned long long)__dmul_rn((double)q[i], (double)R);
                const unsigned long long ri = r[i];
                const unsigned long long nr = ri > qr ? ri - qr : 0ull;
                r[i] = nr;
                sum += nr;
            }
            R = ex.sum(sum);
            if (R == 0) {
                for (int i = v0 + tid; i < v1; i += REJ_THREADS) r[i] = target_weight(L[i], mx, p.inv_t);
                R = Z;
                ex.sync();
            }
        }
        if (next >= 0) {
            if (tid == 0 && rank == 0) {
                emitted[a] = tokens[next];
                path[a] = next;
            }
            a++;
            cur = next;
            if constexpr (CL > 1) ex.sync();  // r[x] has been read everywhere before the next node rewrites r
            continue;
        }
        // residual draw: the smallest j whose inclusive prefix sum over r exceeds t. Thread tid of CTA c owns the
        // contiguous range [lo, hi) of c's slice.
        unsigned long long t = (unsigned long long)__dmul_rn((double)U[2 * cur + 1], (double)R);
        if (t >= R) t = R - 1;
        const int per = (v1 - v0 + REJ_THREADS - 1) / REJ_THREADS;
        const int lo = min(v1, v0 + tid * per), hi = min(v1, lo + per);
        unsigned long long mine = 0;
        for (int i = lo; i < hi; i++) mine += r[i];
        unsigned long long below = 0;
        ex.sum(mine, &below);  // total of the slices of lower rank
        // exclusive prefix of the per-thread sums: inside the warp, then across warps
        unsigned long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((tid & 31) >= o) incl += v;
        }
        __syncthreads();
        if ((tid & 31) == 31) red[tid >> 5] = incl;
        __syncthreads();
        unsigned long long before = below + incl - mine;
        for (int w = 0; w < (tid >> 5); w++) before += red[w];
        if (before <= t && t < before + mine) {
            unsigned long long acc = before;
            for (int i = lo; i < hi; i++) {
                acc += r[i];
                if (acc > t) {
                    emitted[a] = i;  // exactly one thread of the cluster: t < R = the total
                    break;
                }
            }
        }
        break;
    }
    if (rank == 0) {
        for (int i = a + tid; i < N; i += REJ_THREADS) path[i] = -1;
        for (int i = a + 1 + tid; i < N; i += REJ_THREADS) emitted[i] = -1;
        if (tid == 0) p.out.accepted[seq] = a;
    }
    if constexpr (CL > 1) cluster_sync_all();  // no CTA leaves while another may still read its slots
}

int launch_accept_rejection(cudaStream_t s, const float * logits, const float * draft_probs, const float * uniforms,
                            unsigned long long * residual, int vocab, float temperature, const RowMeta & rows,
                            const AcceptOut & out) {
    YK_REQUIRE(temperature > 0.0f, YUUKA_ERR_INVALID_ARGUMENT, "rejection sampling needs a temperature above zero");
    RejectParams p{logits, draft_probs, uniforms, residual, vocab, 1.0f / temperature, rows, out};
    if (vocab >= REJ_CLUSTER_MIN_VOCAB)
        launch_k_cluster(rejection_walk_kernel<REJ_CLUSTER>, dim3(rows.batch * REJ_CLUSTER), REJ_THREADS, 0, s, REJ_CLUSTER, p);
    else
        launch_k(rejection_walk_kernel<1>, rows.batch, REJ_THREADS, 0, s, p);
    YK_CUDA(cudaGetLastError());
    return 1;
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

// ---------------------------------------------------------------------------
// Kernel-level entry point: acceptance over logits that are already on the device (the acceptance case of the
// kernel microbenchmark; hosts whose logits come from elsewhere). Row metadata and scratch live for the call.
extern "C" yuuka_status yuuka_accept_tree(yuuka_stream * stream, const yuuka_buffer * logits, int32_t batch, int32_t nodes,
                                          int32_t vocab, const int32_t * tokens, const int32_t * parent, uint32_t mode,
                                          float temperature, const yuuka_buffer * draft_probs, const float * uniforms,
                                          int32_t * accepted, int32_t * emitted, int32_t * path, yuuka_event * begin,
                                          yuuka_event * end) {
    using namespace yk;
    return guard([&] {
        YK_REQUIRE(stream && logits && tokens && accepted && emitted, YUUKA_ERR_INVALID_ARGUMENT, "accept_tree: null argument");
        YK_REQUIRE(batch > 0 && nodes > 0 && nodes <= 64 && vocab > 0, YUUKA_ERR_INVALID_ARGUMENT, "accept_tree: invalid shape");
        YK_REQUIRE(mode == YUUKA_ACCEPT_GREEDY || mode == YUUKA_ACCEPT_REJECTION, YUUKA_ERR_INVALID_ARGUMENT,
                   "accept_tree: unknown acceptance mode %u", mode);
        const uint64_t R = (uint64_t)batch * nodes, need = R * (uint64_t)vocab * sizeof(float);
        YK_REQUIRE(logits->bytes >= need, YUUKA_ERR_INVALID_ARGUMENT, "accept_tree: logits buffer holds fewer than %llu bytes",
                   (unsigned long long)need);
        if (mode == YUUKA_ACCEPT_REJECTION) {
            YK_REQUIRE(temperature > 0.0f && temperature == temperature, YUUKA_ERR_INVALID_ARGUMENT,
                       "accept_tree: rejection sampling needs a temperature above zero");
            YK_REQUIRE(uniforms && draft_probs && draft_probs->bytes >= need, YUUKA_ERR_INVALID_ARGUMENT,
                       "accept_tree: rejection sampling needs uniforms and a draft_probs buffer of %llu bytes", (unsigned long long)need);
            for (uint64_t i = 0; i < R * 2; i++)
                YK_REQUIRE(uniforms[i] >= 0.0f && uniforms[i] < 1.0f, YUUKA_ERR_INVALID_ARGUMENT,
                           "accept_tree: uniform draw %llu is outside [0, 1)", (unsigned long long)i);
        }
        // row metadata on the host
        std::vector<int32_t> par(R), dep(R);
        std::vector<unsigned long long> anc(R);
        for (int b = 0; b < batch; b++)
            for (int i = 0; i < nodes; i++) {
                const size_t r = (size_t)b * nodes + i;
                YK_REQUIRE(tokens[r] >= 0 && tokens[r] < vocab, YUUKA_ERR_INVALID_ARGUMENT, "token id %d is out of range", tokens[r]);
                const int p = parent ? parent[r] : i - 1;
                YK_REQUIRE((i == 0 && p == -1) || (i > 0 && p >= 0 && p < i), YUUKA_ERR_INVALID_ARGUMENT,
                           "parent[%d][%d] = %d is not a preceding row", b, i, p);
                par[r] = p;
                dep[r] = i == 0 ? 0 : dep[(size_t)b * nodes + p] + 1;
                anc[r] = (i == 0 ? 0ull : anc[(size_t)b * nodes + p]) | (1ull << i);
            }
        set_device(stream->dev);
        const int chunks = argmax_chunks(vocab);
        // one allocation: anc | tokens | parent | depth | accepted | path | emitted | uniforms | argmax val, idx | residual
        const size_t o_anc = 0, o_tok = o_anc + R * 8, o_par = o_tok + R * 4, o_dep = o_par + R * 4, o_acc = o_dep + R * 4,
                     o_path = o_acc + (size_t)batch * 4, o_em = o_path + R * 4, o_uni = o_em + R * 4, o_val = o_uni + R * 8,
                     o_idx = o_val + R * chunks * 4, o_res = ((o_idx + R * chunks * 4 + 255) / 256) * 256,
                     total = o_res + (mode == YUUKA_ACCEPT_REJECTION ? (size_t)batch * vocab * 8 : 0);
        uint8_t * d = nullptr;
        YK_REQUIRE(cudaMalloc((void **)&d, total) == cudaSuccess, YUUKA_ERR_ALLOCATION, "accept_tree: scratch allocation of %llu bytes failed",
                   (unsigned long long)total);
        try {
            cudaStream_t st = stream->s;
            YK_CUDA(cudaMemcpyAsync(d + o_anc, anc.data(), R * 8, cudaMemcpyHostToDevice, st));
            YK_CUDA(cudaMemcpyAsync(d + o_tok, tokens, R * 4, cudaMemcpyHostToDevice, st));
            YK_CUDA(cudaMemcpyAsync(d + o_par, par.data(), R * 4, cudaMemcpyHostToDevice, st));
            YK_CUDA(cudaMemcpyAsync(d + o_dep, dep.data(), R * 4, cudaMemcpyHostToDevice, st));
            if (mode == YUUKA_ACCEPT_REJECTION) YK_CUDA(cudaMemcpyAsync(d + o_uni, uniforms, R * 8, cudaMemcpyHostToDevice, st));
            RowMeta rows{(const int32_t *)(d + o_tok), (const int32_t *)(d + o_par), (const int32_t *)(d + o_dep),
                         (const uint64_t *)(d + o_anc), nullptr, batch, nodes};
            AcceptOut out{(int32_t *)(d + o_acc), (int32_t *)(d + o_path), (int32_t *)(d + o_em)};
            if (begin) YK_CUDA(cudaEventRecord(begin->e, st));
            if (mode == YUUKA_ACCEPT_GREEDY) {
                ArgmaxScratch sc{(float *)(d + o_val), (int32_t *)(d + o_idx), chunks};
                launch_accept_greedy(st, (const float *)logits->ptr, vocab, rows, sc, out);
            } else {
                launch_accept_rejection(st, (const float *)logits->ptr, (const float *)draft_probs->ptr, (const float *)(d + o_uni),
                                        (unsigned long long *)(d + o_res), vocab, temperature, rows, out);
            }
            if (end) YK_CUDA(cudaEventRecord(end->e, st));
            YK_CUDA(cudaMemcpyAsync(accepted, d + o_acc, (size_t)batch * 4, cudaMemcpyDeviceToHost, st));
            YK_CUDA(cudaMemcpyAsync(emitted, d + o_em, R * 4, cudaMemcpyDeviceToHost, st));
            if (path) YK_CUDA(cudaMemcpyAsync(path, d + o_path, R * 4, cudaMemcpyDeviceToHost, st));
            YK_CUDA(cudaStreamSynchronize(st));
        } catch (...) {
            cudaFree(d);
            throw;
        }
        cudaFree(d);
    });
}
