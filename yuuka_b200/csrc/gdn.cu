// Gated DeltaNet over the rows of a verify step, with rollback by delta log.
//
// The scan never writes the recurrent state. For every row it emits what the
// state update needs -- the normalised key, d = beta * (v - S^T k) and the decay
// exp(alpha) -- and the commit kernel applies exactly the accepted rows'
// rank-one updates to the stored state. Rejected rows therefore cost nothing
// and no per-position copy of the 2 MiB/layer state is made.
//
// Math follows forwardRecurrent (model/qwen35/forward.go:245-287) and
// gdnPerTokenScan (model/qwen35/recurrent.go:56-105). Replaces
// conv1d_chunk / gdn_prepare_splitreg / gdn_chunk_prepared of the reference
// (kernels/hip/prefill/prefill.hip:274-521).
#include <cstdlib>

#include "layers.cuh"
#include "xprep.cuh"

namespace yk {

constexpr int GDN_COLS = 32;   // state columns per CTA
constexpr int GDN_WARPS = 4;   // each owns 8 of the 32 columns
constexpr int GDN_MAX_NODES = 64;

// float exp: the CPU reference evaluates exp in f64 and rounds; the difference is below 2e-7 relative
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_ref(float x) { return x * sigmoid_ref(x); }
__device__ __forceinline__ float softplus_ref(float x) {
    if (x > 20.0f) return x;
    return log1pf(expf(x));
}

// One state update, the same expression in the scan and in the commit so both
// produce identical bits: S <- S * decay + k * d.
__device__ __forceinline__ float state_update(float s, float decay, float k, float d) {
    return fmaf(k, d, s * decay);
}

// Two fp32 lanes per instruction (fma.rn.f32x2 / mul.rn.f32x2): the same IEEE results as the scalar forms, half the
// instructions. The recurrence keeps its state, keys and queries as such pairs.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<const unsigned long long *>(&a)), "l"(*reinterpret_cast<const unsigned long long *>(&b)),
          "l"(*reinterpret_cast<const unsigned long long *>(&c)));
    return *reinterpret_cast<const float2 *>(&d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(d)
        : "l"(*reinterpret_cast<const unsigned long long *>(&a)), "l"(*reinterpret_cast<const unsigned long long *>(&b)));
    return *reinterpret_cast<const float2 *>(&d);
}
// state_update on a pair: S <- S * decay + k * d
__device__ __forceinline__ float2 state_update2(float2 s, float2 decay, float2 k, float2 d) { return fma2(k, d, mul2(s, decay)); }

struct ScanParams {
    GdnArgs a;
    RowMeta rows;
    int chain;  // front end only: the rows are one chain (row i follows row i - 1), however many there are
};

// ---------------------------------------------------------------------------
// Front end, fully parallel over (row, 128-channel unit): depthwise causal conv
// over the row's ancestors and the stored history + SiLU (forward.go:253-268),
// L2 norm of the q and k units (forward.go:275-279, 484-493), beta = sigmoid,
// decay = exp(softplus(alpha + dt) * a) (forward.go:245-248).
// grid (2*groups + rank, nodes, batch), S threads.
__global__ void gdn_front_kernel(const ScanParams p) {
    // (releasing the scan from here, so that it could fetch its state while this kernel runs, measured 7 us
    // slower per layer: a dependent grid that starts early and really has to block in griddepcontrol.wait
    // is woken late; only triggers placed at the end of a kernel have paid)
    pdl_entry();
    const GdnArgs & a = p.a;
    const int S = a.S, N = p.rows.nodes;
    const int u = blockIdx.x, node = blockIdx.y, seq = blockIdx.z;
    const int key_dim = a.groups * S, conv_dim = 2 * key_dim + a.rank * S, K1 = a.kernel - 1;
    const int r = seq * N + node;
    __shared__ int par[GDN_MAX_NODES];
    __shared__ double red[4];
    if (!p.chain) {
        for (int i = threadIdx.x; i < N; i += blockDim.x) par[i] = p.rows.parent[seq * N + i];
        __syncthreads();
    }
    const int e = threadIdx.x;
    const int c = u * S + e;  // q units, then k units, then v units: exactly the conv row order
    float taps[8];
    {
        const float * hist = a.conv_state + ((int64_t)seq_of(p.rows, seq) * conv_dim + c) * K1;
        int cur = node, hidx = K1 - 1;
#pragma unroll
        for (int t = 7; t >= 0; t--) {
            if (t >= a.kernel) { taps[t] = 0.0f; continue; }
            if (cur >= 0) {
                taps[t] = a.proj[(int64_t)(seq * N + cur) * a.ldp + c];
                cur = p.chain ? cur - 1 : par[cur];
            } else {
                taps[t] = hist[hidx--];
            }
        }
    }
    float sum = 0.0f;
    const float * w = a.conv_w + (int64_t)c * a.kernel;
#pragma unroll
    for (int t = 0; t < 8; t++)
        if (t < a.kernel) sum += w[t] * taps[t];
    float v = silu_ref(sum);
    if (u < 2 * a.groups) {
        double sq = (double)v * (double)v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
        __syncthreads();
        double tot = 0;
        for (int i = 0; i < (S >> 5); i++) tot += red[i];
        const float scale = (float)(1.0 / sqrt(tot + (double)a.eps));
        if (u < a.groups) a.qn[(int64_t)r * key_dim + u * S + e] = v * (scale * (float)(1.0 / sqrt((double)S)));
        else a.khat[(int64_t)r * key_dim + (u - a.groups) * S + e] = v * (scale * 1.0f);
    } else {
        const int h = u - 2 * a.groups;
        a.vconv[(int64_t)r * (a.rank * S) + h * S + e] = v;
        if (e == 0) {
            const float * row = a.proj + (int64_t)r * a.ldp;
            a.beta[(int64_t)r * a.rank + h] = sigmoid_ref(row[conv_dim + a.rank * S + h]);
            a.decay[(int64_t)r * a.rank + h] = expf(softplus_ref(row[conv_dim + a.rank * S + a.rank + h] + a.dt[h]) * a.a[h]);
        }
    }
}

// ---------------------------------------------------------------------------
// Recurrence (recurrent.go:56-105) + gated RMSNorm (recurrent.go:39-50).
// grid (S/32 column blocks, rank, batch), the column blocks of a head forming one thread-block
// cluster; 4 warps. A warp owns 8 state columns outright: lane = (row quarter, column), S/4 state
// rows per lane in registers, and the two sums over the state rows close with two shuffles, so the
// rows of a step are walked without a CTA-wide barrier (an earlier form split the state rows over
// the warps and met at two barriers per row: 1 us more per layer). For the gated norm the column
// blocks exchange their sums of squares through distributed shared memory, and each finishes its
// own columns and emits them as f32 and in the prepared form the out-projection GEMM reads.
// Redoing the front end inside this kernel (every CTA its head's q and k group and its own v
// columns) to save the launch in between measured 9 us slower per layer: the front end is only
// cheap when spread over its 576 CTAs.
// Depth-first (pre-order) numbering of the rows of a tree whose parents precede their children; children in
// row order. One thread, at most GDN_MAX_NODES rows.
__device__ __noinline__ void depth_first_order(const int * par, int N, int * order) {
    unsigned long long seen = 0ull;
    int cnt = 0, at = -1;
    while (cnt < N) {
        int next = -1;
        for (int c = at + 1; c < N; c++)
            if (!((seen >> c) & 1ull) && par[c] == at) {
                next = c;
                break;
            }
        if (next >= 0) {
            order[cnt++] = next;
            seen |= 1ull << next;
            at = next;
        } else if (at >= 0) {
            at = par[at];
        } else {
            // (unreachable for a valid parent array: rows without a path to the root go last, in row order)
            for (int c = 0; c < N; c++)
                if (!((seen >> c) & 1ull)) order[cnt++] = c;
        }
    }
}

// TREE: the rows of a sequence may branch (the host staged parent pointers); they are then walked depth first.
template <int S, bool TREE>
__global__ void __launch_bounds__(GDN_WARPS * 32) gdn_scan_kernel(const ScanParams p) {
    pdl_entry();
    constexpr int RPL = S / 4;  // state rows per lane
    const GdnArgs & a = p.a;
    const int cb = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
    const int N = p.rows.nodes;
    const int kh = h % a.groups;
    const int key_dim = a.groups * S, inner = a.rank * S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rq = lane >> 3, cl = warp * 8 + (lane & 7);  // row quarter; column within the block
    const int col = cb * GDN_COLS + cl;

    extern __shared__ __align__(16) float sm[];
    // q and k rows are stored quarter by quarter with four words of padding after each (QP words per quarter): the
    // four row quarters of a warp read their 16-byte pieces from distinct banks (dense rows put all four on the
    // same ones: more bank conflicts than loads in the profile of the batched step)
    constexpr int QP = RPL + 4, SP4 = 4 * QP;
    float * qn = sm;                      // [N][4][QP]
    float * kn = qn + N * SP4;            // [N][4][QP]
    float * vv = kn + N * SP4;            // [N][GDN_COLS]
    float * dd = vv + N * GDN_COLS;       // [N][GDN_COLS]
    float * o_s = dd + N * GDN_COLS;      // [N][GDN_COLS] outputs of this column block
    float * dec = o_s + N * GDN_COLS;     // [N]
    float * bet = dec + N;                // [N]
    int * par = reinterpret_cast<int *>(bet + N);  // [N]
    // TREE: [S / 8][threads] pairs, the state after row 0 (8-byte aligned: the arrays before it hold 2 N (S + 16) + 99 N words)
    float * root_s = reinterpret_cast<float *>(par + N + (N & 1));
    __shared__ double ssq[GDN_MAX_NODES];
    __shared__ float scale_s[GDN_MAX_NODES];
    __shared__ int order_s[TREE ? GDN_MAX_NODES : 1];

    // stored state: the longest fetch (HBM), issued first
    const float * s0 = a.state + ((int64_t)(seq_of(p.rows, seq) * a.rank + h) * S + rq * RPL) * S + col;
    float2 st[RPL / 2];  // state rows (2 i, 2 i + 1) of this lane's quarter, one column
#pragma unroll
    for (int i = 0; i < RPL / 2; i++) st[i] = make_float2(s0[(int64_t)(2 * i) * S], s0[(int64_t)(2 * i + 1) * S]);

    // the front-end kernel has left normalised q and k, the conv output of v, beta and decay in global memory
    // (16-byte loads, eight in flight per thread: with 64 rows of a prompt sub-chunk a scalar loop spent most
    // of the kernel waiting for one L2 round trip after another)
    constexpr int SQ = S / 4;
#pragma unroll 8
    for (int i = threadIdx.x; i < N * SQ; i += blockDim.x) {
        const int node = i / SQ, e4 = i - node * SQ;
        const int64_t at = (int64_t)(seq * N + node) * key_dim + kh * S + e4 * 4;
        const int spot = node * SP4 + (e4 / (RPL / 4)) * QP + (e4 % (RPL / 4)) * 4;
        *reinterpret_cast<float4 *>(qn + spot) = *reinterpret_cast<const float4 *>(a.qn + at);
        *reinterpret_cast<float4 *>(kn + spot) = *reinterpret_cast<const float4 *>(a.khat + at);
    }
#pragma unroll 4
    for (int i = threadIdx.x; i < N * (GDN_COLS / 4); i += blockDim.x) {
        const int node = i / (GDN_COLS / 4), e4 = i - node * (GDN_COLS / 4);
        reinterpret_cast<float4 *>(vv)[i] =
            *reinterpret_cast<const float4 *>(a.vconv + (int64_t)(seq * N + node) * inner + h * S + cb * GDN_COLS + e4 * 4);
    }
    for (int node = threadIdx.x; node < N; node += blockDim.x) {
        par[node] = p.rows.parent[seq * N + node];
        bet[node] = a.beta[(int64_t)(seq * N + node) * a.rank + h];
        dec[node] = a.decay[(int64_t)(seq * N + node) * a.rank + h];
    }
    __syncthreads();

    // the gate values the last phase needs (up to three per thread: a 9-row step needs 2.25) are fetched
    // now, so that the end of the kernel does not wait for them
    constexpr int ZPRE = 3;
    float zpre[ZPRE];
#pragma unroll
    for (int k = 0; k < ZPRE; k++) {
        const int i = threadIdx.x + k * (GDN_WARPS * 32);
        const int node = i / GDN_COLS, c = i - node * GDN_COLS;
        zpre[k] = i < N * GDN_COLS ? a.z[(int64_t)(seq * N + node) * a.ldz + h * S + cb * GDN_COLS + c] : 0.0f;
    }

    // The rows are walked in depth-first order: a row then follows its parent directly unless it is a later
    // sibling, so a branch is replayed from the stored state only when the walk backtracks. In row order
    // (breadth first, as draft trees are numbered) almost every row of a tree switched branches: the 16-node
    // tree of the batched configuration cost 24 replayed updates on top of its 16, depth first it costs 2.
    if constexpr (TREE) {
        if (threadIdx.x == 0) depth_first_order(par, N, order_s);
        __syncthreads();
    }

    // ---- recurrence (recurrent.go:56-105) ----
    int cur = -1;  // node whose state st currently holds (-1: the stored state)
    for (int step = 0; step < N; step++) {
        const int node = TREE ? order_s[step] : step;
        const int pnode = par[node];
        if (pnode != cur) {
            // a sibling branch: rebuild the parent's state by replaying the log of its path, from the state after row 0
            // (every row of a step descends from row 0, the pending token; a tree keeps that state in shared memory)
            // or, failing that, from the stored one
            int path[GDN_MAX_NODES], len = 0;
            if (TREE && pnode >= 0) {
#pragma unroll
                for (int i = 0; i < RPL / 2; i++) st[i] = reinterpret_cast<const float2 *>(root_s)[i * (GDN_WARPS * 32) + threadIdx.x];
                for (int c = pnode; c > 0; c = par[c]) path[len++] = c;
            } else {
#pragma unroll
                for (int i = 0; i < RPL / 2; i++) st[i] = make_float2(s0[(int64_t)(2 * i) * S], s0[(int64_t)(2 * i + 1) * S]);
                for (int c = pnode; c >= 0; c = par[c]) path[len++] = c;
            }
            for (int j = len - 1; j >= 0; j--) {
                const int c = path[j];
                const float dc = dec[c], dv = dd[c * GDN_COLS + cl];
                const float2 dc2 = make_float2(dc, dc), dv2 = make_float2(dv, dv);
#pragma unroll
                for (int i = 0; i < RPL / 2; i++)
                    st[i] = state_update2(st[i], dc2, *reinterpret_cast<const float2 *>(kn + c * SP4 + rq * QP + 2 * i), dv2);
            }
        }
        // this lane's S/4 key and query values, fetched as float4 (a quarter of the shared-memory loads)
        float2 kx[RPL / 2], qx[RPL / 2];
#pragma unroll
        for (int i = 0; i < RPL; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4 *>(kn + node * SP4 + rq * QP + i);
            const float4 q4 = *reinterpret_cast<const float4 *>(qn + node * SP4 + rq * QP + i);
            kx[i / 2] = make_float2(k4.x, k4.y); kx[i / 2 + 1] = make_float2(k4.z, k4.w);
            qx[i / 2] = make_float2(q4.x, q4.y); qx[i / 2 + 1] = make_float2(q4.z, q4.w);
        }
        const float dc = dec[node];
        const float2 dc2 = make_float2(dc, dc);
        // sk = (decay * S)^T k over this lane's rows (four partial sums: rows i mod 4), then over the four row quarters
        float2 sd[RPL / 2], sk01 = make_float2(0.0f, 0.0f), sk23 = sk01;
#pragma unroll
        for (int i = 0; i < RPL / 2; i++) {
            sd[i] = mul2(st[i], dc2);
            if (i & 1) sk23 = fma2(sd[i], kx[i], sk23);
            else sk01 = fma2(sd[i], kx[i], sk01);
        }
        float sk = (sk01.x + sk01.y) + (sk23.x + sk23.y);
        sk += __shfl_xor_sync(0xffffffffu, sk, 8);
        sk += __shfl_xor_sync(0xffffffffu, sk, 16);
        const float d = (vv[node * GDN_COLS + cl] - sk) * bet[node];
        const float2 d2 = make_float2(d, d);
        float2 o01 = make_float2(0.0f, 0.0f), o23 = o01;
#pragma unroll
        for (int i = 0; i < RPL / 2; i++) {
            st[i] = fma2(kx[i], d2, sd[i]);  // state_update with the product S * decay already at hand
            if (i & 1) o23 = fma2(st[i], qx[i], o23);
            else o01 = fma2(st[i], qx[i], o01);
        }
        float o = (o01.x + o01.y) + (o23.x + o23.y);
        o += __shfl_xor_sync(0xffffffffu, o, 8);
        o += __shfl_xor_sync(0xffffffffu, o, 16);
        if (rq == 0) {
            o_s[node * GDN_COLS + cl] = o;
            dd[node * GDN_COLS + cl] = d;
            a.dlog[(int64_t)(seq * N + node) * inner + h * S + col] = d;
        }
        if (TREE && node == 0) {
#pragma unroll
            for (int i = 0; i < RPL / 2; i++) reinterpret_cast<float2 *>(root_s)[i * (GDN_WARPS * 32) + threadIdx.x] = st[i];
        }
        __syncwarp();  // dd of this row is read by the other row quarters when a later branch replays it
        cur = node;
    }

    pdl_trigger_late();
    // ---- gated RMSNorm of the head (recurrent.go:39-50), sums of squares exchanged across the cluster ----
    __syncthreads();
    for (int node = warp; node < N; node += GDN_WARPS) {
        const double v = (double)o_s[node * GDN_COLS + lane];
        double sq = v * v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) ssq[node] = sq;
    }
    cluster_sync_all();
    for (int node = threadIdx.x; node < N; node += blockDim.x) {
        double tot = 0;
        for (unsigned r = 0; r < gridDim.x; r++) tot += ld_cluster_f64(ssq + node, r);  // the cluster spans gridDim.x
        const float mean = (float)(tot / (double)S);
        scale_s[node] = (float)(1.0 / sqrt((double)(mean + a.eps)));
    }
    cluster_sync_all();  // scales visible to the CTA; no CTA leaves while another may still read its sums
#pragma unroll
    for (int k = 0; k < ZPRE; k++) {
        const int i = threadIdx.x + k * (GDN_WARPS * 32);
        if (i < N * GDN_COLS) {
            const int node = i / GDN_COLS, c = i - node * GDN_COLS;
            float t = o_s[i];
            t *= scale_s[node] * a.norm[cb * GDN_COLS + c];
            o_s[i] = t * silu_ref(zpre[k]);
        }
    }
#pragma unroll 8
    for (int i = threadIdx.x + ZPRE * (GDN_WARPS * 32); i < N * GDN_COLS; i += blockDim.x) {
        const int node = i / GDN_COLS, c = i - node * GDN_COLS;
        const int64_t r = seq * N + node;
        const float zv = a.z[r * a.ldz + h * S + cb * GDN_COLS + c];
        float t = o_s[i];
        t *= scale_s[node] * a.norm[cb * GDN_COLS + c];
        o_s[i] = t * silu_ref(zv);
    }
    __syncthreads();
    for (int gi = threadIdx.x; gi < N * (GDN_COLS >> 4); gi += blockDim.x) {
        const int node = gi / (GDN_COLS >> 4), part = gi - node * (GDN_COLS >> 4);
        const int64_t r = seq * N + node;
        const int c0 = h * S + cb * GDN_COLS + part * 16;
        float g16[16];
#pragma unroll
        for (int i = 0; i < 16; i++) g16[i] = o_s[node * GDN_COLS + part * 16 + i];
        float4 * dst = reinterpret_cast<float4 *>(a.out + r * inner + c0);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = make_float4(g16[4 * i], g16[4 * i + 1], g16[4 * i + 2], g16[4 * i + 3]);
        if (a.prep.xh) xprep_store16(a.prep.xh + r * inner + c0, a.prep.xl + r * inner + c0, a.prep.xs16 + r * (inner >> 4) + (c0 >> 4), g16);
    }
}

int launch_gdn_scan(cudaStream_t s, const GdnArgs & a, const RowMeta & rows) {
    YK_REQUIRE(rows.nodes <= GDN_MAX_NODES, YUUKA_ERR_UNSUPPORTED, "gdn: at most %d rows per sequence", GDN_MAX_NODES);
    YK_REQUIRE(a.kernel >= 2 && a.kernel <= 8, YUUKA_ERR_UNSUPPORTED, "gdn: conv kernel %d is outside 2..8", a.kernel);
    YK_REQUIRE(a.S == 64 || a.S == 128, YUUKA_ERR_UNSUPPORTED, "gdn: state size %d is not 64 or 128", a.S);
    ScanParams p{a, rows, 0};
    const int N = rows.nodes;
    dim3 grid(a.S / GDN_COLS, a.rank, rows.batch);
    dim3 fgrid(2 * a.groups + a.rank, N, rows.batch);
    launch_k(gdn_front_kernel, fgrid, a.S, 0, s, p);
    YK_CUDA(cudaGetLastError());
    const size_t smem = sizeof(float) * ((size_t)2 * N * (a.S + 16) + 3 * N * GDN_COLS + 3 * N + (rows.chains ? 0 : (size_t)(a.S / 4) * GDN_WARPS * 32 + 1));
    auto launch = [&](auto kern) {
        YK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_k_cluster(kern, grid, GDN_WARPS * 32, smem, s, grid.x, p);
    };
    if (a.S == 128) {
        if (rows.chains) launch(gdn_scan_kernel<128, false>);
        else launch(gdn_scan_kernel<128, true>);
    } else {
        if (rows.chains) launch(gdn_scan_kernel<64, false>);
        else launch(gdn_scan_kernel<64, true>);
    }
    YK_CUDA(cudaGetLastError());
    return 2;
}

// ---------------------------------------------------------------------------
// Chunkwise (WY-form) scan for chains whose rows are all committed: the sub-chunks of a prompt pass.
// gdnChunkedScan (model/qwen35/recurrent.go:107-351) expresses the rows of a chunk relative to the state S_0 at
// its start; here the same algebra is arranged so that every decay factor is a ratio exp(g_r - g_s) <= 1 (the
// reference scales the values by exp(-g), which overflows for strongly decaying heads over 64 rows). With g the
// cumulative log decay, gam_r = exp(g_r), and d_r = beta_r (v_r - (decayed state)^T k_r) the per-token delta:
//   (I + B) D = diag(beta) (V - diag(gam) K S_0),   B[r][s] = beta_r exp(g_r - g_s) (k_r . k_s)  for s < r
//   o_r = gam_r q_r S_0 + sum_{s <= r} exp(g_r - g_s) (q_r . k_s) d_s
//   S_C = gam_C S_0 + sum_s exp(g_C - g_s) k_s d_s^T
// grid (S/32 column blocks, rank, batch), the column blocks of a head one cluster (gated norm as in the scan
// kernel); a CTA owns 32 columns of the state, of V, D and the outputs, and computes the row-by-row matrices
// (K K^T, Q K^T: they do not depend on the column) itself. The state is rewritten in place: no delta log, no
// separate state commit.
//
// Every product is a tensor-core product, mma.sync m16n8k8 on tf32 operands, with both operands split into two
// tf32 parts (x = hi + lo, three products: lo hi, hi lo, hi hi), which keeps fp32-level accuracy: the two forms
// of the recurrence have to agree to 1e-4 (model/qwen35/recurrent_test.go:60-64). A first form of this kernel
// on fp32 FMAs with 4 x 4 register tiles was bound by shared-memory loads and latency chains (48 k cycles per
// 64-row chunk against 100 k for the row-by-row scan).
constexpr int GC_THREADS = 512;
constexpr int GC_WARPS = GC_THREADS / 32;
constexpr int GC_CP = GDN_COLS + 8;  // pitch of the [row][32 columns] arrays and of the state block: the four k rows
                                     // a B fragment reads fall on distinct banks (8 t + g)

// x = hi + lo with hi the leading 10 mantissa bits (the tensor core ignores the low 13 bits of a tf32 operand, so
// lo, exact in fp32, is used as it is: its own truncation is 2^-20 of x). Masking instead of cvt.rna.tf32: the
// conversion instruction issues at a fraction of the ALU rate and was the whole cost of this kernel's products.
__device__ __forceinline__ void tf32_split(float x, uint32_t & hi, uint32_t & lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// acc[j] += A (16 x 8 ksteps) * B (8 ksteps x 8, NT tiles side by side). fa(row, k) and fb(k, col) read one
// element of the operands; lane (g, t) of the warp holds rows g, g + 8 and k columns t, t + 4 of A, k rows t, t + 4
// and column g of B, and elements (g, 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1) of each 16 x 8 result.
template <int NT, class FA, class FB>
__device__ __forceinline__ void warp_mma_3x(float (&acc)[NT][4], int ksteps, FA fa, FB fb, int g, int t) {
    for (int ks = 0; ks < ksteps; ks++) {
        const int k0 = ks * 8;
        uint32_t ah[4], al[4];
        tf32_split(fa(g, k0 + t), ah[0], al[0]);
        tf32_split(fa(g + 8, k0 + t), ah[1], al[1]);
        tf32_split(fa(g, k0 + t + 4), ah[2], al[2]);
        tf32_split(fa(g + 8, k0 + t + 4), ah[3], al[3]);
#pragma unroll
        for (int j = 0; j < NT; j++) {
            uint32_t bh[2], bl[2];
            tf32_split(fb(k0 + t, 8 * j + g), bh[0], bl[0]);
            tf32_split(fb(k0 + t + 4, 8 * j + g), bh[1], bl[1]);
            mma_tf32(acc[j], al, bh);
            mma_tf32(acc[j], ah, bl);
            mma_tf32(acc[j], ah, bh);
        }
    }
}

template <int S>
__global__ void __launch_bounds__(GC_THREADS, 1) gdn_chunk_kernel(const ScanParams p) {
    pdl_entry();
    const GdnArgs & a = p.a;
    const int cb = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
    const int N = p.rows.nodes;
    const int kh = h % a.groups;
    const int key_dim = a.groups * S, inner = a.rank * S;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int KP = S + 4;            // pitch of a q / k row: the eight rows an A fragment reads fall on banks 4 g + t
    constexpr int CP = GC_CP;
    const int MT = (N + 15) >> 4;        // 16-row tiles
    const int NR = MT * 16;              // rows with padding (zero rows)
    const int NP = NR + 4;               // pitch of the row-by-row matrices (banks 4 g + t again)

    extern __shared__ __align__(16) float sm[];
    float * qn = sm;                     // [NR][KP]
    float * kn = qn + NR * KP;           // [NR][KP]
    float * s0 = kn + NR * KP;           // [S][CP]  this CTA's columns of the stored state
    float * vv = s0 + S * CP;            // [NR][CP] v, later exp(g_C - g_s) d_s
    float * ks = vv + NR * CP;           // [NR][CP] K S_0, then the right-hand side
    float * dd = ks + NR * CP;           // [NR][CP] D
    float * o_s = dd + NR * CP;          // [NR][CP] Q S_0, then the outputs
    float * Bm = o_s + NR * CP;          // [NR][NP] beta_r w_rs (k_r . k_s), s < r
    float * Am = Bm + NR * NP;           // [NR][NP] w_rs (q_r . k_s), s <= r
    float * Tm = Am + NR * NP;           // [NR][20] inverses of the 16 x 16 diagonal blocks of I + B
    float * lg = Tm + NR * 20;           // [NR] cumulative log decay
    float * bet = lg + NR;               // [NR]
    __shared__ double ssq[GDN_MAX_NODES];
    __shared__ float scale_s[GDN_MAX_NODES];

    // ---- loads, asynchronous: q and k (needed first), then this CTA's block of the state and v; beta, decay ----
    constexpr int SQ = S / 4;
    for (int i = tid; i < NR * SQ; i += GC_THREADS) {
        const int node = i / SQ, e4 = i - node * SQ;
        if (node < N) {
            const int64_t at = (int64_t)(seq * N + node) * key_dim + kh * S + e4 * 4;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(qn + node * KP + e4 * 4)),
                         "l"(a.qn + at) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(kn + node * KP + e4 * 4)),
                         "l"(a.khat + at) : "memory");
        } else {
            *reinterpret_cast<float4 *>(qn + node * KP + e4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(kn + node * KP + e4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    float * state = const_cast<float *>(a.state) + ((int64_t)(seq_of(p.rows, seq) * a.rank + h) * S) * S + cb * GDN_COLS;
    for (int i = tid; i < S * (GDN_COLS / 4); i += GC_THREADS) {
        const int row = i / (GDN_COLS / 4), c4 = i - row * (GDN_COLS / 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(s0 + row * CP + c4 * 4)),
                     "l"(state + (int64_t)row * S + c4 * 4) : "memory");
    }
    for (int i = tid; i < NR * (GDN_COLS / 4); i += GC_THREADS) {
        const int node = i / (GDN_COLS / 4), e4 = i - node * (GDN_COLS / 4);
        if (node < N)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(vv + node * CP + e4 * 4)),
                         "l"(a.vconv + (int64_t)(seq * N + node) * inner + h * S + cb * GDN_COLS + e4 * 4) : "memory");
        else *reinterpret_cast<float4 *>(vv + node * CP + e4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the gate values and the norm weight the last phase needs (a 64-row chunk: four per thread) are fetched now
    constexpr int ZPRE = GDN_MAX_NODES * GDN_COLS / GC_THREADS;
    float zpre[ZPRE];
#pragma unroll
    for (int k = 0; k < ZPRE; k++) {
        const int i = tid + k * GC_THREADS;
        const int node = i / GDN_COLS, c = i - node * GDN_COLS;
        zpre[k] = i < N * GDN_COLS ? a.z[(int64_t)(seq * N + node) * a.ldz + h * S + cb * GDN_COLS + c] : 0.0f;
    }
    const float norm_w = a.norm[cb * GDN_COLS + (tid & (GDN_COLS - 1))];
    for (int node = tid; node < NR; node += GC_THREADS) {
        float b = 0.0f, l = 0.0f;
        if (node < N) {
            b = a.beta[(int64_t)(seq * N + node) * a.rank + h];
            const float dc = a.decay[(int64_t)(seq * N + node) * a.rank + h];
            l = dc > 0.0f ? fmaxf(logf(dc), -100.0f) : -100.0f;  // a decay that underflowed still wipes the state
        }
        bet[node] = b;
        o_s[node] = l;  // (scratch until the outputs are written)
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // q and k have landed; the state may still be on its way
    __syncthreads();
    if (warp == 0) {
        // inclusive scan of the (at most 64) log decays: two per lane
        const float l0 = lane < NR ? o_s[lane] : 0.0f, l1 = lane + 32 < NR ? o_s[lane + 32] : 0.0f;
        float s0v = l0, s1v = l1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float u0 = __shfl_up_sync(0xffffffffu, s0v, o), u1 = __shfl_up_sync(0xffffffffu, s1v, o);
            if (lane >= o) { s0v += u0; s1v += u1; }
        }
        const float first = __shfl_sync(0xffffffffu, s0v, 31);
        if (lane < NR) lg[lane] = s0v;
        if (lane + 32 < NR) lg[lane + 32] = first + s1v;
    }
    __syncthreads();

    // ---- B and A: K K^T and Q K^T on the lower triangle (16 x 16 tiles up to the diagonal one), decay ratios and
    // beta folded in on the way out; entries above the diagonal inside the diagonal tiles are zero ----
    {
        const int per_mat = MT * (MT + 1) / 2;
        for (int tile = warp; tile < 2 * per_mat; tile += GC_WARPS) {
            const int mat = tile >= per_mat, rest = tile - mat * per_mat;
            int mt = 0;
            while ((mt + 1) * (mt + 2) / 2 <= rest) mt++;
            const int nt = rest - mt * (mt + 1) / 2;
            const float * arow = (mat ? qn : kn) + (16 * mt) * KP, * brow = kn + (16 * nt) * KP;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            warp_mma_3x<2>(acc, S / 8, [&](int r, int k) { return arow[r * KP + k]; }, [&](int k, int c) { return brow[c * KP + k]; }, g, t);
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int r = 16 * mt + g + (e >> 1) * 8, c = 16 * nt + 8 * j + 2 * t + (e & 1);
                    const float wgt = c <= r ? expf(lg[r] - lg[c]) : 0.0f;
                    if (mat) Am[r * NP + c] = wgt * acc[j][e];
                    else Bm[r * NP + c] = c < r ? bet[r] * wgt * acc[j][e] : 0.0f;
                }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();

    // ---- K S_0 and Q S_0 for this CTA's columns: a warp per (matrix, 16-row tile, 16-column half) ----
    for (int task = warp; task < 4 * MT; task += GC_WARPS) {
        const int nh = task & 1, mt = (task >> 1) % MT, which = task / (2 * MT);
        const float * arow = (which ? qn : kn) + (16 * mt) * KP, * bcol = s0 + 16 * nh;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        warp_mma_3x<2>(acc, S / 8, [&](int r, int k) { return arow[r * KP + k]; }, [&](int k, int c) { return bcol[k * CP + c]; }, g, t);
        float * dst = (which ? o_s : ks) + (16 * mt) * CP + 16 * nh;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            *reinterpret_cast<float2 *>(dst + g * CP + 8 * j + 2 * t) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2 *>(dst + (g + 8) * CP + 8 * j + 2 * t) = make_float2(acc[j][2], acc[j][3]);
        }
    }
    __syncthreads();

    // ---- right-hand side beta (v - gam K S_0); meanwhile two warps invert the 16 x 16 diagonal blocks of I + B ----
    for (int i = tid; i < NR * GDN_COLS; i += GC_THREADS) {
        const int r = i / GDN_COLS, c = i - r * GDN_COLS;
        ks[r * CP + c] = bet[r] * (vv[r * CP + c] - expf(lg[r]) * ks[r * CP + c]);
    }
    if (warp >= GC_WARPS - 2) {
        // half a warp per block, lane = column s of the inverse T: row r of T is e_r minus the rows before it
        // weighted by row r of B (forward substitution, as inverseLower of recurrent.go:307-331 does for the
        // whole chunk). Rows beyond the chunk have B = 0 and stay rows of the identity.
        const int blk = (warp - (GC_WARPS - 2)) * 2 + (lane >> 4), sc = lane & 15, b0 = blk * 16;
        if (b0 < N) {
            float tv[16];
#pragma unroll
            for (int r = 0; r < 16; r++) {
                float v = r == sc ? 1.0f : 0.0f;
                const float * brow = Bm + (b0 + r) * NP + b0;
#pragma unroll
                for (int u = 0; u < r; u++) v = fmaf(-brow[u], tv[u], v);
                tv[r] = v;
                Tm[(b0 + r) * 20 + sc] = v;
            }
        }
    }
    __syncthreads();
    // ---- forward substitution over the blocks: D_b = T_b (rhs_b - B[b][earlier] D[earlier]); a warp per 8 columns ----
    for (int b0 = 0; b0 < N; b0 += 16) {
        if (b0 > 0) {
            if (warp < 4) {
                float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
                const float * arow = Bm + b0 * NP, * bcol = dd + 8 * warp;
                warp_mma_3x<1>(acc, b0 / 8, [&](int r, int k) { return arow[r * NP + k]; }, [&](int k, int c) { return bcol[k * CP + c]; }, g, t);
                float * dst = ks + b0 * CP + 8 * warp + 2 * t;
                dst[g * CP] -= acc[0][0];
                dst[g * CP + 1] -= acc[0][1];
                dst[(g + 8) * CP] -= acc[0][2];
                dst[(g + 8) * CP + 1] -= acc[0][3];
            }
            __syncthreads();
        }
        if (warp < 4) {
            float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
            const float * arow = Tm + b0 * 20, * bcol = ks + b0 * CP + 8 * warp;
            warp_mma_3x<1>(acc, 2, [&](int r, int k) { return arow[r * 20 + k]; }, [&](int k, int c) { return bcol[k * CP + c]; }, g, t);
            float * dst = dd + b0 * CP + 8 * warp + 2 * t;
            *reinterpret_cast<float2 *>(dst + g * CP) = make_float2(acc[0][0], acc[0][1]);
            *reinterpret_cast<float2 *>(dst + (g + 8) * CP) = make_float2(acc[0][2], acc[0][3]);
        }
        __syncthreads();
    }
    // vv <- exp(g_C - g_s) d_s for the state update
    {
        const float lc = lg[N - 1];
        for (int i = tid; i < NR * GDN_COLS; i += GC_THREADS) {
            const int r = i / GDN_COLS, c = i - r * GDN_COLS;
            vv[r * CP + c] = r < N ? expf(lc - lg[r]) * dd[r * CP + c] : 0.0f;
        }
    }
    __syncthreads();

    // ---- outputs gam_r (Q S_0)_r + sum_{s <= r} A[r][s] d_s (2 MT tasks) and the new state gam_C S_0 + K^T (w d),
    // written in place (S / 8 tasks): a warp per 16 rows x 16 columns ----
    {
        const float gam_c = expf(lg[N - 1]);
        for (int task = warp; task < 2 * MT + S / 8; task += GC_WARPS) {
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            if (task < 2 * MT) {
                const int nh = task & 1, mt = task >> 1;
                const float * arow = Am + (16 * mt) * NP, * bcol = dd + 16 * nh;
                warp_mma_3x<2>(acc, 2 * mt + 2, [&](int r, int k) { return arow[r * NP + k]; }, [&](int k, int c) { return bcol[k * CP + c]; }, g, t);
                float * dst = o_s + (16 * mt) * CP + 16 * nh;
                const float g0 = expf(lg[16 * mt + g]), g1 = expf(lg[16 * mt + g + 8]);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    float2 * lo = reinterpret_cast<float2 *>(dst + g * CP + 8 * j + 2 * t), * hi = reinterpret_cast<float2 *>(dst + (g + 8) * CP + 8 * j + 2 * t);
                    *lo = make_float2(fmaf(g0, lo->x, acc[j][0]), fmaf(g0, lo->y, acc[j][1]));
                    *hi = make_float2(fmaf(g1, hi->x, acc[j][2]), fmaf(g1, hi->y, acc[j][3]));
                }
            } else {
                const int e = task - 2 * MT, nh = e & 1, it = e >> 1;  // state rows 16 it .., columns 16 nh ..
                const float * acol = kn + 16 * it, * bcol = vv + 16 * nh;
                warp_mma_3x<2>(acc, NR / 8, [&](int r, int k) { return acol[k * KP + r]; }, [&](int k, int c) { return bcol[k * CP + c]; }, g, t);
                const float * old = s0 + (16 * it) * CP + 16 * nh;
                float * dst = state + (int64_t)(16 * it) * S + 16 * nh;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const float2 o0 = *reinterpret_cast<const float2 *>(old + g * CP + 8 * j + 2 * t);
                    const float2 o1 = *reinterpret_cast<const float2 *>(old + (g + 8) * CP + 8 * j + 2 * t);
                    *reinterpret_cast<float2 *>(dst + (int64_t)g * S + 8 * j + 2 * t) = make_float2(fmaf(gam_c, o0.x, acc[j][0]), fmaf(gam_c, o0.y, acc[j][1]));
                    *reinterpret_cast<float2 *>(dst + (int64_t)(g + 8) * S + 8 * j + 2 * t) = make_float2(fmaf(gam_c, o1.x, acc[j][2]), fmaf(gam_c, o1.y, acc[j][3]));
                }
            }
        }
    }
    __syncthreads();

    pdl_trigger_late();
    // ---- gated RMSNorm of the head (recurrent.go:39-50), sums of squares exchanged across the cluster ----
    for (int node = warp; node < N; node += GC_WARPS) {
        const double v = (double)o_s[node * CP + lane];
        double sq = v * v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) ssq[node] = sq;
    }
    cluster_sync_all();
    for (int node = tid; node < N; node += GC_THREADS) {
        double tot = 0;
        for (unsigned r = 0; r < gridDim.x; r++) tot += ld_cluster_f64(ssq + node, r);  // the cluster spans gridDim.x
        const float mean = (float)(tot / (double)S);
        scale_s[node] = (float)(1.0 / sqrt((double)(mean + a.eps)));
    }
    cluster_sync_all();  // scales visible to the CTA; no CTA leaves while another may still read its sums
#pragma unroll
    for (int k = 0; k < ZPRE; k++) {
        const int i = tid + k * GC_THREADS;
        if (i < N * GDN_COLS) {
            const int node = i / GDN_COLS, c = i - node * GDN_COLS;
            o_s[node * CP + c] = o_s[node * CP + c] * (scale_s[node] * norm_w) * silu_ref(zpre[k]);
        }
    }
    __syncthreads();
    for (int gi = tid; gi < N * (GDN_COLS >> 4); gi += GC_THREADS) {
        const int node = gi / (GDN_COLS >> 4), part = gi - node * (GDN_COLS >> 4);
        const int64_t r = seq * N + node;
        const int c0 = h * S + cb * GDN_COLS + part * 16;
        float g16[16];
#pragma unroll
        for (int i = 0; i < 16; i++) g16[i] = o_s[node * CP + part * 16 + i];
        float4 * dst = reinterpret_cast<float4 *>(a.out + r * inner + c0);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = make_float4(g16[4 * i], g16[4 * i + 1], g16[4 * i + 2], g16[4 * i + 3]);
        if (a.prep.xh) xprep_store16(a.prep.xh + r * inner + c0, a.prep.xl + r * inner + c0, a.prep.xs16 + r * (inner >> 4) + (c0 >> 4), g16);
    }
}

static size_t gdn_chunk_smem(int N, int S) {
    const size_t nr = (size_t)((N + 15) & ~15);
    return sizeof(float) * (2 * nr * (S + 4) + (size_t)S * GC_CP + 4 * nr * GC_CP + 2 * nr * (nr + 4) + nr * 20 + 2 * nr);
}

// The front end alone for one chain of any length (a whole prompt pass of one sequence): conv taps come from the
// preceding rows of the pass and, for its first kernel - 1 rows, from the stored history.
void launch_gdn_front_chain(cudaStream_t s, const GdnArgs & a, int seq_slot, int n_rows) {
    YK_REQUIRE(a.kernel >= 2 && a.kernel <= 8, YUUKA_ERR_UNSUPPORTED, "gdn: conv kernel %d is outside 2..8", a.kernel);
    YK_REQUIRE(a.S == 64 || a.S == 128, YUUKA_ERR_UNSUPPORTED, "gdn: state size %d is not 64 or 128", a.S);
    (void)seq_slot;
    RowMeta rows{};
    rows.batch = 1;
    rows.nodes = n_rows;
    ScanParams p{a, rows, 1};
    dim3 fgrid(2 * a.groups + a.rank, n_rows, 1);
    launch_k(gdn_front_kernel, fgrid, a.S, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

// Chunkwise scan of a chain of at most 64 rows that are all committed, after the front end has run for them; the
// state is rewritten in place (the conv history still moves with launch_gdn_commit(..., conv_only)).
void launch_gdn_chunk(cudaStream_t s, const GdnArgs & a, const RowMeta & rows) {
    YK_REQUIRE(rows.nodes <= GDN_MAX_NODES, YUUKA_ERR_UNSUPPORTED, "gdn: at most %d rows per chunk", GDN_MAX_NODES);
    YK_REQUIRE(a.S == 64 || a.S == 128, YUUKA_ERR_UNSUPPORTED, "gdn: state size %d is not 64 or 128", a.S);
    ScanParams p{a, rows, 0};
    const int N = rows.nodes;
    dim3 grid(a.S / GDN_COLS, a.rank, rows.batch);
    const size_t smem = gdn_chunk_smem(N, a.S);
    if (a.S == 128) {
        YK_CUDA(cudaFuncSetAttribute(gdn_chunk_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_k_cluster(gdn_chunk_kernel<128>, grid, GC_THREADS, smem, s, grid.x, p);
    } else {
        YK_CUDA(cudaFuncSetAttribute(gdn_chunk_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_k_cluster(gdn_chunk_kernel<64>, grid, GC_THREADS, smem, s, grid.x, p);
    }
    YK_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// commit

struct CommitParams {
    const GdnLayerCommit * layers;
    int groups, rank, S, kernel, conv_dim;
    int seq_base;  // first sequence of the step within the session's state arrays
    int row_base;  // first row of the step within the layer's per-row logs (sub-chunks of a wide prompt pass)
    int conv_only; // the grid holds only the conv-history blocks (the chunkwise scan has written the state itself)
    RowMeta rows;
    AcceptOut acc;
};

// grid (4 * rank + 8, batch, layers): blocks 0..4*rank-1 update a quarter of one head's state (S/4 rows),
// the last eight rewrite the conv history, an eighth of the channels each.
constexpr int COMMIT_PARTS = 4;
constexpr int COMMIT_CONV_PARTS = 8;
__global__ void __launch_bounds__(256, 4) gdn_commit_kernel(const CommitParams p) {
    pdl_entry();
    const GdnLayerCommit L = p.layers[blockIdx.z];
    const int seq = blockIdx.y, N = p.rows.nodes, S = p.S;
    const int a = p.acc.accepted[seq];
    const int32_t * path = p.acc.path + (int64_t)seq * N;
    auto node_at = [&](int t) { return t == 0 ? 0 : path[t - 1]; };  // t = 0..a
    if (!p.conv_only && (int)blockIdx.x < COMMIT_PARTS * p.rank) {
        // S/4 rows of one head's S x S state, read and written once as float4 however many rows were accepted.
        // A thread owns four columns j and up to four rows i and keeps them in registers. The accepted rows'
        // keys (this part's S/4 of them), d values and decays are brought into shared memory in one round of
        // loads, all rows at once (up to 64 in a prompt sub-chunk: fetching them nine at a time between
        // barriers made that commit a chain of L2 round trips, 57 us per layer).
        constexpr int MAXR = 4;
        const int h = blockIdx.x / COMMIT_PARTS, part = blockIdx.x % COMMIT_PARTS, kh = h % p.groups;
        const int rows_part = S / COMMIT_PARTS, i_base = part * rows_part;
        float * st = L.state + (int64_t)((p.seq_base + seq_of(p.rows, seq)) * p.rank + h) * S * S;
        __shared__ float kh_s[GDN_MAX_NODES][32];
        __shared__ __align__(16) float d_s[GDN_MAX_NODES][128];
        __shared__ float dec_s[GDN_MAX_NODES];
        __shared__ int row_s[GDN_MAX_NODES];
        const int quads = S >> 2;
        const int j4 = threadIdx.x % quads, i0 = threadIdx.x / quads, istep = blockDim.x / quads;
        float4 v[MAXR];
#pragma unroll
        for (int q = 0; q < MAXR; q++) {
            const int i = i0 + q * istep;
            v[q] = i < rows_part ? *reinterpret_cast<const float4 *>(st + (int64_t)(i_base + i) * S + j4 * 4)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const int nt = a + 1;  // <= N <= GDN_MAX_NODES
        for (int t = threadIdx.x; t < nt; t += blockDim.x) {
            const int r = p.row_base + seq * N + node_at(t);
            row_s[t] = r;
            dec_s[t] = L.decay[(int64_t)r * p.rank + h];
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * rows_part; idx += blockDim.x) {
            const int t = idx / rows_part, i = idx - t * rows_part;
            kh_s[t][i] = L.khat[(int64_t)row_s[t] * (p.groups * S) + kh * S + i_base + i];
        }
        for (int idx = threadIdx.x; idx < nt * quads; idx += blockDim.x) {
            const int t = idx / quads, c4 = idx - t * quads;
            reinterpret_cast<float4 *>(d_s[t])[c4] =
                *reinterpret_cast<const float4 *>(L.dlog + (int64_t)row_s[t] * (p.rank * S) + h * S + c4 * 4);
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float dc = dec_s[t];
            const float4 d = reinterpret_cast<const float4 *>(d_s[t])[j4];
#pragma unroll
            for (int q = 0; q < MAXR; q++) {
                const int i = i0 + q * istep;
                const float k = kh_s[t][i < rows_part ? i : 0];
                v[q].x = state_update(v[q].x, dc, k, d.x);
                v[q].y = state_update(v[q].y, dc, k, d.y);
                v[q].z = state_update(v[q].z, dc, k, d.z);
                v[q].w = state_update(v[q].w, dc, k, d.w);
            }
        }
#pragma unroll
        for (int q = 0; q < MAXR; q++) {
            const int i = i0 + q * istep;
            if (i < rows_part) *reinterpret_cast<float4 *>(st + (int64_t)(i_base + i) * S + j4 * 4) = v[q];
        }
    } else {
        // history after the step = last kernel-1 raw inputs of [old history, accepted rows]: entry t takes the
        // combined index n_new - K1 + t, where the old history occupies [-K1, -1] and the accepted rows
        // [0, n_new - 1]. The (at most kernel-1) source rows are looked up once per CTA; the channels are
        // spread over COMMIT_CONV_PARTS CTAs (one CTA walking all channels with a path look-up per entry was
        // a 45 us chain of dependent loads: most of this kernel's time).
        const int K1 = p.kernel - 1, n_new = a + 1;
        __shared__ int src_row[8];
        if (threadIdx.x < K1) {
            const int src = n_new + (int)threadIdx.x - K1;
            src_row[threadIdx.x] = src >= 0 ? p.row_base + seq * N + node_at(src) : -1;
        }
        __syncthreads();
        const int part = p.conv_only ? (int)blockIdx.x : (int)blockIdx.x - COMMIT_PARTS * p.rank;
        const int per = (p.conv_dim + COMMIT_CONV_PARTS - 1) / COMMIT_CONV_PARTS;
        const int c_end = min(p.conv_dim, (part + 1) * per);
        for (int c = part * per + threadIdx.x; c < c_end; c += blockDim.x) {
            float * hist = L.conv_state + ((int64_t)(p.seq_base + seq_of(p.rows, seq)) * p.conv_dim + c) * K1;
            float nv[8];
#pragma unroll
            for (int t = 0; t < 8; t++) {
                if (t >= K1) continue;
                const int src = n_new + t - K1;
                nv[t] = src >= 0 ? L.proj[(int64_t)src_row[t] * L.ldp + c] : hist[K1 + src];
            }
#pragma unroll
            for (int t = 0; t < 8; t++)
                if (t < K1) hist[t] = nv[t];
        }
    }
}

void launch_gdn_commit(cudaStream_t s, const GdnLayerCommit * layers_dev, int n_layers, int groups, int rank, int S,
                       int kernel, int conv_dim, int seq_base, const RowMeta & rows, const AcceptOut & acc, int row_base,
                       bool conv_only) {
    if (n_layers == 0) return;
    CommitParams p{layers_dev, groups, rank, S, kernel, conv_dim, seq_base, row_base, conv_only ? 1 : 0, rows, acc};
    dim3 grid(conv_only ? COMMIT_CONV_PARTS : COMMIT_PARTS * rank + COMMIT_CONV_PARTS, rows.batch, n_layers);
    launch_k(gdn_commit_kernel, grid, 256, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// KV commit: accepted row t (t >= 1) of a tree moves from slot pos0 + node to
// its final position pos0 + t. A chain is already in place.

struct KvCommitParams {
    const KvLayerCommit * layers;
    KvPool geom;
    RowMeta rows;
    AcceptOut acc;
};

__global__ void kv_commit_kernel(const KvCommitParams p) {
    pdl_entry();
    const KvLayerCommit L = p.layers[blockIdx.y];
    const int seq = blockIdx.x, N = p.rows.nodes;
    const int a = p.acc.accepted[seq];
    const int sq = seq_of(p.rows, seq);
    const int pos0 = p.rows.pos0[sq];
    const int32_t * path = p.acc.path + (int64_t)seq * N;
    const int words = p.geom.row_bytes / 2;
    for (int t = 1; t <= a; t++) {
        const int node = path[t - 1];
        if (node != t) {
            auto off = [&](int slot) {
                int block = p.geom.tables[(int64_t)sq * p.geom.table_stride + slot / p.geom.block_size];
                return ((int64_t)block * p.geom.block_size + slot % p.geom.block_size) * p.geom.row_bytes;
            };
            const int64_t src = off(pos0 + node), dst = off(pos0 + t);
            const uint16_t * ks = reinterpret_cast<const uint16_t *>(L.k + src);
            const uint16_t * vs = reinterpret_cast<const uint16_t *>(L.v + src);
            uint16_t * kd = reinterpret_cast<uint16_t *>(L.k + dst);
            uint16_t * vd = reinterpret_cast<uint16_t *>(L.v + dst);
            for (int i = threadIdx.x; i < words; i += blockDim.x) {
                kd[i] = ks[i];
                vd[i] = vs[i];
            }
        }
        __syncthreads();
    }
}

void launch_kv_commit(cudaStream_t s, const KvLayerCommit * layers_dev, int n_layers, const KvPool & geom,
                      const RowMeta & rows, const AcceptOut & acc) {
    if (n_layers == 0) return;
    KvCommitParams p{layers_dev, geom, rows, acc};
    dim3 grid(rows.batch, n_layers);
    launch_k(kv_commit_kernel, grid, 256, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

__global__ void advance_positions_kernel(int32_t * pos0, const int32_t * accepted, int batch, const int32_t * seq_map) {
    pdl_entry();
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) pos0[seq_map ? seq_map[b] : b] += accepted[b] + 1;
}

void launch_advance_positions(cudaStream_t s, int32_t * pos0, const AcceptOut & acc, int batch, const int32_t * seq_map) {
    launch_k(advance_positions_kernel, (batch + 127) / 128, 128, 0, s, pos0, acc.accepted, batch, seq_map);
    YK_CUDA(cudaGetLastError());
}

}  // namespace yk
