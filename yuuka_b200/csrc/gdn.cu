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
#include "layers.cuh"

namespace yk {

constexpr int GDN_COLS = 32;   // state columns per CTA (one per lane)
constexpr int GDN_WARPS = 4;   // state rows are split over the warps
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

struct ScanParams {
    GdnArgs a;
    RowMeta rows;
};

// Depthwise causal conv + SiLU for local channel lc of row node, from the staged
// raw inputs: taps run over the row's ancestors, then into the stored conv
// history (forward.go:253-268). raw is [N + kernel-1][NCH]: rows 0..kernel-2
// hold the history (oldest first), row kernel-1+i holds node i.
template <int NCH>
__device__ __forceinline__ float conv_channel(const float * raw, const float * w, const int * par, int kernel, int node,
                                              int lc) {
    float taps[8];
    int cur = node, hidx = kernel - 2;
    for (int t = kernel - 1; t >= 0; t--) {
        if (cur >= 0) {
            taps[t] = raw[(kernel - 1 + cur) * NCH + lc];
            cur = par[cur];
        } else {
            taps[t] = raw[hidx-- * NCH + lc];
        }
    }
    float sum = 0.0f;
    for (int i = 0; i < kernel - 1; i++) sum += w[lc * kernel + i] * taps[i];
    sum += w[lc * kernel + kernel - 1] * taps[kernel - 1];
    return silu_ref(sum);
}

template <int S>
__global__ void __launch_bounds__(GDN_WARPS * 32) gdn_scan_kernel(const ScanParams p) {
    constexpr int RPW = S / GDN_WARPS;        // state rows per warp
    constexpr int NCH = 2 * S + GDN_COLS;     // channels this CTA needs: q[S] | k[S] | v[GDN_COLS]
    const GdnArgs & a = p.a;
    const int cb = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
    const int N = p.rows.nodes;
    const int kh = h % a.groups;
    const int key_dim = a.groups * S;
    const int conv_dim = 2 * key_dim + a.rank * S;
    const int K1 = a.kernel - 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = cb * GDN_COLS + lane;

    extern __shared__ __align__(16) float sm[];
    float * qn = sm;                      // [N][S]
    float * kn = qn + N * S;              // [N][S]
    float * vv = kn + N * S;              // [N][GDN_COLS]
    float * dd = vv + N * GDN_COLS;       // [N][GDN_COLS]
    float * dec = dd + N * GDN_COLS;      // [N]
    float * bet = dec + N;                // [N]
    float * red = bet + N;                // [GDN_WARPS][GDN_COLS]
    float * red2 = red + GDN_WARPS * GDN_COLS;
    float * raw = red2 + GDN_WARPS * GDN_COLS;   // [K1 + N][NCH] raw inputs of this CTA's channels
    float * wts = raw + (K1 + N) * NCH;           // [NCH][kernel]
    int * par = reinterpret_cast<int *>(wts + NCH * a.kernel);  // [N]
    __shared__ float nrm[2 * GDN_MAX_NODES];  // 1 / sqrt(sum of squares + eps) of q then k rows

    // The recurrent state does not depend on this step's projections: start its loads first.
    const float * s0 = a.state + ((int64_t)(seq * a.rank + h) * S + warp * RPW) * S + col;
    float st[RPW];
#pragma unroll
    for (int i = 0; i < RPW; i++) st[i] = s0[(int64_t)i * S];

    // ---- stage raw inputs, history, taps and parents with coalesced loads ----
    auto channel = [&](int lc) {  // local channel -> channel of the conv row
        return lc < S ? kh * S + lc : (lc < 2 * S ? key_dim + kh * S + (lc - S) : 2 * key_dim + h * S + cb * GDN_COLS + (lc - 2 * S));
    };
    for (int i = threadIdx.x; i < N * NCH; i += blockDim.x) {
        const int node = i / NCH, lc = i - node * NCH;
        raw[(K1 + node) * NCH + lc] = a.proj[(int64_t)(seq * N + node) * a.ldp + channel(lc)];
    }
    for (int i = threadIdx.x; i < NCH * K1; i += blockDim.x) {
        const int lc = i / K1, t = i - lc * K1;
        raw[t * NCH + lc] = a.conv_state[((int64_t)seq * conv_dim + channel(lc)) * K1 + t];
    }
    for (int i = threadIdx.x; i < NCH * a.kernel; i += blockDim.x) {
        const int lc = i / a.kernel, t = i - lc * a.kernel;
        wts[i] = a.conv_w[(int64_t)channel(lc) * a.kernel + t];
    }
    for (int node = threadIdx.x; node < N; node += blockDim.x) {
        par[node] = p.rows.parent[seq * N + node];
        const float * row = a.proj + (int64_t)(seq * N + node) * a.ldp;
        const float b = row[conv_dim + a.rank * S + h];
        const float al = row[conv_dim + a.rank * S + a.rank + h];
        bet[node] = sigmoid_ref(b);
        dec[node] = expf(softplus_ref(al + a.dt[h]) * a.a[h]);
    }
    __syncthreads();
    // ---- front end: conv + SiLU ----
    for (int i = threadIdx.x; i < N * NCH; i += blockDim.x) {
        const int node = i / NCH, lc = i - node * NCH;
        const float v = conv_channel<NCH>(raw, wts, par, a.kernel, node, lc);
        if (lc < S) qn[node * S + lc] = v;
        else if (lc < 2 * S) kn[node * S + lc - S] = v;
        else vv[node * GDN_COLS + lc - 2 * S] = v;
    }
    __syncthreads();
    // l2NormHead (forward.go:484-493): f64 sum, scale = f32(1/sqrt(sum + eps)) * extra
    for (int v = warp; v < 2 * N; v += GDN_WARPS) {
        const float * x = (v < N ? qn : kn) + (v % N) * S;
        double sum = 0;
        for (int i = lane; i < S; i += 32) sum += (double)x[i] * (double)x[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) nrm[v] = (float)(1.0 / sqrt(sum + (double)a.eps));
    }
    __syncthreads();
    {
        const float q_scale = (float)(1.0 / sqrt((double)S));
        for (int i = threadIdx.x; i < N * S; i += blockDim.x) {
            int node = i / S;
            qn[i] *= nrm[node] * q_scale;
            kn[i] *= nrm[N + node] * 1.0f;
        }
    }
    __syncthreads();
    if (cb == 0 && h < a.groups) {
        for (int i = threadIdx.x; i < N * S; i += blockDim.x) {
            int node = i / S, e = i - node * S;
            a.khat[(int64_t)(seq * N + node) * key_dim + h * S + e] = kn[i];
        }
    }
    if (cb == 0)
        for (int node = threadIdx.x; node < N; node += blockDim.x) a.decay[(int64_t)(seq * N + node) * a.rank + h] = dec[node];

    // ---- recurrence: this thread holds rows [warp*RPW, +RPW) of column col ----
    int cur = -1;  // node whose state st currently holds (-1: the stored state)

    for (int node = 0; node < N; node++) {
        const int pnode = par[node];
        if (pnode != cur) {
            // a sibling branch: rebuild the parent's state from the stored one
            // by replaying the log of the parent's path
#pragma unroll
            for (int i = 0; i < RPW; i++) st[i] = s0[(int64_t)i * S];
            int path[GDN_MAX_NODES], len = 0;
            for (int c = pnode; c >= 0; c = par[c]) path[len++] = c;
            for (int j = len - 1; j >= 0; j--) {
                const int c = path[j];
                const float dc = dec[c], dv = dd[c * GDN_COLS + lane];
#pragma unroll
                for (int i = 0; i < RPW; i++) st[i] = state_update(st[i], dc, kn[c * S + warp * RPW + i], dv);
            }
        }
        const float * kx = kn + node * S + warp * RPW;
        const float * qx = qn + node * S + warp * RPW;
        const float dc = dec[node];
        // sk = (decay * S)^T k
        float sk = 0.0f;
#pragma unroll
        for (int i = 0; i < RPW; i++) sk = fmaf(st[i] * dc, kx[i], sk);
        red[warp * GDN_COLS + lane] = sk;
        __syncthreads();
        sk = 0.0f;
#pragma unroll
        for (int w = 0; w < GDN_WARPS; w++) sk += red[w * GDN_COLS + lane];
        const float d = (vv[node * GDN_COLS + lane] - sk) * bet[node];
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < RPW; i++) {
            st[i] = state_update(st[i], dc, kx[i], d);
            o = fmaf(st[i], qx[i], o);
        }
        red2[warp * GDN_COLS + lane] = o;
        if (warp == 0) dd[node * GDN_COLS + lane] = d;
        __syncthreads();
        // red is rewritten only after the next barrier, red2 only after the one after that
        if (warp == 0) {
            o = 0.0f;
#pragma unroll
            for (int w = 0; w < GDN_WARPS; w++) o += red2[w * GDN_COLS + lane];
            a.out[(int64_t)(seq * N + node) * (a.rank * S) + h * S + col] = o;
            a.dlog[(int64_t)(seq * N + node) * (a.rank * S) + h * S + col] = d;
        }
        cur = node;
    }
}

void launch_gdn_scan(cudaStream_t s, const GdnArgs & a, const RowMeta & rows) {
    YK_REQUIRE(rows.nodes <= GDN_MAX_NODES, YUUKA_ERR_UNSUPPORTED, "gdn: at most %d rows per sequence", GDN_MAX_NODES);
    YK_REQUIRE(a.kernel >= 2 && a.kernel <= 8, YUUKA_ERR_UNSUPPORTED, "gdn: conv kernel %d is outside 2..8", a.kernel);
    ScanParams p{a, rows};
    const int N = rows.nodes;
    const int nch = 2 * a.S + GDN_COLS;
    size_t smem = sizeof(float) * ((size_t)2 * N * a.S + 2 * N * GDN_COLS + 2 * N + 2 * GDN_WARPS * GDN_COLS +
                                   (size_t)(a.kernel - 1 + N) * nch + (size_t)nch * a.kernel + N);
    dim3 grid(a.S / GDN_COLS, a.rank, rows.batch);
    if (a.S == 128) {
        YK_CUDA(cudaFuncSetAttribute(gdn_scan_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        gdn_scan_kernel<128><<<grid, GDN_WARPS * 32, smem, s>>>(p);
    } else if (a.S == 64) {
        YK_CUDA(cudaFuncSetAttribute(gdn_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        gdn_scan_kernel<64><<<grid, GDN_WARPS * 32, smem, s>>>(p);
    } else {
        YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED, "gdn: state size %d is not 64 or 128", a.S);
    }
    YK_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// commit

struct CommitParams {
    const GdnLayerCommit * layers;
    int groups, rank, S, kernel, conv_dim;
    int seq_base;  // first sequence of the step within the session's state arrays
    RowMeta rows;
    AcceptOut acc;
};

// grid (rank + 1, batch, layers): blocks 0..rank-1 update one head's state,
// block `rank` rewrites the conv history.
__global__ void __launch_bounds__(256) gdn_commit_kernel(const CommitParams p) {
    const GdnLayerCommit L = p.layers[blockIdx.z];
    const int seq = blockIdx.y, N = p.rows.nodes, S = p.S;
    const int a = p.acc.accepted[seq];
    const int32_t * path = p.acc.path + (int64_t)seq * N;
    auto node_at = [&](int t) { return t == 0 ? 0 : path[t - 1]; };  // t = 0..a
    if ((int)blockIdx.x < p.rank) {
        const int h = blockIdx.x, kh = h % p.groups;
        float * st = L.state + (int64_t)((p.seq_base + seq) * p.rank + h) * S * S;
        for (int e = threadIdx.x; e < S * S; e += blockDim.x) {
            const int i = e / S, j = e - i * S;
            float v = st[e];
            for (int t = 0; t <= a; t++) {
                const int r = seq * N + node_at(t);
                v = state_update(v, L.decay[(int64_t)r * p.rank + h], L.khat[(int64_t)r * (p.groups * S) + kh * S + i],
                                 L.dlog[(int64_t)r * (p.rank * S) + h * S + j]);
            }
            st[e] = v;
        }
    } else {
        // history after the step = last kernel-1 raw inputs of [old history, accepted rows]
        const int K1 = p.kernel - 1, n_new = a + 1;
        for (int c = threadIdx.x; c < p.conv_dim; c += blockDim.x) {
            float * hist = L.conv_state + ((int64_t)(p.seq_base + seq) * p.conv_dim + c) * K1;
            float nv[8];
            for (int t = 0; t < K1; t++) {
                int src = n_new + t - K1 + 0;  // index into the accepted rows; negative = old history
                // combined sequence index: old history occupies [-K1, -1], accepted rows [0, n_new-1];
                // new history entry t takes combined index n_new - K1 + t
                if (src >= 0) nv[t] = L.proj[(int64_t)(seq * N + node_at(src)) * L.ldp + c];
                else nv[t] = hist[K1 + src];
            }
            for (int t = 0; t < K1; t++) hist[t] = nv[t];
        }
    }
}

void launch_gdn_commit(cudaStream_t s, const GdnLayerCommit * layers_dev, int n_layers, int groups, int rank, int S,
                       int kernel, int conv_dim, int seq_base, const RowMeta & rows, const AcceptOut & acc) {
    if (n_layers == 0) return;
    CommitParams p{layers_dev, groups, rank, S, kernel, conv_dim, seq_base, rows, acc};
    dim3 grid(rank + 1, rows.batch, n_layers);
    gdn_commit_kernel<<<grid, 256, 0, s>>>(p);
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
    const KvLayerCommit L = p.layers[blockIdx.y];
    const int seq = blockIdx.x, N = p.rows.nodes;
    const int a = p.acc.accepted[seq];
    const int pos0 = p.rows.pos0[seq];
    const int32_t * path = p.acc.path + (int64_t)seq * N;
    const int words = p.geom.row_bytes / 2;
    for (int t = 1; t <= a; t++) {
        const int node = path[t - 1];
        if (node != t) {
            auto off = [&](int slot) {
                int block = p.geom.tables[(int64_t)seq * p.geom.table_stride + slot / p.geom.block_size];
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
    kv_commit_kernel<<<grid, 256, 0, s>>>(p);
    YK_CUDA(cudaGetLastError());
}

__global__ void advance_positions_kernel(int32_t * pos0, const int32_t * accepted, int batch) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) pos0[b] += accepted[b] + 1;
}

void launch_advance_positions(cudaStream_t s, int32_t * pos0, const AcceptOut & acc, int batch) {
    advance_positions_kernel<<<(batch + 127) / 128, 128, 0, s>>>(pos0, acc.accepted, batch);
    YK_CUDA(cudaGetLastError());
}

}  // namespace yk
