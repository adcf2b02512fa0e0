// Large-M route of the tiled quantized GEMM: tcgen05 tensor cores with the
// accumulator in tensor memory. Included by gemm_tiled.cu (it uses that file's
// record codecs and header decoders).
//
// From 48 rows on (33 on request), re-decoding the packed weights for every 16-row pass of the
// register-fed MMA kernel costs more than the arithmetic. Here a CTA owns 128 weight rows and up to
// 256 activation rows (512 in the warp-specialised kernel, on two accumulators): eight warps decode one
// 16-row tile each into fp16 (s * q - min, rounded: this route does not have the register-fed route's
// exactness), 64 columns at a time, and store it into a shared-memory stage in the K-major core-matrix
// layout (8 rows x 16 bytes, no swizzle); the matching 64 columns of the prepared activations (their fp16
// hi halves) arrive in the same stage by a tensor-map copy (cp.async where the encoder is not available).
// One thread then issues four tcgen05.mma (M = 128, N = rows padded to 16, K = 16 each) that accumulate
// D[weight row][activation row] in tensor memory, and tcgen05.commit releases the stage through an
// mbarrier when they have read it. The ring of stages lets decoding run ahead of the tensor pipe. The
// epilogue reads the accumulator with tcgen05.ld (lane = weight row, column = activation row) and writes
// out[row][n], 128 bytes per warp store.
//
// Every mbarrier wait is bounded; on expiry the device error word is set, the
// kernel carries on (results are then garbage), frees its tensor memory and
// returns.
#pragma once

namespace yk {

constexpr int UM_ROWS = 128;   // weight rows per CTA = UMMA M
constexpr int UM_KC = 64;      // columns per stage
constexpr int UM_STAGES = 4;
constexpr int UM_AHEAD = 2;    // chunks of activations in flight ahead of the decode
constexpr int UM_MAX_N = 256;  // activation rows of one accumulator = UMMA N
constexpr int UM_MAX_N2 = 512; // activation rows per launch of the warp-specialised kernel: two accumulators fill tensor memory
// Weight stage: dense core matrices. Padding them to 160 bytes removes the four-way bank conflicts of the
// decode warps' 16-byte stores and measured the same overall (56.3 vs 55.8 us on 18432 x 2560 at 256 rows),
// so the smaller stage is kept; -DYK_UMMA_A_LBO=160 builds the padded form.
#ifndef YK_UMMA_A_LBO
#define YK_UMMA_A_LBO 128
#endif
constexpr int UM_A_LBO = YK_UMMA_A_LBO;
constexpr int UM_A_SBO = 8 * UM_A_LBO;                // one group of eight rows
constexpr int UM_A_BYTES = (UM_ROWS / 8) * UM_A_SBO;  // 16 KB
// Activation stage: core matrices 144 bytes apart along K (16 bytes of padding each), so that the eight
// 16-byte pieces of one row, copied by eight neighbouring lanes from 128 contiguous global bytes,
// land in different banks.
constexpr int UM_B_LBO = 144;
constexpr int UM_B_SBO = 8 * UM_B_LBO;  // one group of eight rows

struct UParams {
    DecodeConsts kc;
    const uint8_t * w;
    int N, nsb;           // weight rows, superblocks per row
    const __half * xh;    // prepared activations [M][nsb * 256]
    int M, npad;          // activation rows, padded to a multiple of 16
    float * out;
    int64_t ldo;
    int accumulate;
    uint32_t tmem_cols;   // power of two >= npad, >= 32
    uint32_t idesc;
    uint32_t idesc2;      // second accumulator (rows 256...), warp-specialised kernel with more than 256 rows; else 0
    uint32_t box_rows;    // rows of one tensor-map box: npad, or 256 with two accumulators
    uint32_t stages;      // ring depth: UM_STAGES, or fewer when four stages do not fit shared memory (at least 2)
    float * partial;      // [gridDim.y][M][N] when K is split across CTAs
    int * counters;       // one per block of 128 weight rows, zero between launches
};

// K-major, 128-byte swizzle: rows of 64 halves (128 bytes), eight rows per 1024-byte atom, as a tensor-map
// copy with CU_TENSOR_MAP_SWIZZLE_128B lays them out. 16 columns further along K = 32 bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)1u << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// ---- scaled fragments of one 32-column sub-block K of a record, as the register-fed kernel forms
// them: a[h][0], a[h][2] = row g, elements 8t + 4h + {0,1}, {2,3}; a[h][1], a[h][3] = row g + 8.
// `mg`, `mh` receive the half2 that still has to be added (-min, or -32 * scale for Q6_K).
__device__ __forceinline__ uint32_t h2_add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

template <int DT> struct SubBlock;

template <> struct SubBlock<YUUKA_DTYPE_Q4_K> {
    using C = Codec<YUUKA_DTYPE_Q4_K>;
    template <int K>
    __device__ static void frag(const typename C::Regs & r, int lane, const uint8_t * tab, const DecodeConsts & kc,
                                uint32_t (&a)[2][4], uint32_t & mg, uint32_t & mh) {
        constexpr int j = K >> 1, n = K & 1, jj = j >> 1, jl = j & 1;
        const int g = lane >> 2;
        const uint32_t qg[4] = {r.q[jj].x, r.q[jj].y, r.q[jj].z, r.q[jj].w};
        const uint32_t qh[4] = {r.q[2 + jj].x, r.q[2 + jj].y, r.q[2 + jj].z, r.q[2 + jj].w};
        const uint4 sg = reinterpret_cast<const uint4 *>(tab + g * C::SCL_STRIDE)[j];
        const uint4 sh = reinterpret_cast<const uint4 *>(tab + (g + 8) * C::SCL_STRIDE)[j];
        const uint32_t mask = n ? kc.mf0 : kc.m0f;
        const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t vg = qg[2 * jl + h], vh = qh[2 * jl + h];
            a[h][0] = h2_fma(and_or(vg, mask, kc.magic), s_g, c_g);
            a[h][1] = h2_fma(and_or(vh, mask, kc.magic), s_h, c_h);
            a[h][2] = h2_fma(and_or(vg >> 8, mask, kc.magic), s_g, c_g);
            a[h][3] = h2_fma(and_or(vh >> 8, mask, kc.magic), s_h, c_h);
        }
        mg = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + g * C::MN_STRIDE)[K];
        mh = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + (g + 8) * C::MN_STRIDE)[K];
    }
};

template <> struct SubBlock<YUUKA_DTYPE_Q5_K> {
    using C = Codec<YUUKA_DTYPE_Q5_K>;
    template <int K>
    __device__ static void frag(const typename C::Regs & r, int lane, const uint8_t * tab, const DecodeConsts & kc,
                                uint32_t (&a)[2][4], uint32_t & mg, uint32_t & mh) {
        constexpr int j = K >> 1, n = K & 1, jj = j >> 1, jl = j & 1;
        const int g = lane >> 2;
        const uint32_t qg[4] = {r.q[jj].x, r.q[jj].y, r.q[jj].z, r.q[jj].w};
        const uint32_t qh[4] = {r.q[2 + jj].x, r.q[2 + jj].y, r.q[2 + jj].z, r.q[2 + jj].w};
        const uint32_t hg[2] = {r.qh.x, r.qh.y}, hh[2] = {r.qh.z, r.qh.w};
        const uint4 sg = reinterpret_cast<const uint4 *>(tab + g * C::SCL_STRIDE)[j];
        const uint4 sh = reinterpret_cast<const uint4 *>(tab + (g + 8) * C::SCL_STRIDE)[j];
        const uint32_t s_g = n ? sg.z : sg.x, c_g = n ? sg.w : sg.y, s_h = n ? sh.z : sh.x, c_h = n ? sh.w : sh.y;
#pragma unroll
        for (int h = 0; h < 2; h++)
            Mma<YUUKA_DTYPE_Q5_K, 1>::template sub<K>(qg[2 * jl + h], qh[2 * jl + h], hg[h], hh[h], s_g, c_g, s_h, c_h, a[h], kc);
        mg = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + g * C::MN_STRIDE)[K];
        mh = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + (g + 8) * C::MN_STRIDE)[K];
    }
};

template <> struct SubBlock<YUUKA_DTYPE_Q6_K> {
    using C = Codec<YUUKA_DTYPE_Q6_K>;
    // Q6_K records keep a lane's eight elements of a sub-block in two runs of four (pos6): a[0][*] are elements
    // 4t + {0..3} (16-element group 2K), a[1][*] elements 16 + 4t + {0..3} (group 2K + 1). The offsets are added
    // here, per group; mg / mh come back as zero.
    template <int K>
    __device__ static void frag(const typename C::Regs & r, int lane, const uint8_t * tab, const DecodeConsts & kc,
                                uint32_t (&a)[2][4], uint32_t & mg, uint32_t & mh) {
        constexpr int n6 = K >> 2, nib = (K >> 1) & 1, hsel = K & 1;
        constexpr int lsh = 4 - 2 * hsel, rsh = 4 + 2 * hsel;
        const int g = lane >> 2;
        const uint32_t lg[4] = {r.ql[n6].x, r.ql[n6].y, r.ql[n6].z, r.ql[n6].w};
        const uint32_t lh[4] = {r.ql[2 + n6].x, r.ql[2 + n6].y, r.ql[2 + n6].z, r.ql[2 + n6].w};
        const uint32_t hg[2] = {n6 ? r.qh[0].z : r.qh[0].x, n6 ? r.qh[0].w : r.qh[0].y};
        const uint32_t hh[2] = {n6 ? r.qh[1].z : r.qh[1].x, n6 ? r.qh[1].w : r.qh[1].y};
        const uint32_t qm = nib ? kc.mf0 : kc.m0f, hm = nib ? kc.h8 : kc.h4;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int s16 = 2 * K + h;
            const uint2 eg = reinterpret_cast<const uint2 *>(tab + g * C::SCL_STRIDE)[s16];
            const uint2 eh = reinterpret_cast<const uint2 *>(tab + (g + 8) * C::SCL_STRIDE)[s16];
            const uint32_t og = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + g * C::MN_STRIDE)[s16];
            const uint32_t oh = reinterpret_cast<const uint32_t *>(tab + C::MN_OFF + (g + 8) * C::MN_STRIDE)[s16];
            const uint32_t vg = lg[2 * hsel + h], vh = lh[2 * hsel + h];
            a[h][0] = h2_add(h2_fma(and_or(vg, qm, and_or(hg[h] << lsh, hm, kc.magic)), eg.x, eg.y), og);
            a[h][1] = h2_add(h2_fma(and_or(vh, qm, and_or(hh[h] << lsh, hm, kc.magic)), eh.x, eh.y), oh);
            a[h][2] = h2_add(h2_fma(and_or(vg >> 8, qm, and_or(hg[h] >> rsh, hm, kc.magic)), eg.x, eg.y), og);
            a[h][3] = h2_add(h2_fma(and_or(vh >> 8, qm, and_or(hh[h] >> rsh, hm, kc.magic)), eh.x, eh.y), oh);
        }
        mg = 0u;
        mh = 0u;
    }
};

template <> struct SubBlock<YUUKA_DTYPE_Q8_0> {
    using C = Codec<YUUKA_DTYPE_Q8_0>;
    template <int K>
    __device__ static void frag(const typename C::Regs & r, int lane, const uint8_t * tab, const DecodeConsts & kc,
                                uint32_t (&a)[2][4], uint32_t & mg, uint32_t & mh) {
        (void)kc;
        constexpr int kk = K >> 1, kl = K & 1;
        const int g = lane >> 2;
        const uint32_t qg[4] = {r.q[kk].x, r.q[kk].y, r.q[kk].z, r.q[kk].w};
        const uint32_t qh[4] = {r.q[4 + kk].x, r.q[4 + kk].y, r.q[4 + kk].z, r.q[4 + kk].w};
        const uint32_t sg = reinterpret_cast<const uint32_t *>(tab + g * C::SCL_STRIDE)[K];
        const uint32_t sh = reinterpret_cast<const uint32_t *>(tab + (g + 8) * C::SCL_STRIDE)[K];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t vg = qg[2 * kl + h] ^ 0x80808080u, vh = qh[2 * kl + h] ^ 0x80808080u;
            a[h][0] = h2_mul(h2_sub(bytes02_h2(vg), H2_1152), sg);
            a[h][1] = h2_mul(h2_sub(bytes02_h2(vh), H2_1152), sh);
            a[h][2] = h2_mul(h2_sub(bytes13_h2(vg), H2_1152), sg);
            a[h][3] = h2_mul(h2_sub(bytes13_h2(vh), H2_1152), sh);
        }
        mg = 0u;
        mh = 0u;
    }
};

// K-major, no swizzle: core matrix (8 rows x 16 bytes) at rowgroup * 1024 + kchunk * 128 inside a stage
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo = 128u, uint32_t sbo = 1024u) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t i = 0; i < (1u << 22) && !ok; i++) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
    }
    return ok != 0;
}

template <int DT, int K>
__device__ __forceinline__ void umma_store_subblock(const typename Codec<DT>::Regs & r, int lane, const uint8_t * tab,
                                                    const DecodeConsts & kc, uint8_t * a_stage, int warp, int kblk_in_stage) {
    uint32_t a[2][4], mg, mh;
    SubBlock<DT>::template frag<K>(r, lane, tab, kc, a, mg, mh);
    const int g = lane >> 2, t = lane & 3;
    if constexpr (DT == YUUKA_DTYPE_Q6_K) {
        // two runs of four columns: 4t.. (first half of the sub-block) and 16 + 4t..
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int col = 16 * h + 4 * t, kchunk = 4 * kblk_in_stage + (col >> 3), off = g * 16 + (col & 7) * 2;
            *reinterpret_cast<uint2 *>(a_stage + (2 * warp) * UM_A_SBO + kchunk * UM_A_LBO + off) = make_uint2(a[h][0], a[h][2]);
            *reinterpret_cast<uint2 *>(a_stage + (2 * warp + 1) * UM_A_SBO + kchunk * UM_A_LBO + off) = make_uint2(a[h][1], a[h][3]);
        }
        return;
    }
    const int kchunk = 4 * kblk_in_stage + t;  // eight columns each
    uint4 vg = make_uint4(a[0][0], a[0][2], a[1][0], a[1][2]);
    uint4 vh = make_uint4(a[0][1], a[0][3], a[1][1], a[1][3]);
    if (DT != YUUKA_DTYPE_Q8_0) {
        vg = make_uint4(h2_add(vg.x, mg), h2_add(vg.y, mg), h2_add(vg.z, mg), h2_add(vg.w, mg));
        vh = make_uint4(h2_add(vh.x, mh), h2_add(vh.y, mh), h2_add(vh.z, mh), h2_add(vh.w, mh));
    }
    *reinterpret_cast<uint4 *>(a_stage + (2 * warp) * UM_A_SBO + kchunk * UM_A_LBO + g * 16) = vg;
    *reinterpret_cast<uint4 *>(a_stage + (2 * warp + 1) * UM_A_SBO + kchunk * UM_A_LBO + g * 16) = vh;
}

template <int DT, int Q>
__device__ __forceinline__ void umma_store_chunk(const typename Codec<DT>::Regs & r, int lane, const uint8_t * tab,
                                                 const DecodeConsts & kc, uint8_t * a_stage, int warp) {
    umma_store_subblock<DT, 2 * Q>(r, lane, tab, kc, a_stage, warp, 0);
    umma_store_subblock<DT, 2 * Q + 1>(r, lane, tab, kc, a_stage, warp, 1);
}

// TMA: the activation stage is filled by one cp.async.bulk.tensor per chunk (2-D map over the prepared
// activations, box 64 columns x npad rows, 128-byte swizzle, rows beyond M zero-filled) that completes on
// full_bar; otherwise by 16-byte cp.async copies into padded core matrices.
template <int DT, bool TMA>
__global__ void __launch_bounds__(TW * 32, 2) gemm_umma_kernel(const UParams p, const __grid_constant__ CUtensorMap xmap) {
    using C = Codec<DT>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // the swizzled stage needs 1024-byte alignment
    uint8_t * smem = smem_raw + ((1024u - ((uint32_t)__cvta_generic_to_shared(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t empty_bar[UM_STAGES];
    __shared__ __align__(8) uint64_t full_bar[UM_STAGES];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int last_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b_bytes = TMA ? (uint32_t)p.npad * 128u : (uint32_t)(p.npad >> 3) * UM_B_SBO;
    const uint32_t stage_bytes = UM_A_BYTES + b_bytes;
    uint8_t * tabs = smem + (size_t)p.stages * stage_bytes;
    uint8_t * tab = tabs + warp * C::TAB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < UM_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&empty_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&full_bar[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&done_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(&tmem_slot)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem_slot;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);  // (1024-byte aligned)
    const DecodeConsts kc = p.kc;

    const int n_tiles = (p.N + 15) >> 4;
    const int n_blocks = (p.N + UM_ROWS - 1) / UM_ROWS;
    const size_t rec_row = (size_t)p.nsb * C::REC;
    const int K = p.nsb * 256;
    // this CTA's share of K (superblocks), when K is split across gridDim.y
    const int sb_begin = (int)(((long long)p.nsb * blockIdx.y) / gridDim.y);
    const int sb_end = (int)(((long long)p.nsb * (blockIdx.y + 1)) / gridDim.y);
    const int chunks_per_block = (sb_end - sb_begin) * 4;
    bool expired = false;

    // activations of one chunk: columns [col0, col0 + 64) of every row into the stage
    auto issue_x = [&](uint32_t stage, int col0) {
        uint8_t * b_stage = smem + (size_t)stage * stage_bytes + UM_A_BYTES;
        if constexpr (TMA) {
            if (threadIdx.x == 0) {
                const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&full_bar[stage]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b_bytes) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    :
                    : "r"((uint32_t)__cvta_generic_to_shared(b_stage)), "l"(&xmap), "r"(col0), "r"(0), "r"(bar)
                    : "memory");
            }
        } else {
            for (int i = threadIdx.x; i < p.npad * 8; i += TW * 32) {
                const int tok = i >> 3, kch = i & 7;
                const __half * src = p.xh + (size_t)min(tok, p.M - 1) * K + col0 + kch * 8;
                const uint32_t dst =
                    (uint32_t)__cvta_generic_to_shared(b_stage + (tok >> 3) * UM_B_SBO + kch * UM_B_LBO + (tok & 7) * 16);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
        }
    };
    // column offset of chunk number `ci` counted from this CTA's first chunk (blocks repeat the same columns)
    auto chunk_col = [&](uint32_t ci) { return sb_begin * 256 + (int)(ci % (uint32_t)chunks_per_block) * UM_KC; };

    pdl_trigger();
    typename C::Regs cur, nxt;
    {
        const int rt = min(blockIdx.x * (UM_ROWS / 16) + warp, n_tiles - 1);
        if (sb_begin < sb_end) C::load(p.w + rt * rec_row + (size_t)sb_begin * C::REC, lane, cur);
    }
    pdl_wait();

    uint32_t chunk = 0;  // chunks started by this CTA so far (stage = chunk % p.stages)
    uint32_t block_iter = 0;
    // chunks this CTA will run in total, and the first UM_AHEAD activation copies
    uint32_t total_chunks = 0;
    if (chunks_per_block > 0 && (int)blockIdx.x < n_blocks)
        total_chunks = (uint32_t)((n_blocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1) * (uint32_t)chunks_per_block;
    for (uint32_t ci = 0; ci < UM_AHEAD; ci++) {
        if (ci < total_chunks) issue_x(ci % p.stages, chunk_col(ci));
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int rb = blockIdx.x; rb < n_blocks && chunks_per_block > 0; rb += gridDim.x, block_iter++) {
        const int rt = min(rb * (UM_ROWS / 16) + warp, n_tiles - 1);
        const uint8_t * tile = p.w + rt * rec_row;
        const bool more_blocks = rb + (int)gridDim.x < n_blocks;
        for (int sb = sb_begin; sb < sb_end; sb++) {
            if (sb + 1 < sb_end) {
                C::load(tile + (size_t)(sb + 1) * C::REC, lane, nxt);
            } else if (more_blocks) {
                const int rtn = min((rb + (int)gridDim.x) * (UM_ROWS / 16) + warp, n_tiles - 1);
                C::load(p.w + rtn * rec_row + (size_t)sb_begin * C::REC, lane, nxt);
            }
            Mma<DT, 1>::header(cur, lane, tab);
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t stage = chunk % p.stages;
                uint8_t * a_stage = smem + (size_t)stage * stage_bytes;
                // start the activations of chunk + UM_AHEAD: the tensor pipe must have read that stage's previous contents
                {
                    const uint32_t nchunk = chunk + UM_AHEAD;
                    if (nchunk < total_chunks) {
                        const uint32_t nstage = nchunk % p.stages, nuse = nchunk / p.stages;
                        if (nuse > 0 && !expired &&
                            !mbar_wait((uint32_t)__cvta_generic_to_shared(&empty_bar[nstage]), (nuse - 1) & 1))
                            expired = true;
                        issue_x(nstage, chunk_col(nchunk));
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
                // this chunk's stage: free since the wait made when its activations were started (UM_AHEAD chunks ago)
                // weights: this warp's 16 rows x 64 columns (the stage was waited for when its activations were started)
                if (q == 0) umma_store_chunk<DT, 0>(cur, lane, tab, kc, a_stage, warp);
                else if (q == 1) umma_store_chunk<DT, 1>(cur, lane, tab, kc, a_stage, warp);
                else if (q == 2) umma_store_chunk<DT, 2>(cur, lane, tab, kc, a_stage, warp);
                else umma_store_chunk<DT, 3>(cur, lane, tab, kc, a_stage, warp);
                if constexpr (!TMA) asm volatile("cp.async.wait_group %0;" ::"n"(UM_AHEAD) : "memory");  // this chunk's have landed
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncthreads();
                if (threadIdx.x == 0) {
                    if constexpr (TMA) {
                        if (!expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&full_bar[stage]), (chunk / p.stages) & 1))
                            expired = true;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc(smem_base + stage * stage_bytes, UM_A_LBO, UM_A_SBO);
                    const uint64_t db = TMA ? umma_desc_sw128(smem_base + stage * stage_bytes + UM_A_BYTES)
                                            : umma_desc(smem_base + stage * stage_bytes + UM_A_BYTES, UM_B_LBO, UM_B_SBO);
                    const uint32_t b_step = TMA ? 2u : (uint32_t)(2 * UM_B_LBO / 16);
#pragma unroll
                    for (int j = 0; j < UM_KC / 16; j++) {
                        const uint32_t accumulate = (sb > sb_begin || q > 0 || j > 0) ? 1u : 0u;
                        // 16 columns = two core matrices = 256 bytes further along K
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                            :
                            : "r"(taddr), "l"(da + (uint64_t)(j * (2 * UM_A_LBO / 16))), "l"(db + (uint64_t)(j * b_step)), "r"(p.idesc), "r"(accumulate),
                              "r"(0u)
                            : "memory");
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     (uint32_t)__cvta_generic_to_shared(&empty_bar[stage]))
                                 : "memory");
                }
                chunk++;
            }
            __syncwarp();
            cur = nxt;
        }
        // ---- epilogue of this block of 128 weight rows ----
        if (threadIdx.x == 0)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(&done_bar))
                         : "memory");
        if (!expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&done_bar), block_iter & 1)) expired = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            // warp w reads TMEM lanes 32 * (w % 4) ..; warps 0-3 take the even 32-column groups, 4-7 the odd ones
            const int quad = warp & 3;
            const int n = rb * UM_ROWS + quad * 32 + lane;
            const bool split = gridDim.y > 1;
            float * base = split ? p.partial + (size_t)blockIdx.y * p.M * p.N : p.out;
            const int64_t ld = split ? p.N : p.ldo;
            for (int c0 = (warp >> 2) * 32; c0 < p.npad; c0 += 64) {
                uint32_t v[32];
                const uint32_t src = taddr + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(src)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (n < p.N) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int tok = c0 + i;
                        if (tok < p.M) {
                            float * dst = base + (int64_t)tok * ld + n;
                            const float val = __uint_as_float(v[i]);
                            if (split) __stcg(dst, val);
                            else *dst = p.accumulate ? *dst + val : val;
                        }
                    }
                }
            }
        }
        if (gridDim.y > 1) {
            // K is split across CTAs: the last one to finish this block of rows sums the parts in a fixed order
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) last_flag = atomicAdd(&p.counters[rb], 1) == (int)gridDim.y - 1;
            __syncthreads();
            if (last_flag) {
                __threadfence();
                const int n0 = rb * UM_ROWS, nrows = min(UM_ROWS, p.N - n0);
                // four outputs per thread and trip: all their loads are issued before the first sum is formed
                const int total = p.M * nrows;
                for (int i0 = threadIdx.x; i0 < total; i0 += 4 * TW * 32) {
                    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f}, old[4];
                    float * dst[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int i = min(i0 + u * TW * 32, total - 1);
                        const int tok = i / nrows, n = n0 + i - tok * nrows;
                        dst[u] = p.out + (int64_t)tok * p.ldo + n;
                        old[u] = p.accumulate ? *dst[u] : 0.0f;
                    }
                    for (int part = 0; part < (int)gridDim.y; part++) {
                        float v[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int i = min(i0 + u * TW * 32, total - 1);
                            const int tok = i / nrows, n = n0 + i - tok * nrows;
                            v[u] = __ldcg(p.partial + ((size_t)part * p.M + tok) * p.N + n);
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) sum[u] += v[u];
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (i0 + u * TW * 32 < total) *dst[u] = old[u] + sum[u];
                }
                if (threadIdx.x == 0) p.counters[rb] = 0;
            }
        }
        // the next block overwrites the accumulator: everybody must have read it
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (expired) atomicExch(&g_gemm_wait_expired, 2);
    // every MMA this CTA issued has completed (the last done_bar wait), nothing reads TMEM any more
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(p.tmem_cols) : "memory");
}

// ---------------------------------------------------------------------------
// Warp-specialised variant (tensor-map activations only): eight decode warps, a copy warp and an issue warp.
// The decode warps never meet at a CTA-wide barrier inside a block of rows: each announces its
// share of a stage on afull_bar (eight arrivals) and moves on to the next stage as soon as
// empty_bar says the tensor pipe has drained it. Lane 0 of the copy warp starts the activation copy of
// a stage as soon as it is free; lane 0 of the issue warp waits for (activations landed, weights
// decoded), issues the MMAs and commits the stage back. tmem_free_bar (eight arrivals) tells it that
// the epilogue has read the accumulator before the next block of rows overwrites it. (Sixteen decode
// warps, two per tile on alternate chunks, measured slower on wide matrices: 96 registers per thread
// spill and the doubled scale tables cost a ring stage.)
// 32 accumulator values of one weight row (this lane's) for 32 consecutive activation rows, to out[row][n]:
// MODE 0 stores, 1 adds to what is there, 2 stores a K part past L1. `lim` = rows that exist. One pointer step
// per value: the per-value bounds, mode and 64-bit index arithmetic of a generic loop were a third of the
// kernel's instructions at 256 rows and half of them at 512.
template <int MODE>
__device__ __forceinline__ void umma_store_rows(float * dst, int64_t ld, const uint32_t (&v)[32], int lim) {
    if (lim >= 32) {
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const float val = __uint_as_float(v[i]);
            if (MODE == 2) __stcg(dst, val);
            else if (MODE == 1) *dst += val;
            else *dst = val;
            dst += ld;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) {
            if (i < lim) {
                const float val = __uint_as_float(v[i]);
                if (MODE == 2) __stcg(dst, val);
                else if (MODE == 1) *dst += val;
                else *dst = val;
            }
            dst += ld;
        }
    }
}

// Decode warps of the warp-specialised kernel: TW (one per 16-row tile), or 2 * TW: the two warps of a tile take
// alternate 64-column chunks of every record (-DYK_UMMA_DECODE_WARPS=16). Measured with sixteen (112 registers,
// 60-260 bytes of spills): Q4_K 18432 x 2560 at 256 / 512 rows 52.7 -> 50.4 / 70.6 -> 65.7 us, but the Q6_K
// LM head 567 -> 745 us and a 64-row step 6.66 -> 6.96 ms, so eight stay. Asking the records four or eight
// superblocks ahead into L2 changed nothing either: neither the latency of the weight loads nor the number of
// decoding warps is what bounds the loop.
#ifndef YK_UMMA_DECODE_WARPS
#define YK_UMMA_DECODE_WARPS 8
#endif
constexpr int UM_DW = YK_UMMA_DECODE_WARPS;
static_assert(UM_DW == TW || UM_DW == 2 * TW, "one or two decode warps per 16-row tile");
constexpr int UM_WS_THREADS = (UM_DW + 2) * 32;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(UM_WS_THREADS, 1) gemm_umma_ws_kernel(const UParams p, const __grid_constant__ CUtensorMap xmap) {
    using C = Codec<DT>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t * smem = smem_raw + ((1024u - ((uint32_t)__cvta_generic_to_shared(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t empty_bar[UM_STAGES];
    __shared__ __align__(8) uint64_t xfull_bar[UM_STAGES];
    __shared__ __align__(8) uint64_t afull_bar[UM_STAGES];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ __align__(8) uint64_t tmem_free_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int last_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t halves = p.idesc2 ? 2u : 1u;
    const uint32_t half_bytes = p.box_rows * 128u;
    const uint32_t b_bytes = halves * half_bytes;
    const uint32_t stage_bytes = UM_A_BYTES + b_bytes;
    uint8_t * tabs = smem + (size_t)p.stages * stage_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < UM_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&empty_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&xfull_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&afull_bar[s])), "r"(TW)
                         : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&done_bar)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_free_bar)), "r"(UM_DW)
                     : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(&tmem_slot)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem_slot;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    const int n_tiles = (p.N + 15) >> 4;
    const int n_blocks = (p.N + UM_ROWS - 1) / UM_ROWS;
    const size_t rec_row = (size_t)p.nsb * C::REC;
    const int sb_begin = (int)(((long long)p.nsb * blockIdx.y) / gridDim.y);
    const int sb_end = (int)(((long long)p.nsb * (blockIdx.y + 1)) / gridDim.y);
    const int chunks_per_block = (sb_end - sb_begin) * 4;
    uint32_t my_blocks = 0;
    if (chunks_per_block > 0 && (int)blockIdx.x < n_blocks) my_blocks = (uint32_t)((n_blocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1);
    const uint32_t total_chunks = my_blocks * (uint32_t)chunks_per_block;
    bool expired = false;

    pdl_trigger();
    if (warp == UM_DW) {
        // ---------------- copy warp: starts the activation copy of a stage as soon as it is free ----------------
        pdl_wait();
        if (lane == 0) {
            // ring positions are advanced by hand: the ring depth is a run-time value and a division per
            // chunk on a single thread's critical path would cost more than the work it issues
            uint32_t stage = 0, use = 0, in_block = 0;
            for (uint32_t n = 0; n < total_chunks; n++) {
                if (use > 0 && !expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&empty_bar[stage]), (use - 1) & 1))
                    expired = true;
                const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&xfull_bar[stage]);
                const int col0 = sb_begin * 256 + (int)in_block * UM_KC;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b_bytes) : "memory");
                for (uint32_t h = 0; h < halves; h++)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        :
                        : "r"(smem_base + stage * stage_bytes + UM_A_BYTES + h * half_bytes), "l"(&xmap), "r"(col0),
                          "r"((int)(h * UM_MAX_N)), "r"(bar)
                        : "memory");
                if (++stage == p.stages) { stage = 0; use++; }
                if (++in_block == (uint32_t)chunks_per_block) in_block = 0;
            }
        }
        __syncwarp();
    } else if (warp == UM_DW + 1) {
        // ---------------- issue warp: (activations landed, weights decoded) -> MMAs -> stage released ----------------
        if (lane == 0) {
            uint32_t stage = 0, use = 0, in_block = 0, blk = 0;
            uint32_t a_addr = smem_base, b_addr = smem_base + UM_A_BYTES;
            for (uint32_t c = 0; c < total_chunks; c++) {
                // the epilogue of the previous block must have read the accumulator
                if (in_block == 0 && blk > 0 && !expired &&
                    !mbar_wait((uint32_t)__cvta_generic_to_shared(&tmem_free_bar), (blk - 1) & 1))
                    expired = true;
                if (!expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&xfull_bar[stage]), use & 1)) expired = true;
                if (!expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&afull_bar[stage]), use & 1)) expired = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc(a_addr, UM_A_LBO, UM_A_SBO);
                const uint64_t db = umma_desc_sw128(b_addr);
                // rows 256... accumulate in tensor-memory columns 256...: the decoded weights are multiplied twice
                for (uint32_t h = 0; h < halves; h++) {
                    const uint32_t idesc = h ? p.idesc2 : p.idesc;
                    const uint64_t dbh = db + (uint64_t)(h * (half_bytes >> 4));
#pragma unroll
                    for (int j = 0; j < UM_KC / 16; j++) {
                        const uint32_t accumulate = (in_block > 0 || j > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                            :
                            : "r"(taddr + h * (uint32_t)UM_MAX_N), "l"(da + (uint64_t)(j * (2 * UM_A_LBO / 16))),
                              "l"(dbh + (uint64_t)(j * 2)), "r"(idesc), "r"(accumulate), "r"(0u)
                            : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 (uint32_t)__cvta_generic_to_shared(&empty_bar[stage]))
                             : "memory");
                if (in_block == (uint32_t)chunks_per_block - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     (uint32_t)__cvta_generic_to_shared(&done_bar))
                                 : "memory");
                a_addr += stage_bytes;
                b_addr += stage_bytes;
                if (++stage == p.stages) {
                    stage = 0;
                    use++;
                    a_addr = smem_base;
                    b_addr = smem_base + UM_A_BYTES;
                }
                if (++in_block == (uint32_t)chunks_per_block) { in_block = 0; blk++; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- decode warps ----------------
        uint8_t * tab = tabs + warp * C::TAB;
        const DecodeConsts kc = p.kc;
        const int tile = warp % TW, parity = warp / TW;  // with two warps per tile: chunks q with (q & 1) == parity
        typename C::Regs cur, nxt;
        if (my_blocks > 0) {
            const int rt = min(blockIdx.x * (UM_ROWS / 16) + tile, n_tiles - 1);
            C::load(p.w + rt * rec_row + (size_t)sb_begin * C::REC, lane, cur);
        }
        pdl_wait();
        uint32_t stage = 0, use = 0, block_iter = 0;
        for (int rb = blockIdx.x; rb < n_blocks && chunks_per_block > 0; rb += gridDim.x, block_iter++) {
            const int rt = min(rb * (UM_ROWS / 16) + tile, n_tiles - 1);
            const uint8_t * tile_w = p.w + rt * rec_row;
            const bool more_blocks = rb + (int)gridDim.x < n_blocks;
            for (int sb = sb_begin; sb < sb_end; sb++) {
                if (sb + 1 < sb_end) {
                    C::load(tile_w + (size_t)(sb + 1) * C::REC, lane, nxt);
                } else if (more_blocks) {
                    const int rtn = min((rb + (int)gridDim.x) * (UM_ROWS / 16) + tile, n_tiles - 1);
                    C::load(p.w + rtn * rec_row + (size_t)sb_begin * C::REC, lane, nxt);
                }
                Mma<DT, 1>::header(cur, lane, tab);
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint8_t * a_stage = smem + (size_t)stage * stage_bytes;
                    if (UM_DW > TW && (q & 1) != parity) {
                        if (++stage == p.stages) { stage = 0; use++; }
                        continue;
                    }
                    if (use > 0 && !expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&empty_bar[stage]), (use - 1) & 1))
                        expired = true;
                    if (q == 0) umma_store_chunk<DT, 0>(cur, lane, tab, kc, a_stage, tile);
                    else if (q == 1) umma_store_chunk<DT, 1>(cur, lane, tab, kc, a_stage, tile);
                    else if (q == 2) umma_store_chunk<DT, 2>(cur, lane, tab, kc, a_stage, tile);
                    else umma_store_chunk<DT, 3>(cur, lane, tab, kc, a_stage, tile);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive((uint32_t)__cvta_generic_to_shared(&afull_bar[stage]));
                    if (++stage == p.stages) { stage = 0; use++; }
                }
                __syncwarp();
                cur = nxt;
            }
            // ---- epilogue of this block of 128 weight rows ----
            if (!expired && !mbar_wait((uint32_t)__cvta_generic_to_shared(&done_bar), block_iter & 1)) expired = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool split = gridDim.y > 1;
            {
                const int quad = warp & 3;
                const int n = rb * UM_ROWS + quad * 32 + lane;
                float * base = split ? p.partial + (size_t)blockIdx.y * p.M * p.N : p.out;
                const int64_t ld = split ? p.N : p.ldo;
                for (int c0 = (warp >> 2) * 32; c0 < p.npad; c0 += (UM_DW / 4) * 32) {
                    uint32_t v[32];
                    const uint32_t src = taddr + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(src)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < p.N && c0 < p.M) {
                        float * dst = base + (int64_t)c0 * ld + n;
                        if (split) umma_store_rows<2>(dst, ld, v, p.M - c0);
                        else if (p.accumulate) umma_store_rows<1>(dst, ld, v, p.M - c0);
                        else umma_store_rows<0>(dst, ld, v, p.M - c0);
                    }
                }
            }
            // the accumulator has been read: the issue warp may start the next block of rows
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive((uint32_t)__cvta_generic_to_shared(&tmem_free_bar));
            if (split && p.counters) {
                // K is split across CTAs: the last one to finish this block of rows sums the parts in a fixed order
                // (without counters the parts are summed by umma_reduce_kernel, launched next)
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(UM_DW * 32) : "memory");
                if (threadIdx.x == 0) last_flag = atomicAdd(&p.counters[rb], 1) == (int)gridDim.y - 1;
                asm volatile("bar.sync 1, %0;" ::"n"(UM_DW * 32) : "memory");
                if (last_flag) {
                    __threadfence();
                    const int n0 = rb * UM_ROWS, nrows = min(UM_ROWS, p.N - n0);
                    const int total = p.M * nrows;
                    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * UM_DW * 32) {
                        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f}, old[4];
                        float * dst[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int i = min(i0 + u * UM_DW * 32, total - 1);
                            const int tok = i / nrows, n = n0 + i - tok * nrows;
                            dst[u] = p.out + (int64_t)tok * p.ldo + n;
                            old[u] = p.accumulate ? *dst[u] : 0.0f;
                        }
                        for (int part = 0; part < (int)gridDim.y; part++) {
                            float v[4];
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int i = min(i0 + u * UM_DW * 32, total - 1);
                                const int tok = i / nrows, n = n0 + i - tok * nrows;
                                v[u] = __ldcg(p.partial + ((size_t)part * p.M + tok) * p.N + n);
                            }
#pragma unroll
                            for (int u = 0; u < 4; u++) sum[u] += v[u];
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (i0 + u * UM_DW * 32 < total) *dst[u] = old[u] + sum[u];
                    }
                    if (threadIdx.x == 0) p.counters[rb] = 0;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(UM_DW * 32) : "memory");  // last_flag is reused by the next block
            }
        }
    }
    if (expired) atomicExch(&g_gemm_wait_expired, 3);
    // all MMAs have completed (every block's done_bar was waited for) and all epilogue loads are done
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(p.tmem_cols) : "memory");
}

// Sum of the K parts of a split tensor-memory GEMM, in part order: out[tok][n] (+)= sum over parts of
// partial[part][tok][n]. With many parts and hundreds of activation rows the whole machine sums; the last CTA
// of a 128-row block doing it alone took longer than the decode the split saved.
__global__ void __launch_bounds__(256) umma_reduce_kernel(float * __restrict__ out, int64_t ldo, const float * __restrict__ partial,
                                                          int parts, int M, int N, int accumulate) {
    pdl_entry();
    const int n4 = N >> 2;
    const int64_t total = (int64_t)M * n4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int tok = (int)(i / n4), n = (int)(i - (int64_t)tok * n4) * 4;
        float4 * dst = reinterpret_cast<float4 *>(out + (int64_t)tok * ldo + n);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int part = 0; part < parts; part++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(partial + ((size_t)part * M + tok) * N + n));
            sum.x += v.x;
            sum.y += v.y;
            sum.z += v.z;
            sum.w += v.w;
        }
        if (accumulate) {
            const float4 old = *dst;
            sum.x = old.x + sum.x;
            sum.y = old.y + sum.y;
            sum.z = old.z + sum.z;
            sum.w = old.w + sum.w;
        }
        *dst = sum;
    }
}

}  // namespace yk
