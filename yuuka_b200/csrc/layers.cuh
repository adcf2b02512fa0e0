// Host interface of the non-GEMM kernels of the verify step.
#pragma once

#include "common.cuh"
#include "xprep.cuh"

namespace yk {

// Per-step row metadata, all device pointers. Row r = seq * nodes + node.
struct RowMeta {
    const int32_t * tokens;    // [rows]
    const int32_t * parent;    // [rows] node index of the preceding row within the sequence, -1 for node 0
    const int32_t * depth;     // [rows] number of ancestors
    const uint64_t * anc_mask; // [rows] bit j set iff node j is the row itself or one of its ancestors
    const int32_t * pos0;      // committed positions, indexed by sequence (see seq_map)
    int batch, nodes;
    // [batch] or null: which of the session's sequences each slot of the step is. Positions, block tables,
    // recurrent state and conv history are indexed by it; everything that only lives for the step (rows,
    // logits, results) is indexed by the slot. Null: slot b is sequence b of the arrays as passed.
    const int32_t * seq_map = nullptr;
    // set by the host when it staged no parent pointers: every sequence of the step is a chain (row i follows
    // row i - 1), which lets the delta-net scan walk the rows in order without looking for branches
    int chains = 0;
};
#ifdef __CUDACC__
__device__ __forceinline__ int seq_of(const RowMeta & rows, int slot) { return rows.seq_map ? rows.seq_map[slot] : slot; }
#endif

struct KvPool {
    uint8_t * k;
    uint8_t * v;
    int format;        // yuuka_kv_format
    int block_size;
    int pool_blocks;
    int kv_dim;
    int row_bytes;
    const int32_t * tables;  // [batch][table_stride]
    int table_stride;
};

// x[r][:] = dequantized row tokens[r] of the embedding table (forward.go:120-129)
void launch_embedding(cudaStream_t s, float * x, int ldx, const uint8_t * table, uint32_t dtype, int hidden,
                      int vocab, const int32_t * tokens, int rows);
// The same with the first layer's input RMSNorm of every row (and, rope_cs non-null, the rows' RoPE table, positions
// counted in table_rows' layout) done by the row's CTA: one launch instead of three at the start of a step.
void launch_embedding_first(cudaStream_t s, float * x, int ldx, const uint8_t * table, uint32_t dtype, int hidden, int vocab,
                            const int32_t * tokens, int rows, const float * norm_w, float * xn, int ldxn, float eps, XPrepOut prep,
                            unsigned long long * sumsq_out, float2 * rope_cs, const RowMeta & table_rows, int rope_dim,
                            double rope_base);
// dst[r][:] = src[r][:] * rsqrt(mean(src^2) + eps) * weight (forward.go:460-470)
void launch_rmsnorm(cudaStream_t s, float * dst, int ldd, const float * src, int lds, const float * weight,
                    int cols, int rows, float eps, XPrepOut prep = XPrepOut(),
                    unsigned long long * sumsq_out = nullptr);
// act[r][i] = silu(gate[r][i]) * up[r][i] (forward.go:307-309). gstride: distance between consecutive
// 16-column groups of gate (and of up); 32 when the two alternate 16 columns at a time in one row.
void launch_silu_mul(cudaStream_t s, float * act, int lda, const float * gate, const float * up, int ld, int cols,
                     int rows, XPrepOut prep = XPrepOut(), int gstride = 16);
// Per-head RMSNorm of q and k, RoPE at pos0 + depth, and the paged KV write of
// every row at slot pos0 + node (forward.go:172-186, kv_pool.go:117-134).
// rope_cs: (cos, sin) of each row's angles, [rows][rope_dim / 2], written once per step by launch_rope_table.
void launch_attn_prep(cudaStream_t s, float * q, int ldq, float * k, int ldk, const float * v, int ldv,
                      const float * q_norm, const float * k_norm, int heads, int kv_heads, int head_dim,
                      int rope_dim, const float2 * rope_cs, float eps, const RowMeta & rows, const KvPool & pool);
void launch_rope_table(cudaStream_t s, float2 * cs, const RowMeta & rows, int rope_dim, double rope_base);
// Paged attention of every row over the committed positions and the row's own
// ancestors, split over key ranges, then merged and gated (forward.go:188-220).
struct AttnScratch {
    float * partial;   // [rows*heads][splits][head_dim + 2]
    int splits;
    int key_split;     // keys per split
};
int launch_attention(cudaStream_t s, float * out, int ldo, const float * q, int ldq, int heads, int kv_heads,
                     int head_dim, const RowMeta & rows, const KvPool & pool, int max_total_keys,
                     const AttnScratch & scratch, XPrepOut prep = XPrepOut());
size_t attention_scratch_floats(int rows, int heads, int head_dim, int splits);
// CTAs per (sequence, KV head) of the tensor-core kernel for q_rows = rows per sequence x query heads per KV head.
int attention_query_tiles(int q_rows);

// Gated DeltaNet over the rows of a step (forward.go:245-287, recurrent.go:56-105).
struct GdnArgs {
    const float * proj;      // [rows][ldp]: qkv (conv_dim) | z (inner) | beta (rank) | alpha (rank)
    int ldp;
    const float * conv_w;    // [conv_dim][kernel]
    const float * dt;        // [rank]
    const float * a;         // [rank]
    const float * conv_state;  // [batch][conv_dim][kernel-1]
    const float * state;       // [batch][rank][S][S]
    const float * z;         // gate projection rows (= proj + conv_dim), leading dimension ldz
    int ldz;
    const float * norm;      // [S] gated-norm weight
    float * out;             // [rows][inner] gated head outputs (f32)
    XPrepOut prep;           // same, prepared for the out-projection GEMM
    float * qn;              // [rows][groups*S] scratch: normalised queries
    float * vconv;           // [rows][inner] scratch: conv output of v
    float * beta;            // [rows][rank] scratch
    float * khat;            // [rows][groups*S] log: normalised keys
    float * dlog;            // [rows][rank*S]   log: beta * (v - S^T k)
    float * decay;           // [rows][rank]     log: exp(alpha)
    int groups, rank, S, kernel;
    float eps;
};
// conv + norms, the recurrence and the gated RMSNorm; returns the number of kernels launched
int launch_gdn_scan(cudaStream_t s, const GdnArgs & a, const RowMeta & rows);
// Prompt passes (one chain, every row committed): the front end once for the whole pass, then the chunkwise WY
// form of the recurrence over chunks of at most 64 rows, which rewrites the state in place and writes no delta
// log; the conv history moves once per pass with launch_gdn_commit(..., conv_only = true).
void launch_gdn_front_chain(cudaStream_t s, const GdnArgs & a, int seq_slot, int n_rows);
void launch_gdn_chunk(cudaStream_t s, const GdnArgs & a, const RowMeta & rows);
// First-maximum argmax of every logits row (speculative.go:263-271) followed by
// the greedy tree walk (speculative.go:193-202 generalised to a tree).
struct AcceptOut {
    int32_t * accepted;  // [batch]
    int32_t * path;      // [batch][nodes]
    int32_t * emitted;   // [batch][nodes]
};
struct ArgmaxScratch {
    float * val;     // [rows][chunks]
    int32_t * idx;   // [rows][chunks]
    int chunks;
};
int launch_accept_greedy(cudaStream_t s, const float * logits, int vocab, const RowMeta & rows,
                         const ArgmaxScratch & scratch, const AcceptOut & out);
// Rejection-sampling walk (rule in accept.cu). residual is scratch of batch * vocab 64-bit words;
// draft_probs [batch][nodes][vocab] and uniforms [batch][nodes][2] are device arrays.
int launch_accept_rejection(cudaStream_t s, const float * logits, const float * draft_probs, const float * uniforms,
                            unsigned long long * residual, int vocab, float temperature, const RowMeta & rows,
                            const AcceptOut & out);
// Accept every row of a chain (prefill / forced commit): accepted = nodes-1.
void launch_accept_all(cudaStream_t s, const RowMeta & rows, const AcceptOut & out);
int argmax_chunks(int vocab);

// Commit of the accepted path: recurrent state, conv history, KV row moves,
// positions.
struct GdnLayerCommit {
    const float * proj;  // raw qkv rows of the step (first conv_dim columns of proj)
    int ldp;
    const float * khat;
    const float * dlog;
    const float * decay;
    float * conv_state;
    float * state;
};
void launch_gdn_commit(cudaStream_t s, const GdnLayerCommit * layers_dev, int n_layers, int groups, int rank, int S,
                       int kernel, int conv_dim, int seq_base, const RowMeta & rows, const AcceptOut & acc, int row_base = 0,
                       bool conv_only = false);
struct KvLayerCommit {
    uint8_t * k;
    uint8_t * v;
};
void launch_kv_commit(cudaStream_t s, const KvLayerCommit * layers_dev, int n_layers, const KvPool & geom,
                      const RowMeta & rows, const AcceptOut & acc);
// Device-side prompt-lookup draft of one sequence (draft.cu). The kernel first appends the tokens the previous
// step emitted (accepted != null) to the history, then looks up the next draft and writes the next step's token
// rows: the pending token, the draft, and the pending token again in the rows the draft does not fill.
struct DraftParams {
    int32_t * hist;            // tokens of the sequence so far; the last one is pending (emitted, not yet run)
    int32_t * hist_len;
    int hist_cap;
    const int32_t * accepted;  // the step that just ran: accepted count and emitted tokens of the slot, or null
    const int32_t * emitted;
    int32_t * rows_tokens;     // [nodes] token rows of the next step, or null
    int nodes;
    int max_draft, min_match;
    int32_t * stats;           // [4] or null: steps, draft tokens, accepted drafts, draft length of the staged step
    int32_t * draft_out;       // optional: the draft tokens alone
    int32_t * k_out;           // optional: the draft length
};
void launch_spec_draft(cudaStream_t s, const DraftParams & p);

void launch_advance_positions(cudaStream_t s, int32_t * pos0, const AcceptOut & acc, int batch, const int32_t * seq_map = nullptr);

// qwen35moe block (moe.cu)
struct GemmSegment;
int moe_max_segments(int pairs, int experts);
void launch_moe_route(cudaStream_t s, const float * xn, const float * router, const float * sh_gate, int hidden, int experts,
                      int used, int rows, int32_t * ids, float * weights, float * shared_gate, float * logits, int * counters);
void launch_moe_group(cudaStream_t s, const int32_t * ids, int rows, int used, int experts, int32_t * pos_of_pair,
                      int32_t * row_of_pos, GemmSegment * segments, int max_segments);
void launch_moe_combine(cudaStream_t s, float * x, const float * expert_out, const float * shared_out,
                        const int32_t * pos_of_pair, const float * weights, const float * shared_gate, int hidden, int used,
                        int rows);

}  // namespace yk
