/* CPU oracle for the yuuka speculative-decoding verify path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU decoder (tensor/, model/qwen35/, memory/, engine/speculative.go). It is
 * the checker for the CUDA library and the timed CPU baseline of the bench; the
 * product library never links, loads or calls it.
 *
 * Parity status. The numeric primitives (dequantizers, half codec, matvec, KV
 * row codec, block-table map, lookupDraft, argmax, selectExperts, the
 * speculative accept loop) are pinned by the known-answer vectors of the
 * reference's own unit tests. End-to-end logits and token streams are
 * "parity unpinned": the reference keeps golden token ids only for real model
 * files that are not available, and it cannot be executed here (Go toolchain
 * absent). Tree verification and rejection sampling have no counterpart in the
 * reference at all; they are defined by this file and checked through
 * properties (tree == per-path chain, T->0 rejection == greedy).
 */
#ifndef YUUKA_ORACLE_H
#define YUUKA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML dtype ids (tensor/dtype.go:14-48). */
enum {
    YO_F32 = 0, YO_F16 = 1, YO_Q4_0 = 2, YO_Q5_0 = 6, YO_Q8_0 = 8,
    YO_Q4_K = 12, YO_Q5_K = 13, YO_Q6_K = 14
};
/* KV storage formats (model/qwen35/kv_format.go:16-24). */
enum { YO_KV_F32 = 0, YO_KV_F16 = 1, YO_KV_Q8_0 = 2 };

typedef struct yo_config {
    int32_t block_count, context_length, hidden, ffn;
    int32_t heads, kv_heads, head_dim, rope_dim;
    double rope_freq_base;
    float rms_eps;
    int32_t vocab;
    int32_t conv_kernel, state_size, group_count, time_step_rank, inner_size;
    int32_t full_attention_interval;
    int32_t expert_count, expert_used, expert_ffn, shared_ffn;
} yo_config;

typedef struct yo_model yo_model;
typedef struct yo_state yo_state;

/* ---- numeric primitives ---- */
uint16_t yo_f32_to_f16(float f);
float yo_f16_to_f32(uint16_t h);
int64_t yo_row_bytes(int dtype, int64_t cols);                 /* <0 on error */
int yo_dequantize_row(float *dst, int64_t dst_len, int dtype, const uint8_t *src, int64_t src_len);
int yo_matmul(float *dst, const float *x, int batch, const uint8_t *w, int dtype,
              int64_t rows, int64_t cols);
void yo_set_threads(int n);   /* 0 = all cores */
int yo_get_threads(void);

int64_t yo_kv_row_bytes(int format, int kv_dim);
int yo_kv_encode_row(uint8_t *dst, int format, const float *src, int kv_dim);
int yo_kv_decode_row(float *dst, int format, const uint8_t *src, int kv_dim);
int yo_table_map(const int32_t *blocks, int n_blocks, int block_size, int pos,
                 int32_t *block, int32_t *offset);

int yo_config_validate(const yo_config *cfg, char *msg, size_t msg_len);
int yo_is_recurrent(const yo_config *cfg, int layer);

/* ---- isolated layer math, exposed for kernel-level parity tests ---- */
void yo_rms_norm(float *dst, const float *src, const float *weight, int n, float eps);
void yo_l2_norm_head(float *x, int n, float eps, float extra);
void yo_apply_rope(float *vec, int heads, int stride, int head_dim, int rot_dim, int pos, double base);
void yo_softmax_inplace(float *x, int n);
void yo_gdn_per_token_scan(float *state, const float *conv, const float *alpha, const float *beta,
                           float *out, int rows, int groups, int rank, int state_size, int conv_dim);
/* gdnChunkedScan (model/qwen35/recurrent.go:107-351): the chunkwise WY form, chunks of 32 rows */
void yo_gdn_chunked_scan(float *state, const float *conv, const float *alpha, const float *beta,
                         float *out, int rows, int groups, int rank, int S, int conv_dim);
void yo_gdn_norm_gate(float *out, const float *z, const float *norm, int rows, int rank,
                      int state_size, float eps);
void yo_select_experts(const float *logits, int n_experts, int32_t *ids, float *weights, int k);
float yo_sigmoid(float x);
float yo_silu(float x);
float yo_softplus(float x);

/* ---- model ---- */
yo_model *yo_model_create(const yo_config *cfg);
void yo_model_destroy(yo_model *m);
/* Tensor names follow the GGUF names read by model/qwen35/load.go:80-215.
 * Data is borrowed; the caller keeps it alive. rows/cols are the logical
 * matrix shape (vectors: rows = 1). Expert tensors pass rows = per-expert rows
 * times expert_count. */
int yo_model_set_tensor(yo_model *m, const char *name, int dtype, const void *data,
                        int64_t rows, int64_t cols);
int yo_model_check(const yo_model *m, char *msg, size_t msg_len);

/* ---- per-request state ---- */
/* table == NULL: blocks 0..n-1 in order, which is what a fresh allocator hands
 * out (memory/memory.go:65-67). */
yo_state *yo_state_create(const yo_model *m, int capacity, int kv_format, int pool_blocks,
                          int block_size, const int32_t *table, int table_len);
void yo_state_destroy(yo_state *s);
void yo_state_reset(yo_state *s);
int yo_state_pos(const yo_state *s);
int yo_state_set_pos(yo_state *s, int pos);
int64_t yo_state_snapshot_bytes(const yo_state *s);
int yo_state_snapshot(const yo_state *s, uint8_t *dst, int64_t len);
int yo_state_restore(yo_state *s, const uint8_t *src, int64_t len);
uint8_t *yo_state_kv(yo_state *s, int layer, int which /*0=K,1=V*/, int64_t *bytes);
float *yo_state_conv(yo_state *s, int layer, int64_t *count);
float *yo_state_s(yo_state *s, int layer, int64_t *count);
const float *yo_state_last_hidden(const yo_state *s);

/* ---- forward (model/qwen35/forward.go) ---- */
int yo_forward_one(const yo_model *m, yo_state *s, int32_t token, int want_logits);
const float *yo_logits(const yo_state *s);
int yo_forward(const yo_model *m, yo_state *s, const int32_t *tokens, int n, float *last_logits);
int yo_prefill_logits(const yo_model *m, yo_state *s, const int32_t *tokens, int n, float *out);

/* ---- speculative loop pieces (engine/speculative.go) ---- */
int32_t yo_argmax(const float *logits, int n);
int yo_lookup_draft(const int32_t *history, int n, int max_draft, int min_match, int32_t *out);
/* The reference's verify: logits holds the distribution after the last fed
 * token; k draft rows, greedy prefix match, restore + replay on a miss
 * (speculative.go:181-239). Updates logits to the next distribution. */
int yo_spec_verify_reference(const yo_model *m, yo_state *s, float *logits, const int32_t *draft,
                             int k, int32_t *accepted, int32_t *emitted, int32_t *n_emitted);
/* k+1-row formulation: rows = [pending, d1..dk]; emits d1..da and the
 * correction/bonus token, leaves the state committed through row a. If
 * all_logits != NULL it receives all (k+1) rows, rejected rows included. */
int yo_verify_chain(const yo_model *m, yo_state *s, int32_t pending, const int32_t *draft, int k,
                    int32_t *accepted, int32_t *emitted, float *all_logits);
/* Tree verification, greedy. tokens[0] is the pending token (root, parent -1);
 * parent[i] < i. Per-node logits are produced by running each root-to-node
 * path as a chain. path_out receives the accepted node ids (excluding root). */
int yo_verify_tree_greedy(const yo_model *m, yo_state *s, const int32_t *tokens,
                          const int32_t *parent, int n_nodes, int32_t *accepted,
                          int32_t *path_out, int32_t *emitted, float *all_logits);

/* ---- acceptance over given logits (no model), integer-exact ---- */
int yo_accept_greedy_tree(const float *logits, int vocab, const int32_t *tokens,
                          const int32_t *parent, int n_nodes, int32_t *accepted,
                          int32_t *path_out, int32_t *emitted);
float yo_exp_det(float x);
/* Rejection sampling on a tree; see oracle/ACCEPT_RULE in yuuka_oracle.c. */
int yo_accept_rejection_tree(const float *logits, const float *draft_probs, int vocab,
                             const int32_t *tokens, const int32_t *parent, int n_nodes,
                             float temperature, const float *uniforms,
                             int32_t *accepted, int32_t *path_out, int32_t *emitted);

#ifdef __cplusplus
}
#endif
#endif
