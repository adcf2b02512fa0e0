/* libyuuka_cuda: B200 (sm_100a) backend for yuuka's speculative-decoding
 * verify path. Plain C ABI for cgo; no C++ types, no PyTorch, no CPU fallback.
 *
 * Conventions follow the reference's HIP bridge (backend/hip/bridge/yuuka_hip.h):
 * opaque handles owned by the caller and freed exactly once, every call
 * returns a yuuka_status, yuuka_last_error() is thread-local, no exception
 * crosses the boundary, host transfers are synchronous with respect to the
 * host buffer, asynchronous work touches device buffers only.
 *
 * Each declaration cites the reference interface it replaces or extends.
 */
#ifndef YUUKA_CUDA_H
#define YUUKA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YUUKA_CUDA_ABI_VERSION 1

#if defined(__GNUC__)
#define YUUKA_API __attribute__((visibility("default")))
#else
#define YUUKA_API
#endif

/* yuuka_hip.h:21-35 */
typedef struct yuuka_device yuuka_device;
typedef struct yuuka_buffer yuuka_buffer;
typedef struct yuuka_stream yuuka_stream;
typedef struct yuuka_event yuuka_event;

typedef enum yuuka_status {
    YUUKA_OK = 0,
    YUUKA_ERR_INVALID_ARGUMENT = 1,
    YUUKA_ERR_UNSUPPORTED = 2,
    YUUKA_ERR_DEVICE = 3,
    YUUKA_ERR_ALLOCATION = 4,
    YUUKA_ERR_INTERNAL = 5
} yuuka_status;

/* yuuka_hip.h:37-47 (gcn_arch/hip_version become sm arch / CUDA version) */
typedef struct yuuka_device_info {
    char name[256];
    char arch[64];
    char cuda_version[64];
    uint64_t total_memory;
    uint32_t multiprocessors;
    uint32_t clock_mhz;
    uint32_t l2_bytes;
    uint32_t smem_per_block_optin;
    int32_t pci_domain;
    int32_t pci_bus;
    int32_t pci_device;
} yuuka_device_info;

/* GGML dtype ids, as yuuka_hip.h:198-207. BF16 (GGML id 30) is accepted for
 * activations of the kernel-level GEMM only. */
typedef enum yuuka_dtype {
    YUUKA_DTYPE_F32 = 0,
    YUUKA_DTYPE_F16 = 1,
    YUUKA_DTYPE_Q8_0 = 8,
    YUUKA_DTYPE_Q4_K = 12,
    YUUKA_DTYPE_Q5_K = 13,
    YUUKA_DTYPE_Q6_K = 14,
    YUUKA_DTYPE_BF16 = 30
} yuuka_dtype;

/* KV pool formats: model/qwen35/kv_format.go:16-24 */
typedef enum yuuka_kv_format { YUUKA_KV_F32 = 0, YUUKA_KV_F16 = 1, YUUKA_KV_Q8_0 = 2 } yuuka_kv_format;

/* yuuka_hip.h:49-53 */
YUUKA_API uint32_t yuuka_abi_version(void);
YUUKA_API const char * yuuka_last_error(void);

/* yuuka_hip.h:55-58 */
YUUKA_API yuuka_status yuuka_device_open(int32_t index, yuuka_device ** out);
YUUKA_API void yuuka_device_close(yuuka_device * dev);
YUUKA_API yuuka_status yuuka_device_info_get(const yuuka_device * dev, yuuka_device_info * info);

/* yuuka_hip.h:60-64 */
/* Free and total bytes of device memory right now (cudaMemGetInfo): lets a host that
 * sizes its pools from what is left, or a test, see what a call allocated. */
YUUKA_API yuuka_status yuuka_device_memory_get(const yuuka_device * dev, uint64_t * free_bytes, uint64_t * total_bytes);

YUUKA_API yuuka_status yuuka_buffer_alloc(yuuka_device * dev, uint64_t bytes, yuuka_buffer ** out);
YUUKA_API void yuuka_buffer_free(yuuka_buffer * buf);
YUUKA_API uint64_t yuuka_buffer_size(const yuuka_buffer * buf);
YUUKA_API void * yuuka_buffer_ptr(const yuuka_buffer * buf);

/* yuuka_hip.h:66-72. Events here can also be recorded explicitly and timed,
 * which the reference does inside yuuka_plan_execute_profiled (:491-496). */
YUUKA_API yuuka_status yuuka_stream_create(yuuka_device * dev, yuuka_stream ** out);
YUUKA_API void yuuka_stream_destroy(yuuka_stream * stream);
YUUKA_API yuuka_status yuuka_stream_synchronize(yuuka_stream * stream);
YUUKA_API yuuka_status yuuka_event_create(yuuka_device * dev, yuuka_event ** out);
YUUKA_API void yuuka_event_destroy(yuuka_event * event);
YUUKA_API yuuka_status yuuka_event_record(yuuka_stream * stream, yuuka_event * event);
YUUKA_API yuuka_status yuuka_event_wait(yuuka_event * event);
YUUKA_API yuuka_status yuuka_event_elapsed_ms(yuuka_event * start, yuuka_event * end, float * ms);

/* yuuka_hip.h:74-79 (+ an offset form for uploads) */
YUUKA_API yuuka_status yuuka_memcpy_h2d(yuuka_buffer * dst, const void * src, uint64_t bytes);
YUUKA_API yuuka_status yuuka_memcpy_h2d_at(yuuka_buffer * dst, uint64_t offset, const void * src, uint64_t bytes);
YUUKA_API yuuka_status yuuka_memcpy_d2h(void * dst, const yuuka_buffer * src, uint64_t bytes);
YUUKA_API yuuka_status yuuka_memcpy_d2h_at(void * dst, const yuuka_buffer * src, uint64_t offset, uint64_t bytes);
YUUKA_API yuuka_status yuuka_memset(yuuka_stream * stream, yuuka_buffer * dst, int value, uint64_t bytes);
/* yuuka_hip.h:81-86 */
YUUKA_API yuuka_status yuuka_buffer_copy(yuuka_stream * stream, yuuka_buffer * dst, uint64_t dst_offset,
                                         const yuuka_buffer * src, uint64_t src_offset, uint64_t bytes,
                                         yuuka_event * completion);

/* ------------------------------------------------------------------------
 * Kernel-level entry points (what yuuka_gemv_batch / yuuka_gemm_wmma and the
 * LM_HEAD, ATTENTION_PREFILL_PAGED and RECURRENT_CHUNK plan ops are in the
 * reference: yuuka_hip.h:209-300,340-440). All are asynchronous on stream.
 * ---------------------------------------------------------------------- */

/* GEMM route. AUTO: tile-ordered weights go to the tensor-core kernels whatever the row count (the register-fed
 * exact route up to 47 rows per launch, the tensor-memory route from 48), GGUF-ordered weights to the fp32
 * kernel; the others force one kernel family. */
#define YUUKA_GEMM_PATH_AUTO 0u
#define YUUKA_GEMM_PATH_FP32 1u /* CUDA-core dot products, the reference's fp32 decode arithmetic */
#define YUUKA_GEMM_PATH_MMA 2u  /* tensor-core MMA on fp16 operands, fp32 accumulate */

/* out[rows, n_out] (f32) = x[rows, n_in] * W[n_out, n_in]^T, W in the packed
 * GGUF row layout of w_dtype (replaces yuuka_gemv_batch, yuuka_hip.h:291-300,
 * and YUUKA_OP_LM_HEAD). x_dtype is F32 or BF16. Byte offsets select
 * sub-ranges of the buffers. flags: bit 0 adds the product to out instead of
 * overwriting it (GEMV_RESIDUAL, yuuka_hip.h:398-401).
 * The call keeps one scratch area per device (prepared activations, split-K
 * partial sums and arrival counters) that it grows with cudaMalloc when a larger
 * shape arrives. Host threads may call concurrently (the growth is serialized), but
 * kernels of two calls that can overlap on one device (different streams) share
 * that area and race on it: keep the calls of a device on one stream or order them
 * with events. Growing the area frees the old one, so a larger shape must not
 * arrive while an earlier call's kernels may still run on another stream. */
#define YUUKA_GEMM_ACCUMULATE 0x1u
/* bit 1: w holds the tile-ordered copy made by yuuka_weights_tile (required by
 * the mma route and by the fast fp32 route; GGUF-layout weights take a slower
 * generic kernel). */
#define YUUKA_GEMM_TILED 0x2u
/* bit 31, test hook: the register-fed kernel never issues the copies of its activations and its wait for them
 * gives up after a short limit, so that the expiry path (device error word, YUUKA_ERR_DEVICE at the next
 * session fetch) can be exercised with nothing in flight. The outputs of such a launch are garbage. */
#define YUUKA_GEMM_TEST_DROP_COPIES 0x80000000u
YUUKA_API yuuka_status yuuka_gemm_quant(yuuka_stream * stream,
                                        yuuka_buffer * out, uint64_t out_offset,
                                        const yuuka_buffer * x, uint64_t x_offset, uint32_t x_dtype,
                                        const yuuka_buffer * w, uint64_t w_offset, uint32_t w_dtype,
                                        uint64_t n_in, uint64_t n_out, uint64_t rows,
                                        uint32_t path, uint32_t flags, yuuka_event * completion);

/* The tiled GEMM above with its scratch memory in a fixed device array of this
 * library instead of the per-device scratch that yuuka_gemm_quant grows with
 * cudaMalloc when a larger shape arrives. No counterpart in the reference. It is
 * for hosts that may not cause a device allocation once serving has started:
 * an engine that hands all free HBM to its weight and KV pools at start-up
 * (a later cudaMalloc can fail there, and it stalls every stream of the device
 * while it runs), or a real-time loop that must not take the allocator's lock.
 * This call allocates and frees nothing, on the device or through a library.
 *  - Same arguments, routes and bit-identical results as yuuka_gemm_quant with
 *    YUUKA_GEMM_TILED, which flags must carry.
 *  - The scratch holds the prepared fp16 activations (rows * n_in * 2.25 bytes),
 *    the split-K partial sums and 4096 arrival counters. A shape that needs more
 *    than YUUKA_GEMM_STATIC_SCRATCH_BYTES returns YUUKA_ERR_UNSUPPORTED and
 *    launches nothing; yuuka_last_error() names the bytes needed.
 *  - The first call on each device does the set-up (it looks up the array's
 *    device address, zeroes the counters, has the driver load the code of
 *    every kernel this entry point can launch, whatever the shape, so that no
 *    later call makes the driver place code in device memory, and synchronizes
 *    the device): make that call before any stream capture begins. Later calls
 *    only launch; yuuka_device_memory_get reports the same free bytes before
 *    and after them.
 *  - One scratch per device: two calls whose kernels can overlap (different
 *    streams, or two host threads) race on it. Keep calls on one stream, or
 *    order them with events. */
#define YUUKA_GEMM_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
YUUKA_API yuuka_status yuuka_gemm_quant_static(yuuka_stream * stream,
                                               yuuka_buffer * out, uint64_t out_offset,
                                               const yuuka_buffer * x, uint64_t x_offset, uint32_t x_dtype,
                                               const yuuka_buffer * w, uint64_t w_offset, uint32_t w_dtype,
                                               uint64_t n_in, uint64_t n_out, uint64_t rows,
                                               uint32_t path, uint32_t flags, yuuka_event * completion);

/* Tile-ordered weight copy: a byte permutation of a K-quant / Q8_0 GGUF matrix
 * into 16-row x 256-column records laid out in the order a warp consumes them
 * (the reference uploads GGUF bytes verbatim, engine/gpu/model.go:288-301; its
 * docs list an offline re-layout as future work). Dequantized values are
 * bit-identical. yuuka_weights_tiled_bytes returns 0 for dtypes / widths
 * without a tiled form. */
YUUKA_API uint64_t yuuka_weights_tiled_bytes(uint32_t dtype, uint64_t n_out, uint64_t n_in);
YUUKA_API yuuka_status yuuka_weights_tile(yuuka_stream * stream, yuuka_buffer * dst, uint64_t dst_offset,
                                          const yuuka_buffer * src, uint64_t src_offset, uint32_t dtype,
                                          uint64_t n_out, uint64_t n_in, yuuka_event * completion);

/* ------------------------------------------------------------------------
 * Model and verify session (what engine/gpu's Model/Session/plan builders do
 * in Go through yuuka_plan_*; here the plan lives behind the ABI so that one
 * call runs the whole verify step).
 * ---------------------------------------------------------------------- */

typedef struct yuuka_model yuuka_model;
typedef struct yuuka_session yuuka_session;

/* model/qwen35/config.go:18-44 */
typedef struct yuuka_model_config {
    int32_t block_count, context_length, hidden, ffn;
    int32_t heads, kv_heads, head_dim, rope_dim;
    double rope_freq_base;
    float rms_eps;
    int32_t vocab;
    int32_t conv_kernel, state_size, group_count, time_step_rank, inner_size;
    int32_t full_attention_interval;
    int32_t expert_count, expert_used, expert_ffn, shared_ffn;
} yuuka_model_config;

/* Validates cfg with the rules of model/qwen35/config.go:231-276. */
YUUKA_API yuuka_status yuuka_model_create(yuuka_device * dev, const yuuka_model_config * cfg, yuuka_model ** out);
YUUKA_API void yuuka_model_destroy(yuuka_model * model);
/* Uploads one GGUF tensor verbatim (engine/gpu/model.go:288-301). name is the
 * GGUF tensor name read by model/qwen35/load.go:80-215; rows/cols the logical
 * shape (vectors: rows = 1; expert tensors: rows = per-expert rows * experts). */
YUUKA_API yuuka_status yuuka_model_set_tensor(yuuka_model * model, const char * name, uint32_t dtype,
                                              const void * data, uint64_t rows, uint64_t cols);
/* Checks that every required tensor is present with the right shape. */
YUUKA_API yuuka_status yuuka_model_finalize(yuuka_model * model);
YUUKA_API uint64_t yuuka_model_weight_bytes(const yuuka_model * model);

/* ---- GGUF files (gguf/reader.go, gguf/metadata.go) ----
 * A reader maps the file (and the other shards of a split model, named
 * name-NNNNN-of-NNNNN.gguf) read-only and validates magic, version 2..3,
 * metadata, the tensor directory, general.alignment, offsets, byte ranges and
 * overlaps before anything is exposed (reader.go:248-393, 547-704). Malformed
 * files give YUUKA_ERR_INVALID_ARGUMENT, unknown versions and tensor types
 * YUUKA_ERR_UNSUPPORTED; the message names file and field. Pointers handed out
 * stay valid until yuuka_gguf_close. */
typedef struct yuuka_gguf yuuka_gguf;
typedef struct yuuka_gguf_tensor {
    const char * name;
    uint32_t dtype;      /* GGML type id, the same numbers as yuuka_dtype */
    uint32_t rank;
    uint64_t dims[8];    /* GGML order: dims[0] is the contiguous row width (Tensor.Columns, reader.go:62-67) */
    uint64_t bytes;
    const void * data;   /* read-only mapping (Tensor.Data, reader.go:89-100) */
} yuuka_gguf_tensor;
YUUKA_API yuuka_status yuuka_gguf_open(const char * path, yuuka_gguf ** out);
YUUKA_API void yuuka_gguf_close(yuuka_gguf * g);
YUUKA_API uint32_t yuuka_gguf_version(const yuuka_gguf * g);
YUUKA_API uint64_t yuuka_gguf_alignment(const yuuka_gguf * g);
YUUKA_API uint64_t yuuka_gguf_tensor_count(const yuuka_gguf * g);
YUUKA_API uint64_t yuuka_gguf_metadata_count(const yuuka_gguf * g);
/* Tensors in directory order, shard after shard (Reader.Tensors), or by name (Reader.Tensor). */
YUUKA_API yuuka_status yuuka_gguf_tensor_at(const yuuka_gguf * g, uint64_t index, yuuka_gguf_tensor * out);
YUUKA_API yuuka_status yuuka_gguf_tensor_find(const yuuka_gguf * g, const char * name, yuuka_gguf_tensor * out);
/* Reader.Int / Float / String (reader.go:741-782) with the conversions of Value.AsInt / AsFloat /
 * AsString (metadata.go:87-128); a missing key or a value of another kind is YUUKA_ERR_INVALID_ARGUMENT. */
YUUKA_API yuuka_status yuuka_gguf_meta_int(const yuuka_gguf * g, const char * key, int64_t * out);
YUUKA_API yuuka_status yuuka_gguf_meta_float(const yuuka_gguf * g, const char * key, double * out);
YUUKA_API yuuka_status yuuka_gguf_meta_string(const yuuka_gguf * g, const char * key, const char ** out, uint64_t * len);
YUUKA_API yuuka_status yuuka_gguf_meta_array_len(const yuuka_gguf * g, const char * key, uint64_t * out);
/* LoadConfig (model/qwen35/config.go:48-174): general.architecture qwen35 or qwen35moe, the
 * <arch>.* hyperparameters, vocabulary size from tokenizer.ggml.tokens or <arch>.vocab_size. */
YUUKA_API yuuka_status yuuka_gguf_model_config(const yuuka_gguf * g, yuuka_model_config * out);
/* Opens the file, creates the model from its metadata, uploads every tensor verbatim and finalizes
 * (engine/gpu/model.go:288-301 over model/qwen35/load.go:80-215). */
YUUKA_API yuuka_status yuuka_model_load_gguf(yuuka_device * dev, const char * path, yuuka_model ** out);

/* A session owns a paged KV pool, per-sequence block tables, positions and
 * recurrent state for max_batch sequences (engine/gpu/session.go:58-182 holds
 * one; serving needs many), plus the activations of one verify step of up to
 * max_nodes rows per sequence. */
typedef struct yuuka_session_config {
    int32_t max_batch;     /* sequences */
    int32_t max_nodes;     /* rows per sequence per step, pending token included (<= 64) */
    int32_t capacity;      /* positions per sequence, <= context_length */
    int32_t block_size;    /* tokens per KV block; 0 = 16 (model/qwen35/state.go:68) */
    int32_t pool_blocks;   /* 0 = max_batch * ceil(capacity / block_size) */
    int32_t kv_format;     /* yuuka_kv_format */
    int32_t want_logits;   /* keep f32 logits [max_batch*max_nodes, vocab] for download */
    uint32_t flags;        /* YUUKA_SESSION_* */
} yuuka_session_config;
/* Steps and prompt passes of 48 rows or more normally take the tensor-memory GEMM route, which rounds
 * the decoded weights and the activations to fp16 (about 1e-3 relative per product; logits of a deep
 * model then sit around 1e-2 of the fp32 CPU path, and a qwen35moe router may pick another expert at a
 * near-tie). With this flag such passes run as 16-row passes of the register-fed route instead, which
 * multiplies exact integer weights with two-half activations (fp32-level results, weights streamed once
 * per 16 rows). */
#define YUUKA_SESSION_EXACT_WIDE 0x1u
/* The other way round: steps of 33..47 rows, which by default run as three exact 16-row passes, also take the
 * tensor-memory route (one pass over the weights: a 36-row step of the 4B model 8.1 -> 4.7 ms) at that route's
 * fp16-rounded precision. For hosts that batch a handful of sequences per step and prefer the speed. */
#define YUUKA_SESSION_WIDE_FROM_33 0x2u
/* Test hook: every GEMM of the session's steps carries YUUKA_GEMM_TEST_DROP_COPIES. */
#define YUUKA_SESSION_TEST_DROP_COPIES 0x80000000u
/* Replaces the session's flags between steps (no step may be staged or in flight; captured steps are dropped,
 * since the flags select kernels). */
YUUKA_API yuuka_status yuuka_session_set_flags(yuuka_session * s, uint32_t flags);

YUUKA_API yuuka_status yuuka_session_create(yuuka_model * model, const yuuka_session_config * cfg,
                                            yuuka_session ** out);
YUUKA_API void yuuka_session_destroy(yuuka_session * s);
/* Block table of one sequence: int32 block ids, as memory.Table.Blocks()
 * returns them (memory/memory.go:199). Ids must be < pool_blocks. The default
 * is the identity mapping over the sequence's own slice of the pool. */
YUUKA_API yuuka_status yuuka_session_set_block_table(yuuka_session * s, int32_t seq, const int32_t * blocks,
                                                     int32_t count);
/* KVPool.CopyBlock (model/qwen35/kv_pool.go:156-170; engine/gpu/model.go:600-626): copies block src of the
 * K and V pool of every attention layer onto block dst, device to device on the session stream and
 * synchronously. The prefix cache uses it to give a request a private copy of a shared, partly filled
 * block before the request appends to it. */
YUUKA_API yuuka_status yuuka_session_copy_block(yuuka_session * s, int32_t dst_block, int32_t src_block);
/* State.Reset / State.SetPos (model/qwen35/state.go:174-208). Reset, set_position and restore are refused with
 * YUUKA_ERR_INVALID_ARGUMENT between yuuka_verify_launch and yuuka_verify_fetch: the fetch adds what the step
 * accepted to the positions these calls would replace. */
YUUKA_API yuuka_status yuuka_session_reset(yuuka_session * s, int32_t seq);
YUUKA_API yuuka_status yuuka_session_set_position(yuuka_session * s, int32_t seq, int32_t position);
YUUKA_API yuuka_status yuuka_session_position(yuuka_session * s, int32_t seq, int32_t * position);
/* State.Snapshot / Restore byte format (model/qwen35/state.go:211-263): for each
 * recurrent layer in order, conv then s, little-endian f32. */
YUUKA_API uint64_t yuuka_session_snapshot_bytes(const yuuka_session * s);
YUUKA_API yuuka_status yuuka_session_snapshot(yuuka_session * s, int32_t seq, void * dst, uint64_t bytes);
YUUKA_API yuuka_status yuuka_session_restore(yuuka_session * s, int32_t seq, const void * src, uint64_t bytes);

/* engine.SpeculativeRuntime.PrefillLogits (engine/engine.go:55-63;
 * engine/gpu/session.go:246-303): runs n tokens of sequence seq as a chain,
 * commits all of them, and (logits != NULL) returns f32 logits [n, vocab].
 * n may exceed max_nodes; it is processed in chunks. Synchronous. */
YUUKA_API yuuka_status yuuka_session_prefill_logits(yuuka_session * s, int32_t seq, const int32_t * tokens,
                                                    int32_t n, float * logits);
/* Runtime.Forward (engine/engine.go:67-74): as above but only the last row's
 * logits are computed and returned (last_logits may be NULL). */
YUUKA_API yuuka_status yuuka_session_forward(yuuka_session * s, int32_t seq, const int32_t * tokens, int32_t n,
                                             float * last_logits);

/* Acceptance modes of a verify step. */
#define YUUKA_ACCEPT_GREEDY 0u    /* engine/speculative.go:193-202 with argmaxLogit :263-271 */
#define YUUKA_ACCEPT_REJECTION 1u /* not in the reference; the rule is stated above rejection_walk_kernel (accept.cu) */
#define YUUKA_ACCEPT_NONE 2u      /* run and commit nothing: logits only */

/* One verify step over `batch` sequences (seq ids 0..batch-1 of the session).
 * Per sequence, `nodes` rows: row 0 is the pending token (the last emitted
 * token that has not been run), rows 1.. are draft tokens; parent[b][i] is the
 * row that precedes row i (-1 for row 0, < i otherwise; a chain is i-1).
 * All pointers are HOST memory; the call uploads them, runs the step, performs
 * acceptance and the KV / recurrent-state commit on the device, downloads the
 * results and returns when they are in the output arrays.
 *   accepted[b]        number of accepted draft rows a
 *   emitted[b][0..a]   a accepted draft tokens followed by the correction or
 *                      bonus token (which is the next pending token)
 *   path[b][0..a-1]    accepted row ids (may be NULL)
 * For rejection sampling draft_probs is f32 [batch, nodes, vocab] (row i holds
 * the distribution token i was drawn from; row 0 unused), uniforms f32
 * [batch, nodes, 2]. */
typedef struct yuuka_verify_batch {
    int32_t batch;
    int32_t nodes;
    const int32_t * tokens;      /* [batch, nodes] */
    const int32_t * parent;      /* [batch, nodes]; NULL = chain */
    uint32_t mode;
    float temperature;
    const yuuka_buffer * draft_probs; /* device buffer, rejection mode only */
    const float * uniforms;      /* host, rejection mode only */
    int32_t * accepted;          /* [batch] */
    int32_t * emitted;           /* [batch, nodes] */
    int32_t * path;              /* [batch, nodes] or NULL */
    float * logits;              /* optional host [batch, nodes, vocab]; needs want_logits */
    /* [batch] or NULL: the session sequence behind each slot of the batch, distinct values in
     * 0..max_batch-1; NULL means slot b is sequence b. A scheduler iteration verifies whichever of
     * its runs are ready (scheduler/scheduler.go:590-623 walks them one DecodeOnce at a time): it
     * lists their sequences here instead of moving state between slots. */
    const int32_t * seq_ids;
} yuuka_verify_batch;

YUUKA_API yuuka_status yuuka_verify_step(yuuka_session * s, const yuuka_verify_batch * batch);

/* The acceptance stage on its own, over f32 logits [batch, nodes, vocab] that are already on the device: the
 * greedy walk (argmaxLogit first-maximum rule, engine/speculative.go:263-271, along the tree) or the rejection-
 * sampling walk, with the arguments' meaning as in yuuka_verify_batch (tokens, parent, uniforms on the host;
 * draft_probs on the device). Row metadata and scratch are allocated for the call. begin / end (optional) are
 * recorded around the acceptance kernels. Synchronous. */
YUUKA_API yuuka_status yuuka_accept_tree(yuuka_stream * stream, const yuuka_buffer * logits, int32_t batch, int32_t nodes,
                                         int32_t vocab, const int32_t * tokens, const int32_t * parent, uint32_t mode,
                                         float temperature, const yuuka_buffer * draft_probs, const float * uniforms,
                                         int32_t * accepted, int32_t * emitted, int32_t * path, yuuka_event * begin,
                                         yuuka_event * end);

/* Device-resident variant for benchmarking and pipelined serving: inputs were
 * staged with yuuka_verify_stage, the step only enqueues kernels on the
 * session stream (no host synchronisation); results are fetched later. */
YUUKA_API yuuka_status yuuka_verify_stage(yuuka_session * s, const yuuka_verify_batch * batch);
YUUKA_API yuuka_status yuuka_verify_launch(yuuka_session * s, yuuka_event * completion);
YUUKA_API yuuka_status yuuka_verify_fetch(yuuka_session * s, const yuuka_verify_batch * batch);

/* Diagnostic launch: as yuuka_verify_launch, with an event pair around every
 * operation and one synchronisation at the end; returns per-op codes and
 * elapsed nanoseconds (yuuka_plan_execute_profiled, yuuka_hip.h:491-496). The
 * step still has to be fetched. Not for the hot path. */
typedef enum yuuka_op_code {
    YUUKA_OP_GEMM = 16,          /* numbering follows yuuka_hip.h:104-149 where an op exists there */
    YUUKA_OP_RMSNORM = 18,
    YUUKA_OP_ATTN_PREP = 20,
    YUUKA_OP_RECURRENT_CHUNK = 23,
    YUUKA_OP_EMBEDDING = 24,
    YUUKA_OP_ATTENTION = 29,
    YUUKA_OP_LM_HEAD = 37,
    YUUKA_OP_SILU_MUL = 9,
    YUUKA_OP_GDN_SCAN = 100,    /* conv + norms, recurrence, gated norm (101 was the gated norm on its own) */
    YUUKA_OP_ACCEPT = 102,
    YUUKA_OP_COMMIT = 103,
    YUUKA_OP_MOE_ROUTE = 104,   /* router logits, top-k, grouping of (row, slot) pairs by expert */
    YUUKA_OP_MOE_EXPERTS = 105, /* grouped expert gate|up GEMM, SwiGLU, grouped down GEMM */
    YUUKA_OP_MOE_COMBINE = 106
} yuuka_op_code;
YUUKA_API yuuka_status yuuka_verify_launch_profiled(yuuka_session * s, uint32_t * op_codes, uint64_t * op_times_ns,
                                                    uint64_t capacity, uint64_t * op_count);
YUUKA_API yuuka_stream * yuuka_session_stream(yuuka_session * s);
/* Kernel launches enqueued by the last yuuka_verify_launch. */
YUUKA_API uint32_t yuuka_session_last_launch_count(const yuuka_session * s);

/* ------------------------------------------------------------------------
 * Host-side block allocator and block-table helpers (memory.Allocator and
 * memory.Table, memory/memory.go:34-266). The free list is LIFO and starts
 * descending, so a fresh allocator hands out block 0 first. No evictor hook:
 * an exhausted pool answers YUUKA_ERR_ALLOCATION (ErrOutOfBlocks).
 * ---------------------------------------------------------------------- */
typedef struct yuuka_allocator yuuka_allocator;
typedef struct yuuka_allocator_stats {
    int32_t block_size, total, used, free, shared;
    uint64_t allocated, released;
} yuuka_allocator_stats;
YUUKA_API yuuka_status yuuka_allocator_create(int32_t blocks, int32_t block_size, yuuka_allocator ** out);
YUUKA_API void yuuka_allocator_destroy(yuuka_allocator * a);
YUUKA_API yuuka_status yuuka_allocator_acquire(yuuka_allocator * a, int32_t * id);
YUUKA_API yuuka_status yuuka_allocator_retain(yuuka_allocator * a, int32_t id);
YUUKA_API yuuka_status yuuka_allocator_release(yuuka_allocator * a, int32_t id);
YUUKA_API int32_t yuuka_allocator_refs(yuuka_allocator * a, int32_t id);
YUUKA_API yuuka_status yuuka_allocator_stats_get(yuuka_allocator * a, yuuka_allocator_stats * out);
/* Table.Cover: grows blocks[0 .. *count) (room for `capacity` ids) until `positions` token positions are
 * mapped; all or nothing. Table.Map: position -> (block id, offset in block). */
YUUKA_API yuuka_status yuuka_table_cover(yuuka_allocator * a, int32_t * blocks, int32_t * count, int32_t capacity,
                                         int32_t positions);
YUUKA_API yuuka_status yuuka_table_map(const int32_t * blocks, int32_t count, int32_t block_size, int32_t pos,
                                       int32_t * block, int32_t * offset);

/* Geometry of a session, for callers that drive it generically. */
typedef struct yuuka_session_info {
    int32_t max_batch, max_nodes, capacity, block_size, pool_blocks, kv_format;
    int32_t vocab;
} yuuka_session_info;
YUUKA_API yuuka_status yuuka_session_info_get(const yuuka_session * s, yuuka_session_info * out);

/* ------------------------------------------------------------------------
 * Exact greedy speculative decoding with prompt-lookup drafts: the host loop
 * of engine/speculative.go over the verify step above.
 * ---------------------------------------------------------------------- */

/* engine/speculative.go:13-19 */
typedef struct yuuka_spec_options {
    int32_t max_draft; /* <= 0: 4; capped at 16 */
    int32_t min_match; /* <= 0: 2; capped at 8 */
} yuuka_spec_options;
/* SpeculativeOptions.normalize, engine/speculative.go:21-34 */
YUUKA_API void yuuka_spec_options_normalize(yuuka_spec_options * options);
/* lookupDraft, engine/speculative.go:39-66. out must hold max_draft ids; returns
 * the number of draft tokens (0: none). */
YUUKA_API int32_t yuuka_spec_lookup_draft(const int32_t * history, int32_t n, int32_t max_draft, int32_t min_match,
                                          int32_t * out);

#define YUUKA_FINISH_LENGTH 0 /* "length" */
#define YUUKA_FINISH_STOP 1   /* "stop" */
typedef struct yuuka_spec_request {
    int32_t max_tokens;          /* GenerateOptions.MaxTokens; clipped to the free context */
    yuuka_spec_options options;
    const int32_t * stop_tokens; /* StopTokens plus the EOS id if it applies; may be NULL with n_stop 0 */
    int32_t n_stop;
} yuuka_spec_request;
/* The counters of engine.GenerateResult that the loop maintains (engine/speculative.go:186-203). */
typedef struct yuuka_spec_result {
    int32_t prompt_tokens, output_tokens, finish_reason;
    int32_t steps;          /* verify steps run */
    int32_t draft_tokens;   /* DraftTokens */
    int32_t accepted_draft; /* AcceptedDraft */
} yuuka_spec_result;
/* generateSpeculative, engine/speculative.go:68-251, for sequence seq of the
 * session: resets it, runs the prompt, then verify steps of [pending token,
 * prompt-lookup drafts] until max_tokens, a stop token (not emitted) or the
 * context capacity. tokens must hold max_tokens ids. The emitted stream equals
 * plain greedy decoding. The session needs max_nodes >= 2 to draft at all
 * (drafts per step are capped at max_nodes - 1). Synchronous. */
YUUKA_API yuuka_status yuuka_spec_generate(yuuka_session * s, int32_t seq, const int32_t * prompt, int32_t n_prompt,
                                           const yuuka_spec_request * request, int32_t * tokens,
                                           yuuka_spec_result * result);
/* lookupDraft on the device (history: int32 ids in a device buffer): out receives the draft length and then the
 * draft ids, int32[1 + max_draft]. Same result as yuuka_spec_lookup_draft, id for id. Synchronous. */
YUUKA_API yuuka_status yuuka_spec_lookup_draft_device(yuuka_stream * stream, const yuuka_buffer * history, int32_t n,
                                                      int32_t max_draft, int32_t min_match, yuuka_buffer * out);
/* yuuka_spec_generate with the drafting done by a kernel between the steps (the step before verify in the
 * loop, engine/speculative.go:161): every step has max_draft + 1 rows, the history stays on the device, and
 * `burst` (1..64) steps are enqueued per host synchronization. The emitted stream is the same greedy stream.
 * Stop tokens and max_tokens are applied when a burst returns, so the sequence may have run up to one burst
 * past the last returned token; result->steps counts the steps that ran. */
YUUKA_API yuuka_status yuuka_spec_generate_device(yuuka_session * s, int32_t seq, const int32_t * prompt, int32_t n_prompt,
                                                  const yuuka_spec_request * req, int32_t burst, int32_t * tokens,
                                                  yuuka_spec_result * result);

#ifdef __cplusplus
}
#endif
#endif
