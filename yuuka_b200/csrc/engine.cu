// Model, session and the verify step: the host-side plan that the reference
// builds in Go (engine/gpu/model.go, session.go, plan.go buildPrefillPlan with
// prefillAllLogits) lives here behind the C ABI, so one call runs a whole
// verify step: k+1 (or tree) rows through every layer, on-device acceptance,
// KV / recurrent-state commit.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "gemm_quant.cuh"
#include "gemm_tiled.cuh"
#include "layers.cuh"

using namespace yk;

namespace {

struct Tensor {
    uint8_t * ptr = nullptr;
    uint32_t dtype = 0;
    uint64_t rows = 0, cols = 0, bytes = 0;
    bool owned = false;
    bool tiled = false;  // ptr holds the tile-ordered copy (gemm_tiled.cuh)
    bool paired = false; // two matrices of equal shape interleaved 16 rows by 16 rows (ffn_gate | ffn_up)
    bool present() const { return ptr != nullptr; }
};

struct LayerW {
    const float * attn_norm = nullptr;
    const float * post_norm = nullptr;
    // full attention
    Tensor q, k, v, o;
    const float * q_norm = nullptr;
    const float * k_norm = nullptr;
    // gated delta-net
    Tensor qkv, gate, beta, alpha, out;
    const float * conv = nullptr;
    const float * dt = nullptr;
    const float * a = nullptr;
    const float * ssm_norm = nullptr;
    // dense FFN
    Tensor ffn_gate, ffn_up, ffn_down;
    // fused row ranges (same dtype, adjacent in memory): one GEMM each
    Tensor proj;     // qkv | gate | beta | alpha
    Tensor qk;       // q | k (| v)
    bool qk_has_v = false;
    Tensor gate_up;  // ffn_gate | ffn_up
    // qwen35moe block (model/qwen35/load.go:171-215)
    const float * router = nullptr;       // ffn_gate_inp [experts][hidden] f32
    const float * sh_gate_inp = nullptr;  // ffn_gate_inp_shexp [hidden] f32
    Tensor sh_gate, sh_up, sh_down, sh_gate_up;
    Tensor exp_gate_up;  // per expert: gate rows then up rows, each expert tiled on its own
    Tensor exp_down;     // per expert [hidden][expert_ffn], each expert tiled on its own
    size_t exp_gate_up_stride = 0, exp_down_stride = 0;
};

void free_tensor(Tensor & t) {
    if (t.owned && t.ptr) cudaFree(t.ptr);
    t = Tensor();
}

}  // namespace

struct yuuka_model {
    yuuka_device * dev = nullptr;
    yuuka_model_config cfg{};
    std::map<std::string, Tensor> tensors;
    std::vector<LayerW> layers;
    Tensor embedding, output;
    const float * output_norm = nullptr;
    std::vector<void *> extra_allocs;
    bool finalized = false;
    uint64_t weight_bytes = 0;

    int conv_dim() const { return 2 * cfg.group_count * cfg.state_size + cfg.inner_size; }
    int q_dim() const { return cfg.heads * cfg.head_dim * 2; }
    int kv_dim() const { return cfg.kv_heads * cfg.head_dim; }
    int o_dim() const { return cfg.heads * cfg.head_dim; }
    bool recurrent(int layer) const { return (layer + 1) % cfg.full_attention_interval != 0; }
};

namespace {

// model/qwen35/config.go:231-276
void validate_config(const yuuka_model_config & c) {
    YK_REQUIRE(c.block_count > 0 && c.hidden > 0 && c.head_dim > 0 && c.heads > 0, YUUKA_ERR_INVALID_ARGUMENT,
               "invalid model size");
    YK_REQUIRE(c.kv_heads > 0 && c.heads % c.kv_heads == 0, YUUKA_ERR_INVALID_ARGUMENT,
               "head count %d is not a multiple of KV head count %d", c.heads, c.kv_heads);
    YK_REQUIRE(c.rope_dim % 2 == 0 && c.rope_dim <= c.head_dim && c.rope_dim >= 0, YUUKA_ERR_INVALID_ARGUMENT,
               "invalid RoPE dimension %d for head dim %d", c.rope_dim, c.head_dim);
    YK_REQUIRE(c.full_attention_interval > 0, YUUKA_ERR_INVALID_ARGUMENT, "full attention interval must be positive");
    YK_REQUIRE(c.inner_size == c.time_step_rank * c.state_size, YUUKA_ERR_INVALID_ARGUMENT,
               "ssm inner size %d != time_step_rank %d * state_size %d", c.inner_size, c.time_step_rank, c.state_size);
    YK_REQUIRE(c.conv_kernel >= 2, YUUKA_ERR_INVALID_ARGUMENT, "invalid ssm conv kernel %d", c.conv_kernel);
    if (c.expert_count > 0) {
        YK_REQUIRE(c.expert_used > 0 && c.expert_used <= c.expert_count, YUUKA_ERR_INVALID_ARGUMENT,
                   "expert used count %d is outside 1..%d", c.expert_used, c.expert_count);
        YK_REQUIRE(c.expert_ffn > 0, YUUKA_ERR_INVALID_ARGUMENT, "invalid expert feed-forward size %d", c.expert_ffn);
        YK_REQUIRE(c.shared_ffn > 0, YUUKA_ERR_INVALID_ARGUMENT, "invalid shared expert feed-forward size %d",
                   c.shared_ffn);
    } else {
        YK_REQUIRE(c.ffn > 0, YUUKA_ERR_INVALID_ARGUMENT, "invalid feed-forward size %d", c.ffn);
    }
    YK_REQUIRE(c.context_length > 0 && c.vocab > 0, YUUKA_ERR_INVALID_ARGUMENT, "invalid context or vocabulary size");
    // limits of this backend's kernels
    YK_REQUIRE(c.hidden % 8 == 0 && c.head_dim % 32 == 0, YUUKA_ERR_UNSUPPORTED, "hidden %% 8 and head_dim %% 32 must be 0");
    YK_REQUIRE(c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256, YUUKA_ERR_UNSUPPORTED,
               "head_dim %d is not 64, 128 or 256", c.head_dim);
    YK_REQUIRE(c.state_size == 64 || c.state_size == 128, YUUKA_ERR_UNSUPPORTED, "ssm state size %d is not 64 or 128",
               c.state_size);
    YK_REQUIRE(c.conv_kernel <= 8, YUUKA_ERR_UNSUPPORTED, "ssm conv kernel %d exceeds 8", c.conv_kernel);
    YK_REQUIRE(c.group_count > 0 && c.time_step_rank % c.group_count == 0, YUUKA_ERR_UNSUPPORTED,
               "time_step_rank %d is not a multiple of group_count %d", c.time_step_rank, c.group_count);
}

const Tensor & need(const yuuka_model * m, const std::string & name, uint64_t rows, uint64_t cols, bool f32_vector) {
    auto it = m->tensors.find(name);
    YK_REQUIRE(it != m->tensors.end(), YUUKA_ERR_INVALID_ARGUMENT, "missing required tensor \"%s\"", name.c_str());
    const Tensor & t = it->second;
    // F32 vectors are taken by element count (ssm_conv1d arrives as [kernel, channels]; model/qwen35/load.go:302-321
    // reads it by byte count)
    YK_REQUIRE(f32_vector ? t.rows * t.cols == rows * cols : (t.rows == rows && t.cols == cols), YUUKA_ERR_INVALID_ARGUMENT,
               "tensor \"%s\" has shape [%llu,%llu], want [%llu,%llu]", name.c_str(), (unsigned long long)t.cols,
               (unsigned long long)t.rows, (unsigned long long)cols, (unsigned long long)rows);
    if (f32_vector)
        YK_REQUIRE(t.dtype == YUUKA_DTYPE_F32, YUUKA_ERR_INVALID_ARGUMENT, "tensor \"%s\" uses dtype %u, want F32",
                   name.c_str(), t.dtype);
    return t;
}

const float * vec(const yuuka_model * m, const std::string & name, uint64_t n) {
    return reinterpret_cast<const float *>(need(m, name, 1, n, true).ptr);
}

// Concatenates row ranges of equal dtype and width into one allocation.
Tensor fuse(yuuka_model * m, std::vector<const Tensor *> parts) {
    Tensor out;
    for (const Tensor * t : parts) {
        if (t->dtype != parts[0]->dtype || t->cols != parts[0]->cols) return out;
    }
    uint64_t total = 0, rows = 0;
    for (const Tensor * t : parts) {
        total += t->bytes;
        rows += t->rows;
    }
    void * ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, total + 256);
    YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "fused weight allocation of %llu bytes failed",
               (unsigned long long)total);
    m->extra_allocs.push_back(ptr);
    uint64_t off = 0;
    for (const Tensor * t : parts) {
        YK_CUDA(cudaMemcpy((uint8_t *)ptr + off, t->ptr, t->bytes, cudaMemcpyDeviceToDevice));
        off += t->bytes;
    }
    YK_CUDA(cudaMemset((uint8_t *)ptr + total, 0, 256));
    out.ptr = (uint8_t *)ptr;
    out.dtype = parts[0]->dtype;
    out.rows = rows;
    out.cols = parts[0]->cols;
    out.bytes = total;
    return out;
}

// ffn_gate and ffn_up as one matrix, 16 rows of the first then the same 16 rows of the second: after
// tiling, row tiles 2i and 2i+1 hold gate and up of the same 16 columns of the FFN, which lets one CTA
// finish silu(gate) * up (forwardFFN, model/qwen35/forward.go:295-315) in its epilogue.
Tensor fuse_paired(yuuka_model * m, const Tensor & a, const Tensor & b) {
    Tensor out;
    if (a.dtype != b.dtype || a.cols != b.cols || a.rows != b.rows || a.rows % 16 != 0) return out;
    const uint64_t rb = row_bytes(a.dtype, a.cols), total = a.bytes + b.bytes;
    void * ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, total + 256);
    YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "fused weight allocation of %llu bytes failed",
               (unsigned long long)total);
    m->extra_allocs.push_back(ptr);
    YK_CUDA(cudaMemcpy2D(ptr, 32 * rb, a.ptr, 16 * rb, 16 * rb, a.rows / 16, cudaMemcpyDeviceToDevice));
    YK_CUDA(cudaMemcpy2D((uint8_t *)ptr + 16 * rb, 32 * rb, b.ptr, 16 * rb, 16 * rb, b.rows / 16, cudaMemcpyDeviceToDevice));
    YK_CUDA(cudaMemset((uint8_t *)ptr + total, 0, 256));
    out.ptr = (uint8_t *)ptr;
    out.dtype = a.dtype;
    out.rows = 2 * a.rows;
    out.cols = a.cols;
    out.bytes = total;
    out.paired = true;
    return out;
}

void drop(yuuka_model * m, const std::string & name) {
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return;
    free_tensor(it->second);
    m->tensors.erase(it);
}

// Replaces the GGUF-layout bytes of a matrix by their tile-ordered copy. name is
// the tensor's key in m->tensors, or empty for a fused allocation.
void tile_in_place(yuuka_model * m, Tensor & t, const std::string & name) {
    if (!t.present() || t.tiled || !tiled_supported(t.dtype, t.cols)) return;
    const uint64_t bytes = tiled_bytes(t.dtype, t.rows, t.cols);
    void * ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, bytes + 256);
    YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "tiled weight allocation of %llu bytes failed",
               (unsigned long long)bytes);
    m->extra_allocs.push_back(ptr);
    launch_tile_weights(nullptr, (uint8_t *)ptr, t.ptr, t.dtype, (int)t.rows, (int)t.cols);
    YK_CUDA(cudaDeviceSynchronize());
    if (!name.empty()) {
        drop(m, name);
    } else {
        for (auto it = m->extra_allocs.begin(); it != m->extra_allocs.end(); ++it)
            if (*it == (void *)t.ptr) {
                cudaFree(*it);
                m->extra_allocs.erase(it);
                break;
            }
    }
    t.ptr = (uint8_t *)ptr;
    t.bytes = bytes;
    t.owned = false;
    t.tiled = true;
}

// Expert matrices of one MoE layer, tile-ordered expert by expert. parts: tensors of `experts`
// stacked matrices of rows_each x cols (expertSlice, model/qwen35/forward.go:441-458); expert e of
// the result holds part[0]'s rows of e, then part[1]'s, ... as one matrix.
Tensor tile_experts(yuuka_model * m, std::vector<const Tensor *> parts, int experts, uint64_t rows_each, size_t * stride) {
    const Tensor & first = *parts[0];
    for (const Tensor * t : parts) {
        YK_REQUIRE(t->dtype == first.dtype && t->cols == first.cols && t->rows == rows_each * (uint64_t)experts, YUUKA_ERR_UNSUPPORTED,
                   "expert tensors of one projection must share dtype and shape");
    }
    YK_REQUIRE(tiled_supported(first.dtype, first.cols) && rows_each % 16 == 0, YUUKA_ERR_UNSUPPORTED,
               "expert matrices of dtype %u, %llu x %llu have no tiled layout", first.dtype, (unsigned long long)rows_each,
               (unsigned long long)first.cols);
    const uint64_t rb = row_bytes(first.dtype, first.cols);
    const uint64_t rows_fused = rows_each * parts.size();
    const uint64_t per_expert = tiled_bytes(first.dtype, rows_fused, first.cols);
    void * dst = nullptr;
    void * tmp = nullptr;
    cudaError_t err = cudaMalloc(&dst, per_expert * experts + 256);
    YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "expert weight allocation of %llu bytes failed",
               (unsigned long long)(per_expert * experts));
    m->extra_allocs.push_back(dst);
    err = cudaMalloc(&tmp, rows_fused * rb + 256);
    YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "expert staging allocation failed");
    try {
        for (int e = 0; e < experts; e++) {
            uint64_t off = 0;
            for (const Tensor * t : parts) {
                YK_CUDA(cudaMemcpyAsync((uint8_t *)tmp + off, t->ptr + (uint64_t)e * rows_each * rb, rows_each * rb,
                                        cudaMemcpyDeviceToDevice, nullptr));
                off += rows_each * rb;
            }
            launch_tile_weights(nullptr, (uint8_t *)dst + (uint64_t)e * per_expert, (const uint8_t *)tmp, first.dtype,
                                (int)rows_fused, (int)first.cols);
        }
        YK_CUDA(cudaDeviceSynchronize());
    } catch (...) {
        cudaFree(tmp);
        throw;
    }
    cudaFree(tmp);
    Tensor out;
    out.ptr = (uint8_t *)dst;
    out.dtype = first.dtype;
    out.rows = rows_fused;  // per expert
    out.cols = first.cols;
    out.bytes = per_expert * experts;
    out.tiled = true;
    *stride = per_expert;
    return out;
}

}  // namespace

extern "C" {

yuuka_status yuuka_model_create(yuuka_device * dev, const yuuka_model_config * cfg, yuuka_model ** out) {
    return guard([&] {
        YK_REQUIRE(dev && cfg && out, YUUKA_ERR_INVALID_ARGUMENT, "model_create: null argument");
        *out = nullptr;
        validate_config(*cfg);
        auto * m = new yuuka_model();
        m->dev = dev;
        m->cfg = *cfg;
        m->layers.resize(cfg->block_count);
        *out = m;
    });
}

void yuuka_model_destroy(yuuka_model * m) {
    if (!m) return;
    cudaSetDevice(m->dev->index);
    for (auto & kv : m->tensors) free_tensor(kv.second);
    for (void * p : m->extra_allocs) cudaFree(p);
    delete m;
}

yuuka_status yuuka_model_set_tensor(yuuka_model * m, const char * name, uint32_t dtype, const void * data,
                                    uint64_t rows, uint64_t cols) {
    return guard([&] {
        YK_REQUIRE(m && name && data, YUUKA_ERR_INVALID_ARGUMENT, "model_set_tensor: null argument");
        YK_REQUIRE(!m->finalized, YUUKA_ERR_INVALID_ARGUMENT, "model_set_tensor: model is finalized");
        uint64_t rb = row_bytes(dtype, cols);
        YK_REQUIRE(rb > 0 && dtype != YUUKA_DTYPE_BF16, YUUKA_ERR_UNSUPPORTED,
                   "tensor \"%s\": dtype %u does not fit a row of %llu columns", name, dtype, (unsigned long long)cols);
        YK_REQUIRE(rows > 0, YUUKA_ERR_INVALID_ARGUMENT, "tensor \"%s\": invalid row count", name);
        set_device(m->dev);
        Tensor t;
        t.dtype = dtype;
        t.rows = rows;
        t.cols = cols;
        t.bytes = rows * rb;
        t.owned = true;
        void * ptr = nullptr;
        cudaError_t err = cudaMalloc(&ptr, t.bytes + 256);  // slack: the GEMM ring copies whole 16-byte lines
        YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "tensor \"%s\": allocation of %llu bytes failed", name,
                   (unsigned long long)t.bytes);
        t.ptr = (uint8_t *)ptr;
        err = cudaMemcpy(ptr, data, t.bytes, cudaMemcpyHostToDevice);
        if (err == cudaSuccess) err = cudaMemset(t.ptr + t.bytes, 0, 256);
        if (err != cudaSuccess) {
            cudaFree(ptr);
            YK_CUDA(err);
        }
        drop(m, name);
        m->tensors[name] = t;
    });
}

yuuka_status yuuka_model_finalize(yuuka_model * m) {
    return guard([&] {
        YK_REQUIRE(m, YUUKA_ERR_INVALID_ARGUMENT, "model_finalize: null model");
        if (m->finalized) return;
        set_device(m->dev);
        const yuuka_model_config & c = m->cfg;
        const uint64_t H = c.hidden, V = c.vocab;
        m->embedding = need(m, "token_embd.weight", V, H, false);
        if (m->tensors.count("output.weight")) m->output = need(m, "output.weight", V, H, false);
        else m->output = m->embedding;  // tied head (model/qwen35/load.go:88-97)
        m->output_norm = vec(m, "output_norm.weight", H);
        const uint64_t S = c.state_size, R = c.time_step_rank, inner = c.inner_size;
        const uint64_t conv_dim = m->conv_dim(), q_dim = m->q_dim(), kv_dim = m->kv_dim(), o_dim = m->o_dim();
        uint64_t moe_bytes = 0;
        for (int i = 0; i < c.block_count; i++) {
            LayerW & L = m->layers[i];
            const std::string p = "blk." + std::to_string(i) + ".";
            L.attn_norm = vec(m, p + "attn_norm.weight", H);
            L.post_norm = vec(m, p + "post_attention_norm.weight", H);
            if (m->recurrent(i)) {
                L.qkv = need(m, p + "attn_qkv.weight", conv_dim, H, false);
                L.gate = need(m, p + "attn_gate.weight", inner, H, false);
                L.out = need(m, p + "ssm_out.weight", H, inner, false);
                L.beta = need(m, p + "ssm_beta.weight", R, H, false);
                L.alpha = need(m, p + "ssm_alpha.weight", R, H, false);
                L.conv = reinterpret_cast<const float *>(need(m, p + "ssm_conv1d.weight", 1, c.conv_kernel * conv_dim, true).ptr);
                L.dt = vec(m, p + "ssm_dt.bias", R);
                L.a = vec(m, p + "ssm_a", R);
                L.ssm_norm = vec(m, p + "ssm_norm.weight", S);
                L.proj = fuse(m, {&L.qkv, &L.gate, &L.beta, &L.alpha});
                if (L.proj.present()) {
                    for (const char * n : {"attn_qkv.weight", "attn_gate.weight", "ssm_beta.weight", "ssm_alpha.weight"})
                        drop(m, p + n);
                    L.qkv = L.gate = L.beta = L.alpha = Tensor();
                }
            } else {
                L.q = need(m, p + "attn_q.weight", q_dim, H, false);
                L.k = need(m, p + "attn_k.weight", kv_dim, H, false);
                L.v = need(m, p + "attn_v.weight", kv_dim, H, false);
                L.o = need(m, p + "attn_output.weight", H, o_dim, false);
                L.q_norm = vec(m, p + "attn_q_norm.weight", c.head_dim);
                L.k_norm = vec(m, p + "attn_k_norm.weight", c.head_dim);
                L.qk = fuse(m, {&L.q, &L.k, &L.v});
                L.qk_has_v = L.qk.present();
                if (!L.qk.present()) L.qk = fuse(m, {&L.q, &L.k});
                if (L.qk.present()) {
                    drop(m, p + "attn_q.weight");
                    drop(m, p + "attn_k.weight");
                    L.q = L.k = Tensor();
                    if (L.qk_has_v) {
                        drop(m, p + "attn_v.weight");
                        L.v = Tensor();
                    }
                }
            }
            if (c.expert_count > 0) {
                const uint64_t E = c.expert_count, EF = c.expert_ffn, SF = c.shared_ffn;
                L.router = reinterpret_cast<const float *>(need(m, p + "ffn_gate_inp.weight", E, H, true).ptr);
                L.sh_gate_inp = vec(m, p + "ffn_gate_inp_shexp.weight", H);
                L.sh_gate = need(m, p + "ffn_gate_shexp.weight", SF, H, false);
                L.sh_up = need(m, p + "ffn_up_shexp.weight", SF, H, false);
                L.sh_down = need(m, p + "ffn_down_shexp.weight", H, SF, false);
                const Tensor ge = need(m, p + "ffn_gate_exps.weight", EF * E, H, false);
                const Tensor ue = need(m, p + "ffn_up_exps.weight", EF * E, H, false);
                const Tensor de = need(m, p + "ffn_down_exps.weight", H * E, EF, false);
                moe_bytes += ge.bytes + ue.bytes + de.bytes;
                L.exp_gate_up = tile_experts(m, {&ge, &ue}, (int)E, EF, &L.exp_gate_up_stride);
                L.exp_down = tile_experts(m, {&de}, (int)E, H, &L.exp_down_stride);
                for (const char * n : {"ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"}) drop(m, p + n);
                L.sh_gate_up = fuse(m, {&L.sh_gate, &L.sh_up});
                if (L.sh_gate_up.present()) {
                    drop(m, p + "ffn_gate_shexp.weight");
                    drop(m, p + "ffn_up_shexp.weight");
                    L.sh_gate = L.sh_up = Tensor();
                }
                continue;
            }
            L.ffn_gate = need(m, p + "ffn_gate.weight", c.ffn, H, false);
            L.ffn_up = need(m, p + "ffn_up.weight", c.ffn, H, false);
            L.ffn_down = need(m, p + "ffn_down.weight", H, c.ffn, false);
            L.gate_up = fuse_paired(m, L.ffn_gate, L.ffn_up);
            if (!L.gate_up.present()) L.gate_up = fuse(m, {&L.ffn_gate, &L.ffn_up});
            if (L.gate_up.present()) {
                drop(m, p + "ffn_gate.weight");
                drop(m, p + "ffn_up.weight");
                L.ffn_gate = L.ffn_up = Tensor();
            }
        }
        // bytes one step streams: every matrix and vector except the embedding table
        uint64_t total = 0;
        for (auto & kv : m->tensors)
            if (kv.first != "token_embd.weight") total += kv.second.bytes;
        for (const LayerW & L : m->layers) total += L.proj.bytes + L.qk.bytes + L.gate_up.bytes + L.sh_gate_up.bytes;
        m->weight_bytes = total + moe_bytes;
        // tile-ordered copies for the GEMM kernels; the GGUF-layout bytes are released
        const bool tied = !m->tensors.count("output.weight");
        for (int i = 0; i < c.block_count; i++) {
            LayerW & L = m->layers[i];
            const std::string p = "blk." + std::to_string(i) + ".";
            tile_in_place(m, L.proj, "");
            tile_in_place(m, L.qk, "");
            tile_in_place(m, L.gate_up, "");
            tile_in_place(m, L.qkv, p + "attn_qkv.weight");
            tile_in_place(m, L.gate, p + "attn_gate.weight");
            tile_in_place(m, L.beta, p + "ssm_beta.weight");
            tile_in_place(m, L.alpha, p + "ssm_alpha.weight");
            tile_in_place(m, L.out, p + "ssm_out.weight");
            tile_in_place(m, L.q, p + "attn_q.weight");
            tile_in_place(m, L.k, p + "attn_k.weight");
            tile_in_place(m, L.v, p + "attn_v.weight");
            tile_in_place(m, L.o, p + "attn_output.weight");
            tile_in_place(m, L.ffn_gate, p + "ffn_gate.weight");
            tile_in_place(m, L.ffn_up, p + "ffn_up.weight");
            tile_in_place(m, L.ffn_down, p + "ffn_down.weight");
            tile_in_place(m, L.sh_gate_up, "");
            tile_in_place(m, L.sh_gate, p + "ffn_gate_shexp.weight");
            tile_in_place(m, L.sh_up, p + "ffn_up_shexp.weight");
            tile_in_place(m, L.sh_down, p + "ffn_down_shexp.weight");
        }
        if (!tied) tile_in_place(m, m->output, "output.weight");
        else if (tiled_supported(m->output.dtype, m->output.cols)) {
            // tied head: the embedding gather needs the GGUF rows, the head a tiled copy
            Tensor head = m->output;
            head.owned = false;
            const uint64_t bytes = tiled_bytes(head.dtype, head.rows, head.cols);
            void * ptr = nullptr;
            cudaError_t err = cudaMalloc(&ptr, bytes + 256);
            YK_REQUIRE(err == cudaSuccess, YUUKA_ERR_ALLOCATION, "tiled head allocation failed");
            m->extra_allocs.push_back(ptr);
            launch_tile_weights(nullptr, (uint8_t *)ptr, head.ptr, head.dtype, (int)head.rows, (int)head.cols);
            YK_CUDA(cudaDeviceSynchronize());
            head.ptr = (uint8_t *)ptr;
            head.bytes = bytes;
            head.tiled = true;
            m->output = head;
        }
        m->finalized = true;
    });
}

uint64_t yuuka_model_weight_bytes(const yuuka_model * m) { return m ? m->weight_bytes : 0; }

}  // extern "C"

// ===========================================================================
// session

namespace {

template <typename T>
T * dalloc(size_t count, std::vector<void *> & owned, bool zero = true) {
    void * p = nullptr;
    size_t bytes = (count > 0 ? count : 1) * sizeof(T);
    cudaError_t err = cudaMalloc(&p, bytes);
    if (err != cudaSuccess) {
        cudaGetLastError();
        YK_REQUIRE(false, YUUKA_ERR_ALLOCATION, "session allocation of %llu bytes failed", (unsigned long long)bytes);
    }
    owned.push_back(p);
    if (zero) YK_CUDA(cudaMemset(p, 0, bytes));
    return (T *)p;
}

struct LayerState {
    // attention layers
    uint8_t * k = nullptr;
    uint8_t * v = nullptr;
    // recurrent layers
    float * conv_state = nullptr;  // [batch][conv_dim][kernel-1]
    float * state = nullptr;       // [batch][rank][S][S]
    float * proj = nullptr;        // [rows][n_proj] kept until the commit
    float * khat = nullptr;
    float * dlog = nullptr;
    float * decay = nullptr;
};

}  // namespace

struct yuuka_session {
    yuuka_model * model = nullptr;
    yuuka_session_config cfg{};
    yuuka_stream stream;
    std::vector<void *> owned;
    int table_stride = 0;
    int kv_row_bytes = 0;
    int64_t conv_count = 0, s_count = 0;
    std::vector<LayerState> layers;
    std::vector<int> gdn_layers, attn_layers;
    GdnLayerCommit * d_gdn_commit = nullptr;
    KvLayerCommit * d_kv_commit = nullptr;
    // per sequence
    int32_t * d_pos0 = nullptr;
    int32_t * d_tables = nullptr;
    std::vector<int> h_pos, h_pos_upper;
    // per step
    // row metadata of a step, one device block [anc | tokens | parent | depth] filled by one copy from the
    // page-locked mirror h_rows; results [accepted | path | emitted] likewise come back in one copy to h_results
    uint8_t * d_rows = nullptr;
    uint8_t * h_rows = nullptr;
    int32_t * d_results = nullptr;
    int32_t * h_results = nullptr;  // + two words for the device error flags
    int rows_cap = 0;
    int32_t * d_pos_sub = nullptr;   // [CHAIN_MAX_SUBS] first position of every sub-chunk of a wide prompt pass
    int32_t * d_acc_sub = nullptr;   // [CHAIN_MAX_SUBS] rows - 1 of every sub-chunk (its forced acceptance)
    int32_t * d_seq_map = nullptr;   // [max_batch] which sequence each slot of the staged step is
    int32_t * d_tokens = nullptr;
    int32_t * d_parent = nullptr;
    int32_t * d_depth = nullptr;
    uint64_t * d_anc = nullptr;
    float *x = nullptr, *xn = nullptr, *qkv_attn = nullptr, *attn_out = nullptr, *gdn_out = nullptr;
    float *gate_up = nullptr, *act = nullptr, *logits = nullptr;
    float2 * rope_cs = nullptr;  // [rows][rope_dim / 2] (cos, sin) of the step's rows, attention layers only
    // qwen35moe scratch: routing, expert-sorted (row, slot) pairs, expert and shared-expert activations
    int32_t *moe_ids = nullptr, *moe_pos = nullptr, *moe_row = nullptr;
    float * moe_logits = nullptr;  // [rows][experts] router logits
    int * moe_counters = nullptr;  // one per group of eight rows, zero between launches
    float *moe_w = nullptr, *moe_sg = nullptr, *moe_gu = nullptr, *moe_act = nullptr, *moe_y = nullptr;
    float *sh_gu = nullptr, *sh_act = nullptr, *sh_y = nullptr;
    GemmSegment * moe_segments = nullptr;
    int moe_max_segments = 0;
    XPrepOut prep_moe_act, prep_sh_act;
    XPrepOut prep_xn, prep_attn, prep_gdn, prep_act;  // fp16 + group sums of the GEMM inputs
    float *gdn_qn = nullptr, *gdn_vconv = nullptr, *gdn_beta = nullptr;
    // RMSNorm folded into the GEMMs around it (NormFuse): one row of fixed-point sums of squares per norm
    // point of a step, zeroed when the step starts; norm_point indexes the row behind the current prep_xn
    bool fold_norm = false;          // the model allows it (every consumer and producer matrix is tile-ordered)
    bool fold_step = false;          // ... and this step's row count does
    bool fold_swiglu = true;         // silu(gate) * up in the gate|up GEMM's epilogue (YUUKA_CUDA_NO_FOLD_SWIGLU=1: own kernel)
    unsigned long long * norm_sumsq = nullptr;  // [norm points][32]
    int norm_point = 0;
    bool xn_raw = false;             // prep_xn holds x * w * pre of norm_point (not normalised rows)
    int chain_rows = 0;  // rows per prompt chunk (prefill_logits / forward)
    // L2 prefetch of the next GEMM's weights: matrices in the order a step streams them
    bool prefetch_next = true;
    bool gdn_chunked = true;  // prompt sub-chunks through the chunkwise delta-net scan (YUUKA_CUDA_NO_GDN_CHUNK=1: row by row)
    uint64_t prefetch_bytes = 16ull << 20;  // measured: 16 MB ahead 3.09 ms/step, none 3.12, 48 MB 3.13
    std::vector<std::pair<const uint8_t *, uint64_t>> gemm_order;
    size_t order_pos = 0;
    int n_proj = 0, n_qkv = 0;
    ArgmaxScratch argmax{};
    AcceptOut acc{};
    float * attn_partial = nullptr;
    size_t attn_partial_floats = 0;
    GemmScratch gemm;
    // staged step
    int st_seq0 = 0, st_batch = 0, st_nodes = 0;
    int st_chains = 0;         // every sequence of the staged step is a chain (no row has a sibling)
    std::vector<int> st_seqs;  // sequences of the staged step, slot by slot
    // device-drafted generation (yuuka_spec_generate_device): token history of the generating sequence,
    // its length, and [steps, draft tokens, accepted drafts, draft length of the staged step]
    int32_t * d_hist = nullptr;
    int32_t * d_hist_len = nullptr;
    int32_t * d_spec_stats = nullptr;
    int hist_cap = 0;
    uint32_t st_mode = 0;
    float st_temperature = 0.0f;
    const float * st_draft_probs = nullptr;   // device, rejection mode
    float * d_uniforms = nullptr;             // [max_batch * max_nodes * 2]
    unsigned long long * reject_residual = nullptr;  // [max_batch][vocab], allocated by the first rejection step
    bool staged = false, launched = false;
    uint32_t launches = 0;
    // captured steps, keyed by (seq0, batch, nodes, chains, mode), least recently used first; at most
    // MAX_STEP_GRAPHS are kept (a scheduler that varies batch and row counts freely would otherwise
    // accumulate one instantiated graph of a few hundred nodes per shape for the life of the session)
    static constexpr size_t MAX_STEP_GRAPHS = 48;
    struct StepGraph {
        int seq0, batch, nodes, chains;
        uint32_t mode;
        cudaGraphExec_t exec;
        uint32_t launches;
    };
    std::vector<StepGraph> graphs;
    bool use_graphs = true;
    // per-op attribution (yuuka_verify_launch_profiled)
    bool profiling = false;
    std::vector<std::pair<uint32_t, cudaEvent_t>> prof;
};

namespace {

// Records an event in front of the next op when a profiled launch is running.
void mark(yuuka_session * s, uint32_t code) {
    if (!s->profiling) return;
    cudaEvent_t e;
    YK_CUDA(cudaEventCreate(&e));
    YK_CUDA(cudaEventRecord(e, s->stream.s));
    s->prof.push_back({code, e});
}

void gemm(yuuka_session * s, const Tensor & w, const float * x, int ldx, XPrepOut prep, float * out, int ldo, int rows,
          uint32_t flags, const float * produce_norm_w = nullptr, const XPrepOut * swiglu = nullptr) {
    mark(s, w.rows > 65536 ? YUUKA_OP_LM_HEAD : YUUKA_OP_GEMM);
    if (w.tiled) {
        TiledGemmArgs t;
        t.w = w.ptr;
        t.w_dtype = w.dtype;
        t.x = x;
        t.xprep = prep;
        t.x_dtype = YUUKA_DTYPE_F32;
        t.ldx = ldx;
        t.out = out;
        t.ldo = ldo;
        t.rows = rows;
        t.n_out = (int)w.rows;
        t.n_in = (int)w.cols;
        t.path = YUUKA_GEMM_PATH_AUTO;
        t.flags = flags;
        t.scratch = &s->gemm;
        t.exact_only = (s->cfg.flags & YUUKA_SESSION_EXACT_WIDE) != 0;
        t.wide_from_33 = (s->cfg.flags & YUUKA_SESSION_WIDE_FROM_33) != 0;
        if (s->cfg.flags & YUUKA_SESSION_TEST_DROP_COPIES) t.flags |= YUUKA_GEMM_TEST_DROP_COPIES;
        if (swiglu) t.swiglu = *swiglu;
        if (s->fold_step) {
            const yuuka_model_config & mc = s->model->cfg;
            t.norm.eps = mc.rms_eps;
            t.norm.cols = mc.hidden;
            if (prep.xh == s->prep_xn.xh && s->xn_raw) {
                // the rows in prep_xn are x * w * pre, not normalised: this GEMM applies scale / pre
                t.norm.consume_now = s->norm_sumsq + (size_t)s->norm_point * 32;
                t.norm.consume_prev = s->norm_sumsq + (size_t)(s->norm_point - 1) * 32;
            }
            if (produce_norm_w) {
                t.norm.produce_w = produce_norm_w;
                t.norm.produce_prev = s->norm_sumsq + (size_t)s->norm_point * 32;
                t.norm.produce_sumsq = s->norm_sumsq + (size_t)(s->norm_point + 1) * 32;
                t.norm.produce_prep = s->prep_xn;
            }
        }
        if (s->prefetch_next) {
            // where this matrix sits in the step's order, and what follows it
            const auto & order = s->gemm_order;
            for (size_t k = s->order_pos; k < order.size(); k++)
                if (order[k].first == w.ptr) {
                    s->order_pos = k + 1;
                    if (k + 1 < order.size()) {
                        t.next_w = order[k + 1].first;
                        t.next_bytes = order[k + 1].second < s->prefetch_bytes ? order[k + 1].second : s->prefetch_bytes;
                    }
                    break;
                }
        }
        s->launches += launch_gemm_tiled(s->model->dev, s->stream.s, t);
        return;
    }
    GemmArgs a;
    a.w = w.ptr;
    a.w_readable = w.bytes + 256;
    a.w_dtype = w.dtype;
    a.x = x;
    a.x_dtype = YUUKA_DTYPE_F32;
    a.ldx = ldx;
    a.out = out;
    a.ldo = ldo;
    a.rows = rows;
    a.n_out = (int)w.rows;
    a.n_in = (int)w.cols;
    a.path = YUUKA_GEMM_PATH_AUTO;
    a.flags = flags;
    a.scratch = &s->gemm;
    s->launches += launch_gemm_quant(s->model->dev, s->stream.s, a);
}

// x += W * in, then xn = rmsnorm(x) * norm_w (skipped when norm_w is null). With up to 32 rows the norm is
// folded into this GEMM's epilogue and the next GEMM's; otherwise it runs as its own kernel.
void gemm_residual_norm(yuuka_session * s, const Tensor & w, const float * in, int ld_in, XPrepOut prep_in, int rows,
                        const float * norm_w) {
    const yuuka_model_config & c = s->model->cfg;
    const int H = c.hidden;
    if (s->fold_step && norm_w) {
        // the norm rides on this GEMM (producer) and on the next one to read prep_xn (consumer)
        gemm(s, w, in, ld_in, prep_in, s->x, H, rows, YUUKA_GEMM_ACCUMULATE, norm_w);
        s->norm_point++;
        s->xn_raw = true;
        return;
    }
    gemm(s, w, in, ld_in, prep_in, s->x, H, rows, YUUKA_GEMM_ACCUMULATE);
    if (norm_w) {
        mark(s, YUUKA_OP_RMSNORM);
        launch_rmsnorm(s->stream.s, s->xn, H, s->x, H, norm_w, H, rows, c.rms_eps, s->prep_xn);
        s->launches++;
    }
}

void reserve_gemm(yuuka_session * s, const Tensor & w, int rows) {
    if (w.present()) gemm_scratch_reserve(s->model->dev, s->gemm, w.dtype, rows, (int)w.rows, (int)w.cols);
}

enum LogitRows { LOGITS_NONE, LOGITS_LAST, LOGITS_ALL };

// Prompt tokens run through the step kernels in chains of up to this many rows (the row masks are 64 bits
// wide); from 48 rows on the GEMMs take the tensor-memory route.
// A prompt runs in passes of up to CHAIN_ROWS rows: the GEMMs and row-wise kernels take the whole pass (the
// tensor-memory GEMM route decodes a weight tile once for up to 512 rows), the sequential mixers (delta-net
// scan + state commit, attention front end + attention) walk it in sub-chunks of CHAIN_SUB rows, the limit
// of their per-step row bookkeeping (64-bit ancestor masks).
constexpr int CHAIN_ROWS = 512;
constexpr int CHAIN_SUB = 64;
constexpr int CHAIN_MAX_SUBS = CHAIN_ROWS / CHAIN_SUB;

// Enqueues one step over sequences [seq0, seq0+batch) with `nodes` rows each.
// sub > 0: a wide prompt pass of one sequence (see CHAIN_ROWS), staged by stage_rows with the same sub.
// mapped: the slots of the step are the sequences listed in d_seq_map (a verify batch; seq0 is 0 then);
// otherwise slot b is sequence seq0 + b.
void run_step(yuuka_session * s, int seq0, int batch, int nodes, uint32_t mode, LogitRows logit_rows, int max_total,
              int sub = 0, bool mapped = false) {
    yuuka_model * m = s->model;
    const yuuka_model_config & c = m->cfg;
    cudaStream_t st = s->stream.s;
    const int R = batch * nodes, H = c.hidden;
    RowMeta rows{s->d_tokens, s->d_parent, s->d_depth, s->d_anc, s->d_pos0 + seq0, batch, nodes};
    rows.chains = sub > 0 ? 1 : s->st_chains;
    if (mapped) rows.seq_map = s->d_seq_map;
    YK_REQUIRE(!mapped || (seq0 == 0 && sub == 0), YUUKA_ERR_INTERNAL, "a mapped step starts at sequence 0 and has no sub-chunks");
    YK_REQUIRE(sub == 0 || (batch == 1 && mode == 3u && nodes <= CHAIN_MAX_SUBS * sub), YUUKA_ERR_INTERNAL,
               "a wide pass is one forced-commit chain");
    const int n_sub = sub > 0 ? (nodes + sub - 1) / sub : 1;
    // sub-chunk k as a step of its own: rows [k * sub, ...), positions from d_pos_sub[k]
    auto sub_rows = [&](int k) {
        const int r0 = k * sub, n = nodes - r0 < sub ? nodes - r0 : sub;
        RowMeta rk{s->d_tokens + r0, s->d_parent + r0, s->d_depth + r0, s->d_anc + r0, s->d_pos_sub + k, 1, n};
        rk.chains = 1;
        return rk;
    };
    int gdn_index = 0;  // position of the current recurrent layer in d_gdn_commit
    if (sub > 0) {
        // the per-layer commits of the sub-chunks walk the identity path 1, 2, 3, ...
        launch_accept_all(st, rows, s->acc);
        s->launches++;
    }
    const int K1 = c.conv_kernel - 1;
    const int conv_dim = m->conv_dim(), inner = c.inner_size, rank = c.time_step_rank, S = c.state_size;
    const int q_dim = m->q_dim(), kv_dim = m->kv_dim(), o_dim = m->o_dim(), F = c.ffn;

    s->order_pos = 0;
    // with up to 32 rows every norm after the first is folded into the GEMM that finishes the residual rows
    // and the GEMM that reads them
    s->fold_step = s->fold_norm && R <= 32;
    s->norm_point = 0;
    s->xn_raw = false;
    if (s->fold_step) YK_CUDA(cudaMemsetAsync(s->norm_sumsq, 0, sizeof(unsigned long long) * 32 * (size_t)(2 * c.block_count + 2), st));
    unsigned long long * sumsq0 = s->fold_step ? s->norm_sumsq : nullptr;
    mark(s, YUUKA_OP_EMBEDDING);
    if (sub == 0 && (H & 7) == 0) {
        // embedding rows, the first layer's input norm and the rows' RoPE table: one launch, one CTA per row
        launch_embedding_first(st, s->x, H, m->embedding.ptr, m->embedding.dtype, H, c.vocab, s->d_tokens, R, m->layers[0].attn_norm,
                               s->xn, H, c.rms_eps, s->prep_xn, sumsq0, s->rope_cs, rows, c.rope_dim, c.rope_freq_base);
        s->launches++;
    } else {
        launch_embedding(st, s->x, H, m->embedding.ptr, m->embedding.dtype, H, c.vocab, s->d_tokens, R);
        s->launches++;
        if (s->rope_cs) {
            // (a wide pass: every sub-chunk counts positions from its own start; rows past the end are scratch)
            RowMeta rr = sub > 0 ? RowMeta{s->d_tokens, s->d_parent, s->d_depth, s->d_anc, s->d_pos_sub, n_sub, sub} : rows;
            launch_rope_table(st, s->rope_cs, rr, c.rope_dim, c.rope_freq_base);
            s->launches++;
        }
        mark(s, YUUKA_OP_RMSNORM);
        launch_rmsnorm(st, s->xn, H, s->x, H, m->layers[0].attn_norm, H, R, c.rms_eps, s->prep_xn, sumsq0);
        s->launches++;
    }
    for (int i = 0; i < c.block_count; i++) {
        const LayerW & L = m->layers[i];
        LayerState & LS = s->layers[i];
        const float * next_norm = i + 1 < c.block_count ? m->layers[i + 1].attn_norm
                                                         : (logit_rows == LOGITS_ALL ? m->output_norm : nullptr);
        if (m->recurrent(i)) {
            const int np = s->n_proj;
            if (L.proj.present()) {
                gemm(s, L.proj, s->xn, H, s->prep_xn, LS.proj, np, R, 0);
            } else {
                gemm(s, L.qkv, s->xn, H, s->prep_xn, LS.proj, np, R, 0);
                gemm(s, L.gate, s->xn, H, s->prep_xn, LS.proj + conv_dim, np, R, 0);
                gemm(s, L.beta, s->xn, H, s->prep_xn, LS.proj + conv_dim + inner, np, R, 0);
                gemm(s, L.alpha, s->xn, H, s->prep_xn, LS.proj + conv_dim + inner + rank, np, R, 0);
            }
            GdnArgs g;
            g.proj = LS.proj;
            g.ldp = np;
            g.conv_w = L.conv;
            g.dt = L.dt;
            g.a = L.a;
            g.conv_state = LS.conv_state + (int64_t)seq0 * conv_dim * K1;
            g.state = LS.state + (int64_t)seq0 * rank * S * S;
            g.out = s->gdn_out;
            g.prep = s->prep_gdn;
            g.z = LS.proj + conv_dim;
            g.ldz = np;
            g.norm = L.ssm_norm;
            g.qn = s->gdn_qn;
            g.vconv = s->gdn_vconv;
            g.beta = s->gdn_beta;
            g.khat = LS.khat;
            g.dlog = LS.dlog;
            g.decay = LS.decay;
            g.groups = c.group_count;
            g.rank = rank;
            g.S = S;
            g.kernel = c.conv_kernel;
            g.eps = c.rms_eps;
            mark(s, YUUKA_OP_GDN_SCAN);
            if (sub == 0) {
                s->launches += launch_gdn_scan(st, g, rows);
            } else {
                // sub-chunk after sub-chunk: scan, then this layer's state and conv history move on before the next.
                // Every row of a prompt pass is committed, so by default the front end runs once for the whole pass,
                // the chunkwise form of the recurrence writes the state itself, and the conv history moves once.
                const int key_dim = c.group_count * S;
                const bool chunked = s->gdn_chunked;
                if (chunked) {
                    launch_gdn_front_chain(st, g, seq0, nodes);
                    s->launches++;
                }
                for (int k = 0; k < n_sub; k++) {
                    const int64_t r0 = (int64_t)k * sub;
                    GdnArgs gk = g;
                    gk.proj = g.proj + r0 * np;
                    gk.z = g.z + r0 * np;
                    gk.out = g.out + r0 * inner;
                    if (g.prep.xh) {
                        gk.prep.xh = g.prep.xh + r0 * inner;
                        gk.prep.xl = g.prep.xl + r0 * inner;
                        gk.prep.xs16 = g.prep.xs16 + r0 * (inner / 16);
                    }
                    gk.qn = g.qn + r0 * key_dim;
                    gk.vconv = g.vconv + r0 * inner;
                    gk.beta = g.beta + r0 * rank;
                    gk.khat = g.khat + r0 * key_dim;
                    gk.dlog = g.dlog + r0 * inner;
                    gk.decay = g.decay + r0 * rank;
                    const RowMeta rk = sub_rows(k);
                    if (chunked) {
                        launch_gdn_chunk(st, gk, rk);
                        s->launches++;
                        continue;
                    }
                    s->launches += launch_gdn_scan(st, gk, rk);
                    AcceptOut ak{s->d_acc_sub + k, s->acc.path, s->acc.emitted};
                    launch_gdn_commit(st, s->d_gdn_commit + gdn_index, 1, c.group_count, rank, S, c.conv_kernel, conv_dim, seq0, rk,
                                      ak, (int)r0);
                    s->launches++;
                }
                if (chunked) {
                    // (rows = the whole pass, accepted = all of it: launch_accept_all has filled the identity path)
                    launch_gdn_commit(st, s->d_gdn_commit + gdn_index, 1, c.group_count, rank, S, c.conv_kernel, conv_dim, seq0, rows,
                                      s->acc, 0, true);
                    s->launches++;
                }
            }
            gdn_index++;
            gemm_residual_norm(s, L.out, s->gdn_out, inner, s->prep_gdn, R, L.post_norm);
        } else {
            const int nq = s->n_qkv;
            float * qb = s->qkv_attn;
            float * kb = qb + q_dim;
            float * vb = kb + kv_dim;
            if (L.qk.present()) {
                gemm(s, L.qk, s->xn, H, s->prep_xn, qb, nq, R, 0);
                if (!L.qk_has_v) gemm(s, L.v, s->xn, H, s->prep_xn, vb, nq, R, 0);
            } else {
                gemm(s, L.q, s->xn, H, s->prep_xn, qb, nq, R, 0);
                gemm(s, L.k, s->xn, H, s->prep_xn, kb, nq, R, 0);
                gemm(s, L.v, s->xn, H, s->prep_xn, vb, nq, R, 0);
            }
            KvPool pool;
            pool.k = LS.k;
            pool.v = LS.v;
            pool.format = s->cfg.kv_format;
            pool.block_size = s->cfg.block_size;
            pool.pool_blocks = s->cfg.pool_blocks;
            pool.kv_dim = kv_dim;
            pool.row_bytes = s->kv_row_bytes;
            pool.tables = s->d_tables + (int64_t)seq0 * s->table_stride;
            pool.table_stride = s->table_stride;
            mark(s, YUUKA_OP_ATTN_PREP);
            if (sub == 0) {
                launch_attn_prep(st, qb, nq, kb, nq, vb, nq, L.q_norm, L.k_norm, c.heads, c.kv_heads, c.head_dim, c.rope_dim,
                                 s->rope_cs, c.rms_eps, rows, pool);
                s->launches++;
            }
            AttnScratch sc;
            const int G = c.heads / c.kv_heads;
            const int qtiles = attention_query_tiles(G * (sub > 0 ? sub : nodes));
            const int base = c.kv_heads * qtiles * batch;
            // about one CTA per SM at capacity (measured at a 1500-token context: 3.11 ms per step, against 3.16 with
            // two or four per SM: fewer partials for the merge kernel outweigh the shorter key ranges)
            int splits = (m->dev->sm_count + base - 1) / base;
            // many sequences of different lengths: key ranges of at most 512 keys, so that the CTAs of a long context
            // spread over the machine instead of one of them walking it alone (ranges beyond a sequence's end exit at once)
            if (base >= m->dev->sm_count && splits < (max_total + 511) / 512) splits = (max_total + 511) / 512;
            int max_splits = (max_total + 31) / 32;
            if (splits > max_splits) splits = max_splits;
            if (splits < 1) splits = 1;
            sc.key_split = (((max_total + splits - 1) / splits + 31) / 32) * 32;
            sc.splits = (max_total + sc.key_split - 1) / sc.key_split;
            sc.partial = s->attn_partial;
            YK_REQUIRE(attention_scratch_floats(sub > 0 ? sub : R, c.heads, c.head_dim, sc.splits) <= s->attn_partial_floats,
                       YUUKA_ERR_INTERNAL, "attention scratch is too small");
            mark(s, YUUKA_OP_ATTENTION);
            if (sub == 0) {
                s->launches += launch_attention(st, s->attn_out, o_dim, qb, nq, c.heads, c.kv_heads, c.head_dim, rows, pool,
                                                max_total, sc, s->prep_attn);
            } else {
                // a sub-chunk's K/V rows are in the pool before the next sub-chunk's queries look for them
                const int half = c.rope_dim / 2;
                for (int k = 0; k < n_sub; k++) {
                    const int64_t r0 = (int64_t)k * sub;
                    const RowMeta rk = sub_rows(k);
                    launch_attn_prep(st, qb + r0 * nq, nq, kb + r0 * nq, nq, vb + r0 * nq, nq, L.q_norm, L.k_norm, c.heads,
                                     c.kv_heads, c.head_dim, c.rope_dim, s->rope_cs + r0 * half, c.rms_eps, rk, pool);
                    XPrepOut pk = s->prep_attn;
                    if (pk.xh) {
                        pk.xh += r0 * o_dim;
                        pk.xl += r0 * o_dim;
                        pk.xs16 += r0 * (o_dim / 16);
                    }
                    s->launches += 1 + launch_attention(st, s->attn_out + r0 * o_dim, o_dim, qb + r0 * nq, nq, c.heads, c.kv_heads,
                                                        c.head_dim, rk, pool, max_total, sc, pk);
                }
            }
            gemm_residual_norm(s, L.o, s->attn_out, o_dim, s->prep_attn, R, L.post_norm);
        }
        if (c.expert_count > 0) {
            // forwardMoEFFN (model/qwen35/forward.go:320-389); xn = rmsnorm(x) * post_norm is in place
            const int E = c.expert_count, U = c.expert_used, EF = c.expert_ffn, SF = c.shared_ffn, P = R * U;
            YK_REQUIRE(s->prep_xn.xh, YUUKA_ERR_UNSUPPORTED, "moe: hidden size must be a multiple of 16");
            mark(s, YUUKA_OP_MOE_ROUTE);
            launch_moe_route(st, s->xn, L.router, L.sh_gate_inp, H, E, U, R, s->moe_ids, s->moe_w, s->moe_sg, s->moe_logits,
                             s->moe_counters);
            launch_moe_group(st, s->moe_ids, R, U, E, s->moe_pos, s->moe_row, s->moe_segments, s->moe_max_segments);
            s->launches += 2;
            mark(s, YUUKA_OP_MOE_EXPERTS);
            GroupedGemmArgs ga;
            ga.w = L.exp_gate_up.ptr;
            ga.w_dtype = L.exp_gate_up.dtype;
            ga.expert_stride = L.exp_gate_up_stride;
            ga.xprep = s->prep_xn;
            ga.row_index = s->moe_row;
            ga.out = s->moe_gu;
            ga.ldo = 2 * EF;
            ga.n_out = 2 * EF;
            ga.n_in = H;
            ga.segments = s->moe_segments;
            ga.max_segments = s->moe_max_segments;
            s->launches += launch_gemm_tiled_grouped(m->dev, st, ga);
            launch_silu_mul(st, s->moe_act, EF, s->moe_gu, s->moe_gu + EF, 2 * EF, EF, P, s->prep_moe_act);
            s->launches++;
            GroupedGemmArgs gd;
            gd.w = L.exp_down.ptr;
            gd.w_dtype = L.exp_down.dtype;
            gd.expert_stride = L.exp_down_stride;
            gd.xprep = s->prep_moe_act;
            gd.out = s->moe_y;
            gd.ldo = H;
            gd.n_out = H;
            gd.n_in = EF;
            gd.segments = s->moe_segments;
            gd.max_segments = s->moe_max_segments;
            s->launches += launch_gemm_tiled_grouped(m->dev, st, gd);
            // shared expert: dense
            mark(s, YUUKA_OP_GEMM);
            if (L.sh_gate_up.present()) {
                gemm(s, L.sh_gate_up, s->xn, H, s->prep_xn, s->sh_gu, 2 * SF, R, 0);
            } else {
                gemm(s, L.sh_gate, s->xn, H, s->prep_xn, s->sh_gu, 2 * SF, R, 0);
                gemm(s, L.sh_up, s->xn, H, s->prep_xn, s->sh_gu + SF, 2 * SF, R, 0);
            }
            mark(s, YUUKA_OP_SILU_MUL);
            launch_silu_mul(st, s->sh_act, SF, s->sh_gu, s->sh_gu + SF, 2 * SF, SF, R, s->prep_sh_act);
            s->launches++;
            gemm(s, L.sh_down, s->sh_act, SF, s->prep_sh_act, s->sh_y, H, R, 0);
            mark(s, YUUKA_OP_MOE_COMBINE);
            launch_moe_combine(st, s->x, s->moe_y, s->sh_y, s->moe_pos, s->moe_w, s->moe_sg, H, U, R);
            s->launches++;
            if (next_norm) {
                mark(s, YUUKA_OP_RMSNORM);
                launch_rmsnorm(st, s->xn, H, s->x, H, next_norm, H, R, c.rms_eps, s->prep_xn);
                s->launches++;
            }
            continue;
        }
        // forwardFFN (model/qwen35/forward.go:295-315); its input norm came with the mixer's output GEMM
        if (L.gate_up.present() && L.gate_up.paired && L.gate_up.tiled && L.ffn_down.tiled && s->fold_swiglu && R <= 32) {
            // silu(gate) * up leaves the GEMM's epilogue in the form the down projection reads
            gemm(s, L.gate_up, s->xn, H, s->prep_xn, s->gate_up, 2 * F, R, 0, nullptr, &s->prep_act);
        } else {
            const bool paired = L.gate_up.present() && L.gate_up.paired;
            if (L.gate_up.present()) {
                gemm(s, L.gate_up, s->xn, H, s->prep_xn, s->gate_up, 2 * F, R, 0);
            } else {
                gemm(s, L.ffn_gate, s->xn, H, s->prep_xn, s->gate_up, 2 * F, R, 0);
                gemm(s, L.ffn_up, s->xn, H, s->prep_xn, s->gate_up + F, 2 * F, R, 0);
            }
            mark(s, YUUKA_OP_SILU_MUL);
            launch_silu_mul(st, s->act, F, s->gate_up, s->gate_up + (paired ? 16 : F), 2 * F, F, R, s->prep_act, paired ? 32 : 16);
            s->launches++;
        }
        gemm_residual_norm(s, L.ffn_down, s->act, F, s->prep_act, R, next_norm);
    }
    // tail: final norm + LM head over the wanted rows (forward.go:147-151)
    if (logit_rows == LOGITS_ALL) {
        gemm(s, m->output, s->xn, H, s->prep_xn, s->logits, c.vocab, R, 0);
    } else if (logit_rows == LOGITS_LAST) {
        // batch == 1: only the last row
        mark(s, YUUKA_OP_RMSNORM);
        launch_rmsnorm(st, s->xn, H, s->x + (int64_t)(R - 1) * H, H, m->output_norm, H, 1, c.rms_eps, s->prep_xn);
        s->xn_raw = false;
        s->launches++;
        gemm(s, m->output, s->xn, H, s->prep_xn, s->logits + (int64_t)(R - 1) * c.vocab, c.vocab, 1, 0);
    }
    // acceptance + commit
    if (mode == YUUKA_ACCEPT_NONE) return;
    mark(s, YUUKA_OP_ACCEPT);
    if (mode == YUUKA_ACCEPT_GREEDY) {
        s->launches += launch_accept_greedy(st, s->logits, c.vocab, rows, s->argmax, s->acc);
    } else if (mode == YUUKA_ACCEPT_REJECTION) {
        s->launches += launch_accept_rejection(st, s->logits, s->st_draft_probs, s->d_uniforms, s->reject_residual, c.vocab,
                                               s->st_temperature, rows, s->acc);
    } else {
        launch_accept_all(st, rows, s->acc);  // forced commit of a chain
        s->launches++;
    }
    mark(s, YUUKA_OP_COMMIT);
    if (sub > 0) {
        // every layer committed its own sub-chunks; a chain's K/V rows already sit at their final positions
        launch_advance_positions(st, s->d_pos0 + seq0, s->acc, batch);
        s->launches++;
        return;
    }
    if (!s->gdn_layers.empty()) {
        launch_gdn_commit(st, s->d_gdn_commit, (int)s->gdn_layers.size(), c.group_count, rank, S, c.conv_kernel, conv_dim,
                          seq0, rows, s->acc);
        s->launches++;
    }
    if (!s->attn_layers.empty()) {
        KvPool geom{};
        geom.block_size = s->cfg.block_size;
        geom.row_bytes = s->kv_row_bytes;
        geom.tables = s->d_tables + (int64_t)seq0 * s->table_stride;
        geom.table_stride = s->table_stride;
        launch_kv_commit(st, s->d_kv_commit, (int)s->attn_layers.size(), geom, rows, s->acc);
        s->launches++;
    }
    launch_advance_positions(st, s->d_pos0 + seq0, s->acc, batch, rows.seq_map);
    s->launches++;
}

}  // namespace

// ===========================================================================
// session ABI

namespace {

void check_seq(const yuuka_session * s, int seq) {
    YK_REQUIRE(s, YUUKA_ERR_INVALID_ARGUMENT, "null session");
    YK_REQUIRE(seq >= 0 && seq < s->cfg.max_batch, YUUKA_ERR_INVALID_ARGUMENT, "sequence %d is outside 0..%d", seq,
               s->cfg.max_batch - 1);
}

void sync_and_check(yuuka_session * s) {
    YK_CUDA(cudaStreamSynchronize(s->stream.s));
    int err = read_device_error(s->model->dev);
    if (err != 0) clear_device_error(s->model->dev);  // reported once; later steps are judged on their own
    YK_REQUIRE(err == 0, YUUKA_ERR_DEVICE, "a bounded wait inside a kernel expired (code %d); results are invalid", err);
}

// bytes of the per-step metadata block: ancestor masks, tokens, parents, depths of `cap` rows, the sub-chunk
// positions and acceptances of a wide prompt pass, and the slot -> sequence map
size_t rows_block_bytes(int cap, int max_batch) {
    return (size_t)cap * 20 + 2 * CHAIN_MAX_SUBS * sizeof(int32_t) + (size_t)max_batch * sizeof(int32_t);
}

// Uploads row metadata of a step: tokens, parents, depths, ancestor masks.
// sub > 0 (one sequence, a chain): the rows are a wide prompt pass whose mixers run in sub-chunks of `sub`
// rows; parents, depths and ancestor masks then restart at every sub-chunk, and the sub-chunks' first
// positions and forced acceptances go along.
void stage_rows(yuuka_session * s, int seq0, int batch, int nodes, const int32_t * tokens, const int32_t * parent,
                int sub = 0, const int32_t * seq_ids = nullptr) {
    const int vocab = s->model->cfg.vocab;
    const int R = batch * nodes, cap = s->rows_cap;
    YK_REQUIRE(R <= cap, YUUKA_ERR_INTERNAL, "stage_rows: %d rows exceed the session's %d", R, cap);
    // the previous copy out of the page-locked mirror has completed: every step is synchronized before the next is staged
    uint64_t * anc = reinterpret_cast<uint64_t *>(s->h_rows);
    int32_t * tok = reinterpret_cast<int32_t *>(s->h_rows + (size_t)cap * 8);
    int32_t * par = tok + cap;
    int32_t * dep = par + cap;
    s->st_chains = 1;
    for (int b = 0; b < batch; b++) {
        for (int i = 0; i < nodes; i++) {
            const int r = b * nodes + i;
            YK_REQUIRE(tokens[r] >= 0 && tokens[r] < vocab, YUUKA_ERR_INVALID_ARGUMENT, "token id %d is out of range",
                       tokens[r]);
            tok[r] = tokens[r];
            if (sub > 0) {
                const int j = i % sub;
                par[r] = j - 1;
                dep[r] = j;
                anc[r] = j == 63 ? ~0ull : ((1ull << (j + 1)) - 1);
                continue;
            }
            int p = parent ? parent[r] : i - 1;
            YK_REQUIRE((i == 0 && p == -1) || (i > 0 && p >= 0 && p < i), YUUKA_ERR_INVALID_ARGUMENT,
                       "parent[%d][%d] = %d is not a preceding row", b, i, p);
            if (p != i - 1) s->st_chains = 0;
            par[r] = p;
            dep[r] = i == 0 ? 0 : dep[b * nodes + p] + 1;
            anc[r] = (i == 0 ? 0ull : anc[b * nodes + p]) | (1ull << i);
        }
        const int sq = seq_ids ? seq_ids[b] : seq0 + b;
        YK_REQUIRE(s->h_pos_upper[sq] + nodes <= s->cfg.capacity, YUUKA_ERR_INVALID_ARGUMENT,
                   "token sequence of %d exceeds remaining context %d", nodes, s->cfg.capacity - s->h_pos_upper[sq]);
    }
    int32_t * pos_sub = reinterpret_cast<int32_t *>(s->h_rows + (size_t)cap * 20);
    int32_t * acc_sub = pos_sub + CHAIN_MAX_SUBS;
    for (int k = 0; k < CHAIN_MAX_SUBS; k++) {
        const int left = sub > 0 ? nodes - k * sub : 0;
        pos_sub[k] = sub > 0 ? s->h_pos[seq0] + k * sub : 0;
        acc_sub[k] = (left > sub ? sub : (left > 0 ? left : 1)) - 1;
    }
    int32_t * seq_map = acc_sub + CHAIN_MAX_SUBS;
    for (int b = 0; b < s->cfg.max_batch; b++) seq_map[b] = b < batch ? (seq_ids ? seq_ids[b] : seq0 + b) : 0;
    // one copy for the whole block (the arrays keep their capacity-sized offsets on both sides)
    YK_CUDA(cudaMemcpyAsync(s->d_rows, s->h_rows, rows_block_bytes(cap, s->cfg.max_batch), cudaMemcpyHostToDevice, s->stream.s));
}

// Key-range bound used to size the attention grid. It is the session capacity,
// not the current positions, so that a captured step stays valid as sequences grow;
// CTAs whose key range is empty return at once.
int max_total_keys(const yuuka_session * s, int seq0, int batch, int nodes) {
    (void)seq0; (void)batch; (void)nodes;
    return s->cfg.capacity;
}

// Runs tokens of one sequence as committed chain chunks (Forward / PrefillLogits).
void run_chain(yuuka_session * s, int seq, const int32_t * tokens, int n, float * all_logits, float * last_logits) {
    check_seq(s, seq);
    YK_REQUIRE(tokens && n > 0, YUUKA_ERR_INVALID_ARGUMENT, "empty token sequence");
    YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "a launched verify step has not been fetched");
    YK_REQUIRE(s->h_pos[seq] + n <= s->cfg.capacity, YUUKA_ERR_INVALID_ARGUMENT,
               "token sequence of %d exceeds remaining context %d", n, s->cfg.capacity - s->h_pos[seq]);
    YK_REQUIRE(!(all_logits || last_logits) || s->logits, YUUKA_ERR_INVALID_ARGUMENT,
               "the session was created without want_logits");
    set_device(s->model->dev);
    const int V = s->model->cfg.vocab;
    for (int done = 0; done < n;) {
        const int chunk = n - done < s->chain_rows ? n - done : s->chain_rows;
        const bool last = done + chunk == n;
        const int sub = chunk > CHAIN_SUB ? CHAIN_SUB : 0;
        stage_rows(s, seq, 1, chunk, tokens + done, nullptr, sub);
        LogitRows lr = all_logits ? LOGITS_ALL : (last && last_logits ? LOGITS_LAST : LOGITS_NONE);
        s->launches = 0;
        run_step(s, seq, 1, chunk, 3u /* forced commit */, lr, s->cfg.capacity, sub);
        sync_and_check(s);
        if (all_logits)
            YK_CUDA(cudaMemcpy(all_logits + (int64_t)done * V, s->logits, sizeof(float) * (size_t)chunk * V,
                               cudaMemcpyDeviceToHost));
        if (last && last_logits)
            YK_CUDA(cudaMemcpy(last_logits, s->logits + (int64_t)(chunk - 1) * V, sizeof(float) * (size_t)V,
                               cudaMemcpyDeviceToHost));
        s->h_pos[seq] += chunk;
        s->h_pos_upper[seq] = s->h_pos[seq];
        done += chunk;
    }
}

void validate_batch(const yuuka_session * s, const yuuka_verify_batch * b) {
    YK_REQUIRE(s && b, YUUKA_ERR_INVALID_ARGUMENT, "verify: null argument");
    YK_REQUIRE(b->batch > 0 && b->batch <= s->cfg.max_batch, YUUKA_ERR_INVALID_ARGUMENT,
               "verify: batch %d is outside 1..%d", b->batch, s->cfg.max_batch);
    YK_REQUIRE(b->nodes > 0 && b->nodes <= s->cfg.max_nodes, YUUKA_ERR_INVALID_ARGUMENT,
               "verify: %d rows per sequence is outside 1..%d", b->nodes, s->cfg.max_nodes);
    YK_REQUIRE(b->tokens, YUUKA_ERR_INVALID_ARGUMENT, "verify: tokens is null");
    if (b->seq_ids) {
        std::vector<char> seen((size_t)s->cfg.max_batch, 0);
        for (int i = 0; i < b->batch; i++) {
            const int sq = b->seq_ids[i];
            YK_REQUIRE(sq >= 0 && sq < s->cfg.max_batch, YUUKA_ERR_INVALID_ARGUMENT, "verify: sequence %d is outside 0..%d", sq,
                       s->cfg.max_batch - 1);
            YK_REQUIRE(!seen[(size_t)sq], YUUKA_ERR_INVALID_ARGUMENT, "verify: sequence %d appears twice in the batch", sq);
            seen[(size_t)sq] = 1;
        }
    }
    YK_REQUIRE(b->mode == YUUKA_ACCEPT_GREEDY || b->mode == YUUKA_ACCEPT_NONE || b->mode == YUUKA_ACCEPT_REJECTION,
               YUUKA_ERR_INVALID_ARGUMENT, "verify: unknown acceptance mode %u", b->mode);
    if (b->mode == YUUKA_ACCEPT_REJECTION) {
        const uint64_t need = (uint64_t)b->batch * b->nodes * s->model->cfg.vocab * sizeof(float);
        YK_REQUIRE(b->temperature > 0.0f && b->temperature == b->temperature, YUUKA_ERR_INVALID_ARGUMENT,
                   "verify: rejection sampling needs a temperature above zero");
        YK_REQUIRE(b->uniforms, YUUKA_ERR_INVALID_ARGUMENT, "verify: rejection sampling needs the uniform draws");
        YK_REQUIRE(b->draft_probs && b->draft_probs->ptr && b->draft_probs->bytes >= need, YUUKA_ERR_INVALID_ARGUMENT,
                   "verify: draft_probs must be a device buffer of at least %llu bytes", (unsigned long long)need);
        YK_REQUIRE(b->draft_probs->dev == s->model->dev, YUUKA_ERR_INVALID_ARGUMENT,
                   "verify: draft_probs lives on another device");
    }
    YK_REQUIRE(s->logits, YUUKA_ERR_INVALID_ARGUMENT, "verify: the session has no logits buffer");
}

// Enqueues the kernels of the staged step on the session stream: by graph replay (captured at the first step
// of a shape), or directly for a rejection step, which carries a temperature and a buffer address that a
// replayed graph would freeze.
void enqueue_staged_step(yuuka_session * s) {
    const int max_total = max_total_keys(s, s->st_seq0, s->st_batch, s->st_nodes);
    if (!s->use_graphs || s->st_mode == YUUKA_ACCEPT_REJECTION) {
        s->launches = 0;
        run_step(s, s->st_seq0, s->st_batch, s->st_nodes, s->st_mode, LOGITS_ALL, max_total, 0, true);
        return;
    }
    yuuka_session::StepGraph * gr = nullptr;
    for (size_t i = 0; i < s->graphs.size(); i++) {
        const auto & g = s->graphs[i];
        if (g.seq0 == s->st_seq0 && g.batch == s->st_batch && g.nodes == s->st_nodes && g.chains == s->st_chains && g.mode == s->st_mode) {
            std::rotate(s->graphs.begin() + (std::ptrdiff_t)i, s->graphs.begin() + (std::ptrdiff_t)i + 1, s->graphs.end());
            gr = &s->graphs.back();
            break;
        }
    }
    if (!gr) {
        // first step of this shape: capture the kernel sequence once, replay it afterwards
        s->launches = 0;
        YK_CUDA(cudaStreamBeginCapture(s->stream.s, cudaStreamCaptureModeThreadLocal));
        cudaGraph_t graph = nullptr;
        try {
            run_step(s, s->st_seq0, s->st_batch, s->st_nodes, s->st_mode, LOGITS_ALL, max_total, 0, true);
        } catch (...) {
            cudaStreamEndCapture(s->stream.s, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        YK_CUDA(cudaStreamEndCapture(s->stream.s, &graph));
        cudaGraphExec_t exec = nullptr;
        cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        YK_CUDA(err);
        if (s->graphs.size() >= yuuka_session::MAX_STEP_GRAPHS) {
            // no replay of it is in flight: a new shape is captured only behind a synchronization (the fetch of the
            // step before it, or the prompt pass of a device-drafted generation)
            cudaGraphExecDestroy(s->graphs.front().exec);
            s->graphs.erase(s->graphs.begin());
        }
        s->graphs.push_back({s->st_seq0, s->st_batch, s->st_nodes, s->st_chains, s->st_mode, exec, s->launches});
        gr = &s->graphs.back();
    }
    s->launches = gr->launches;
    YK_CUDA(cudaGraphLaunch(gr->exec, s->stream.s));
}

}  // namespace

extern "C" {

yuuka_status yuuka_session_create(yuuka_model * model, const yuuka_session_config * cfg, yuuka_session ** out) {
    return guard([&] {
        YK_REQUIRE(model && cfg && out, YUUKA_ERR_INVALID_ARGUMENT, "session_create: null argument");
        *out = nullptr;
        YK_REQUIRE(model->finalized, YUUKA_ERR_INVALID_ARGUMENT, "session_create: model is not finalized");
        const yuuka_model_config & c = model->cfg;
        yuuka_session_config sc = *cfg;
        YK_REQUIRE(sc.max_batch > 0 && sc.max_batch <= 4096, YUUKA_ERR_INVALID_ARGUMENT, "invalid max_batch %d", sc.max_batch);
        YK_REQUIRE(sc.max_nodes > 0 && sc.max_nodes <= 64, YUUKA_ERR_INVALID_ARGUMENT, "max_nodes %d is outside 1..64",
                   sc.max_nodes);
        YK_REQUIRE(sc.capacity > 0, YUUKA_ERR_INVALID_ARGUMENT, "context capacity must be positive");
        YK_REQUIRE(sc.capacity <= c.context_length, YUUKA_ERR_INVALID_ARGUMENT,
                   "context capacity %d exceeds model limit %d", sc.capacity, c.context_length);
        if (sc.block_size <= 0) sc.block_size = sc.capacity < 16 ? sc.capacity : 16;  // state.go:68-72
        const int per_seq = (sc.capacity + sc.block_size - 1) / sc.block_size;
        if (sc.pool_blocks <= 0) sc.pool_blocks = per_seq * sc.max_batch;
        YK_REQUIRE(sc.kv_format == YUUKA_KV_F32 || sc.kv_format == YUUKA_KV_F16 || sc.kv_format == YUUKA_KV_Q8_0,
                   YUUKA_ERR_INVALID_ARGUMENT, "unknown KV format %d", sc.kv_format);
        YK_REQUIRE((sc.flags & ~(YUUKA_SESSION_EXACT_WIDE | YUUKA_SESSION_WIDE_FROM_33 | YUUKA_SESSION_TEST_DROP_COPIES)) == 0, YUUKA_ERR_INVALID_ARGUMENT,
                   "unknown session flags 0x%x", sc.flags);
        set_device(model->dev);
        auto * s = new yuuka_session();
        try {
            s->model = model;
            s->cfg = sc;
            if (const char * e = getenv("YUUKA_CUDA_NO_GRAPH")) s->use_graphs = !(e[0] == '1');
            {
                // norm folding needs every matrix on either side of a norm in the tile-ordered form
                bool ok = c.expert_count == 0 && c.hidden % 16 == 0 && model->output.tiled;
                for (int i = 0; i < c.block_count && ok; i++) {
                    const LayerW & L = model->layers[i];
                    if (model->recurrent(i)) ok = L.proj.tiled && L.out.tiled;
                    else ok = L.qk.tiled && (L.qk_has_v || L.v.tiled) && L.o.tiled;
                    ok = ok && L.gate_up.tiled && L.ffn_down.tiled;
                }
                if (const char * e = getenv("YUUKA_CUDA_NO_FOLD_NORM")) ok = ok && !(e[0] == '1');
                s->fold_norm = ok;
                if (ok) s->norm_sumsq = dalloc<unsigned long long>((size_t)32 * (2 * c.block_count + 2), s->owned);
            }
            if (const char * e = getenv("YUUKA_CUDA_NO_FOLD_SWIGLU")) s->fold_swiglu = !(e[0] == '1');
            if (const char * e = getenv("YUUKA_CUDA_NO_PREFETCH")) s->prefetch_next = !(e[0] == '1');
            if (const char * e = getenv("YUUKA_CUDA_NO_GDN_CHUNK")) s->gdn_chunked = !(e[0] == '1');
            for (const LayerW & L : model->layers) {
                for (const Tensor * t : {&L.proj, &L.qkv, &L.gate, &L.beta, &L.alpha, &L.out, &L.qk, &L.q, &L.k, &L.v, &L.o,
                                         &L.gate_up, &L.ffn_gate, &L.ffn_up, &L.ffn_down})
                    if (t->present() && t->tiled) s->gemm_order.push_back({t->ptr, t->bytes});
            }
            if (model->output.tiled) s->gemm_order.push_back({model->output.ptr, model->output.bytes});
            s->stream.dev = model->dev;
            YK_CUDA(cudaStreamCreateWithFlags(&s->stream.s, cudaStreamNonBlocking));
            const int kv_dim = model->kv_dim();
            s->kv_row_bytes = sc.kv_format == YUUKA_KV_F32 ? kv_dim * 4 : (sc.kv_format == YUUKA_KV_F16 ? kv_dim * 2 : (kv_dim + 31) / 32 * 34);
            s->table_stride = per_seq;
            // row buffers hold a verify step (max_batch x max_nodes rows) or one prompt chunk of chain_rows rows
            const int B = sc.max_batch, N = sc.max_nodes;
            s->chain_rows = CHAIN_ROWS < sc.capacity ? CHAIN_ROWS : sc.capacity;
            if (s->chain_rows < N) s->chain_rows = N;
            const int R = B * N > s->chain_rows ? B * N : s->chain_rows;
            const int conv_dim = model->conv_dim(), K1 = c.conv_kernel - 1, S = c.state_size, rank = c.time_step_rank;
            s->conv_count = (int64_t)conv_dim * K1;
            s->s_count = (int64_t)rank * S * S;
            s->n_proj = conv_dim + c.inner_size + 2 * rank;
            s->n_qkv = model->q_dim() + 2 * kv_dim;
            s->layers.resize(c.block_count);
            const size_t pool_bytes = (size_t)sc.pool_blocks * sc.block_size * s->kv_row_bytes;
            std::vector<GdnLayerCommit> gc;
            std::vector<KvLayerCommit> kc;
            for (int i = 0; i < c.block_count; i++) {
                LayerState & LS = s->layers[i];
                if (model->recurrent(i)) {
                    LS.conv_state = dalloc<float>((size_t)B * s->conv_count, s->owned);
                    LS.state = dalloc<float>((size_t)B * s->s_count, s->owned);
                    LS.proj = dalloc<float>((size_t)R * s->n_proj, s->owned);
                    LS.khat = dalloc<float>((size_t)R * c.group_count * S, s->owned);
                    LS.dlog = dalloc<float>((size_t)R * c.inner_size, s->owned);
                    LS.decay = dalloc<float>((size_t)R * rank, s->owned);
                    s->gdn_layers.push_back(i);
                    gc.push_back(GdnLayerCommit{LS.proj, s->n_proj, LS.khat, LS.dlog, LS.decay, LS.conv_state, LS.state});
                } else {
                    LS.k = dalloc<uint8_t>(pool_bytes, s->owned);
                    LS.v = dalloc<uint8_t>(pool_bytes, s->owned);
                    s->attn_layers.push_back(i);
                    kc.push_back(KvLayerCommit{LS.k, LS.v});
                }
            }
            s->d_gdn_commit = dalloc<GdnLayerCommit>(gc.size(), s->owned);
            s->d_kv_commit = dalloc<KvLayerCommit>(kc.size(), s->owned);
            if (!gc.empty()) YK_CUDA(cudaMemcpy(s->d_gdn_commit, gc.data(), gc.size() * sizeof(GdnLayerCommit), cudaMemcpyHostToDevice));
            if (!kc.empty()) YK_CUDA(cudaMemcpy(s->d_kv_commit, kc.data(), kc.size() * sizeof(KvLayerCommit), cudaMemcpyHostToDevice));
            s->d_pos0 = dalloc<int32_t>(B, s->owned);
            s->d_tables = dalloc<int32_t>((size_t)B * per_seq, s->owned);
            std::vector<int32_t> ident((size_t)B * per_seq);
            for (int b = 0; b < B; b++)
                for (int j = 0; j < per_seq; j++) ident[(size_t)b * per_seq + j] = (b * per_seq + j) % sc.pool_blocks;
            YK_CUDA(cudaMemcpy(s->d_tables, ident.data(), ident.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
            s->h_pos.assign(B, 0);
            s->h_pos_upper.assign(B, 0);
            s->rows_cap = R;
            s->d_rows = dalloc<uint8_t>(rows_block_bytes(R, B), s->owned);
            s->d_pos_sub = reinterpret_cast<int32_t *>(s->d_rows + (size_t)R * 20);
            s->d_acc_sub = s->d_pos_sub + CHAIN_MAX_SUBS;
            s->d_seq_map = s->d_acc_sub + CHAIN_MAX_SUBS;
            s->d_anc = reinterpret_cast<uint64_t *>(s->d_rows);
            s->d_tokens = reinterpret_cast<int32_t *>(s->d_rows + (size_t)R * 8);
            s->d_parent = s->d_tokens + R;
            s->d_depth = s->d_parent + R;
            {
                void * hp = nullptr;
                const size_t rows_bytes = rows_block_bytes(R, B);
                YK_REQUIRE(cudaMallocHost(&hp, rows_bytes + sizeof(int32_t) * ((size_t)B + 2 * R + 2)) == cudaSuccess,
                           YUUKA_ERR_ALLOCATION, "page-locked staging allocation failed");
                s->h_rows = (uint8_t *)hp;
                s->h_results = reinterpret_cast<int32_t *>(s->h_rows + rows_bytes);
            }
            const int H = c.hidden;
            s->x = dalloc<float>((size_t)R * H, s->owned);
            s->xn = dalloc<float>((size_t)R * H, s->owned);
            s->qkv_attn = dalloc<float>((size_t)R * s->n_qkv, s->owned);
            s->attn_out = dalloc<float>((size_t)R * model->o_dim(), s->owned);
            s->gdn_out = dalloc<float>((size_t)R * c.inner_size, s->owned);
            s->gdn_qn = dalloc<float>((size_t)R * c.group_count * S, s->owned);
            s->gdn_vconv = dalloc<float>((size_t)R * c.inner_size, s->owned);
            s->gdn_beta = dalloc<float>((size_t)R * rank, s->owned);
            s->gate_up = dalloc<float>((size_t)R * 2 * c.ffn, s->owned);
            if (c.rope_dim > 0) s->rope_cs = dalloc<float2>((size_t)R * (c.rope_dim / 2), s->owned);
            s->act = dalloc<float>((size_t)R * c.ffn, s->owned);
            auto prep_alloc = [&](int width) {
                XPrepOut o;
                if (width % 16 == 0) {
                    o.xh = dalloc<__half>((size_t)R * width, s->owned);
                    o.xl = dalloc<__half>((size_t)R * width, s->owned);
                    o.xs16 = dalloc<__half2>((size_t)R * (width / 16) + 4, s->owned);
                }
                return o;
            };
            s->prep_xn = prep_alloc(H);
            s->prep_attn = prep_alloc(model->o_dim());
            s->prep_gdn = prep_alloc(c.inner_size);
            s->prep_act = prep_alloc(c.ffn);
            if (c.expert_count > 0) {
                const size_t P = (size_t)R * c.expert_used;
                s->moe_ids = dalloc<int32_t>(P, s->owned);
                s->moe_pos = dalloc<int32_t>(P, s->owned);
                s->moe_row = dalloc<int32_t>(P, s->owned);
                s->moe_w = dalloc<float>(P, s->owned);
                s->moe_sg = dalloc<float>(R, s->owned);
                s->moe_logits = dalloc<float>((size_t)R * c.expert_count, s->owned);
                s->moe_counters = dalloc<int>((size_t)R / 8 + 1, s->owned);
                s->moe_gu = dalloc<float>(P * 2 * c.expert_ffn, s->owned);
                s->moe_act = dalloc<float>(P * c.expert_ffn, s->owned);
                s->moe_y = dalloc<float>(P * H, s->owned);
                s->sh_gu = dalloc<float>((size_t)R * 2 * c.shared_ffn, s->owned);
                s->sh_act = dalloc<float>((size_t)R * c.shared_ffn, s->owned);
                s->sh_y = dalloc<float>((size_t)R * H, s->owned);
                s->moe_max_segments = moe_max_segments((int)P, c.expert_count);
                s->moe_segments = dalloc<GemmSegment>((size_t)s->moe_max_segments, s->owned);
                YK_REQUIRE(c.expert_ffn % 16 == 0 && c.shared_ffn % 16 == 0, YUUKA_ERR_UNSUPPORTED,
                           "expert feed-forward sizes must be multiples of 16");
                s->prep_moe_act.xh = dalloc<__half>(P * c.expert_ffn, s->owned);
                s->prep_moe_act.xl = dalloc<__half>(P * c.expert_ffn, s->owned);
                s->prep_moe_act.xs16 = dalloc<__half2>(P * (c.expert_ffn / 16) + 4, s->owned);
                s->prep_sh_act.xh = dalloc<__half>((size_t)R * c.shared_ffn, s->owned);
                s->prep_sh_act.xl = dalloc<__half>((size_t)R * c.shared_ffn, s->owned);
                s->prep_sh_act.xs16 = dalloc<__half2>((size_t)R * (c.shared_ffn / 16) + 4, s->owned);
            }
            if (sc.want_logits) s->logits = dalloc<float>((size_t)R * c.vocab, s->owned);
            s->argmax.chunks = argmax_chunks(c.vocab);
            s->argmax.val = dalloc<float>((size_t)R * s->argmax.chunks, s->owned);
            s->argmax.idx = dalloc<int32_t>((size_t)R * s->argmax.chunks, s->owned);
            s->d_results = dalloc<int32_t>((size_t)B + 2 * R, s->owned);
            s->acc.accepted = s->d_results;
            s->acc.path = s->d_results + B;
            s->acc.emitted = s->acc.path + R;
            s->d_uniforms = dalloc<float>((size_t)R * 2, s->owned);
            {
                // rows x splits of the flash-decoding partials, for the verify shape and for a prompt chunk
                auto need = [&](int bx, int nx) {
                    const int G = c.heads / c.kv_heads, qt = (G * nx + 39) / 40;
                    size_t splits = (size_t)(4 * model->dev->sm_count / (c.kv_heads * qt * bx) + 2);
                    const size_t by_length = (size_t)(sc.capacity + 511) / 512 + 1;  // batched steps split the keys by length
                    if (splits < by_length) splits = by_length;
                    return (size_t)bx * nx * c.heads * splits * (size_t)(c.head_dim + 2);
                };
                const size_t a = need(B, N), b = need(1, s->chain_rows);
                s->attn_partial_floats = a > b ? a : b;
            }
            s->attn_partial = dalloc<float>(s->attn_partial_floats, s->owned, false);
            // split-K scratch for every matrix shape of the step and of a prompt pass: the register-fed route
            // (up to 32 rows per launch), one row, and the tensor-memory route at the widest pass a launch
            // takes (gemm_tiled_scratch_need covers every row count up to the one it is given)
            for (int rows : {R < 32 ? R : 32, 1, R}) {
                for (const LayerW & L : model->layers) {
                    for (const Tensor * t : {&L.q, &L.k, &L.v, &L.o, &L.qkv, &L.gate, &L.beta, &L.alpha, &L.out, &L.ffn_gate,
                                             &L.ffn_up, &L.ffn_down, &L.proj, &L.qk, &L.gate_up, &L.sh_gate, &L.sh_up,
                                             &L.sh_down, &L.sh_gate_up})
                        reserve_gemm(s, *t, rows);
                }
                reserve_gemm(s, model->output, rows);
            }
            for (int r = 1; r < R && r < 32; r++) reserve_gemm(s, model->layers[0].ffn_down, r);
            for (int r = 1; r < R && r < 32; r++) reserve_gemm(s, model->layers[0].sh_down, r);
        } catch (...) {
            yuuka_session_destroy(s);
            throw;
        }
        *out = s;
    });
}

void yuuka_session_destroy(yuuka_session * s) {
    if (!s) return;
    cudaSetDevice(s->model->dev->index);
    if (s->stream.s) {
        cudaStreamSynchronize(s->stream.s);
        cudaStreamDestroy(s->stream.s);
    }
    for (auto & g : s->graphs) cudaGraphExecDestroy(g.exec);
    for (void * p : s->owned) cudaFree(p);
    if (s->h_rows) cudaFreeHost(s->h_rows);
    gemm_scratch_free(s->gemm);
    delete s;
}

yuuka_status yuuka_session_set_block_table(yuuka_session * s, int32_t seq, const int32_t * blocks, int32_t count) {
    return guard([&] {
        check_seq(s, seq);
        YK_REQUIRE(blocks && count >= s->table_stride, YUUKA_ERR_INVALID_ARGUMENT,
                   "block table maps %d positions, need %d", count * s->cfg.block_size, s->cfg.capacity);
        for (int i = 0; i < s->table_stride; i++)
            YK_REQUIRE(blocks[i] >= 0 && blocks[i] < s->cfg.pool_blocks, YUUKA_ERR_INVALID_ARGUMENT,
                       "block %d is outside the KV pool", blocks[i]);
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        YK_CUDA(cudaMemcpy(s->d_tables + (int64_t)seq * s->table_stride, blocks, sizeof(int32_t) * s->table_stride,
                           cudaMemcpyHostToDevice));
    });
}

yuuka_status yuuka_session_set_flags(yuuka_session * s, uint32_t flags) {
    return guard([&] {
        YK_REQUIRE(s, YUUKA_ERR_INVALID_ARGUMENT, "null session");
        YK_REQUIRE((flags & ~(YUUKA_SESSION_EXACT_WIDE | YUUKA_SESSION_WIDE_FROM_33 | YUUKA_SESSION_TEST_DROP_COPIES)) == 0, YUUKA_ERR_INVALID_ARGUMENT,
                   "unknown session flags 0x%x", flags);
        YK_REQUIRE(!s->staged && !s->launched, YUUKA_ERR_INVALID_ARGUMENT, "set_flags: a step is staged or in flight");
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        for (auto & g : s->graphs) cudaGraphExecDestroy(g.exec);
        s->graphs.clear();
        s->cfg.flags = flags;
    });
}

yuuka_status yuuka_session_copy_block(yuuka_session * s, int32_t dst_block, int32_t src_block) {
    return guard([&] {
        YK_REQUIRE(s, YUUKA_ERR_INVALID_ARGUMENT, "null session");
        YK_REQUIRE(dst_block >= 0 && dst_block < s->cfg.pool_blocks && src_block >= 0 && src_block < s->cfg.pool_blocks,
                   YUUKA_ERR_INVALID_ARGUMENT, "copy_block: block %d or %d is outside the KV pool of %d blocks", dst_block, src_block,
                   s->cfg.pool_blocks);
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "copy_block: a launched verify step has not been fetched");
        if (dst_block == src_block) return;
        set_device(s->model->dev);
        const size_t bytes = (size_t)s->cfg.block_size * s->kv_row_bytes;
        for (int i : s->attn_layers) {
            YK_CUDA(cudaMemcpyAsync(s->layers[i].k + (size_t)dst_block * bytes, s->layers[i].k + (size_t)src_block * bytes, bytes,
                                    cudaMemcpyDeviceToDevice, s->stream.s));
            YK_CUDA(cudaMemcpyAsync(s->layers[i].v + (size_t)dst_block * bytes, s->layers[i].v + (size_t)src_block * bytes, bytes,
                                    cudaMemcpyDeviceToDevice, s->stream.s));
        }
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
    });
}

yuuka_status yuuka_session_reset(yuuka_session * s, int32_t seq) {
    return guard([&] {
        check_seq(s, seq);
        // (the fetch of a launched step adds what it accepted to the host's copy of the positions)
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "session_reset: a launched verify step has not been fetched");
        set_device(s->model->dev);
        cudaStream_t st = s->stream.s;
        for (int i : s->gdn_layers) {
            YK_CUDA(cudaMemsetAsync(s->layers[i].conv_state + (int64_t)seq * s->conv_count, 0, s->conv_count * 4, st));
            YK_CUDA(cudaMemsetAsync(s->layers[i].state + (int64_t)seq * s->s_count, 0, s->s_count * 4, st));
        }
        YK_CUDA(cudaMemsetAsync(s->d_pos0 + seq, 0, sizeof(int32_t), st));
        YK_CUDA(cudaStreamSynchronize(st));
        s->h_pos[seq] = s->h_pos_upper[seq] = 0;
    });
}

yuuka_status yuuka_session_set_position(yuuka_session * s, int32_t seq, int32_t position) {
    return guard([&] {
        check_seq(s, seq);
        YK_REQUIRE(position >= 0 && position <= s->cfg.capacity, YUUKA_ERR_INVALID_ARGUMENT,
                   "position %d exceeds capacity %d", position, s->cfg.capacity);
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "session_set_position: a launched verify step has not been fetched");
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        YK_CUDA(cudaMemcpy(s->d_pos0 + seq, &position, sizeof(int32_t), cudaMemcpyHostToDevice));
        s->h_pos[seq] = s->h_pos_upper[seq] = position;
    });
}

yuuka_status yuuka_session_info_get(const yuuka_session * s, yuuka_session_info * out) {
    return guard([&] {
        YK_REQUIRE(s && out, YUUKA_ERR_INVALID_ARGUMENT, "session_info_get: null argument");
        out->max_batch = s->cfg.max_batch;
        out->max_nodes = s->cfg.max_nodes;
        out->capacity = s->cfg.capacity;
        out->block_size = s->cfg.block_size;
        out->pool_blocks = s->cfg.pool_blocks;
        out->kv_format = s->cfg.kv_format;
        out->vocab = s->model->cfg.vocab;
    });
}

yuuka_status yuuka_session_position(yuuka_session * s, int32_t seq, int32_t * position) {
    return guard([&] {
        check_seq(s, seq);
        YK_REQUIRE(position, YUUKA_ERR_INVALID_ARGUMENT, "session_position: null output");
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        YK_CUDA(cudaMemcpy(position, s->d_pos0 + seq, sizeof(int32_t), cudaMemcpyDeviceToHost));
    });
}

uint64_t yuuka_session_snapshot_bytes(const yuuka_session * s) {
    return s ? (uint64_t)s->gdn_layers.size() * (uint64_t)(s->conv_count + s->s_count) * 4 : 0;
}

yuuka_status yuuka_session_snapshot(yuuka_session * s, int32_t seq, void * dst, uint64_t bytes) {
    return guard([&] {
        check_seq(s, seq);
        YK_REQUIRE(dst && bytes == yuuka_session_snapshot_bytes(s), YUUKA_ERR_INVALID_ARGUMENT,
                   "state snapshot is %llu bytes, want %llu", (unsigned long long)bytes,
                   (unsigned long long)yuuka_session_snapshot_bytes(s));
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        uint8_t * o = (uint8_t *)dst;
        for (int i : s->gdn_layers) {
            YK_CUDA(cudaMemcpy(o, s->layers[i].conv_state + (int64_t)seq * s->conv_count, s->conv_count * 4, cudaMemcpyDeviceToHost));
            o += s->conv_count * 4;
            YK_CUDA(cudaMemcpy(o, s->layers[i].state + (int64_t)seq * s->s_count, s->s_count * 4, cudaMemcpyDeviceToHost));
            o += s->s_count * 4;
        }
    });
}

yuuka_status yuuka_session_restore(yuuka_session * s, int32_t seq, const void * src, uint64_t bytes) {
    return guard([&] {
        check_seq(s, seq);
        YK_REQUIRE(src && bytes == yuuka_session_snapshot_bytes(s), YUUKA_ERR_INVALID_ARGUMENT,
                   "state snapshot is %llu bytes, want %llu", (unsigned long long)bytes,
                   (unsigned long long)yuuka_session_snapshot_bytes(s));
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "session_restore: a launched verify step has not been fetched");
        set_device(s->model->dev);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        const uint8_t * o = (const uint8_t *)src;
        for (int i : s->gdn_layers) {
            YK_CUDA(cudaMemcpy(s->layers[i].conv_state + (int64_t)seq * s->conv_count, o, s->conv_count * 4, cudaMemcpyHostToDevice));
            o += s->conv_count * 4;
            YK_CUDA(cudaMemcpy(s->layers[i].state + (int64_t)seq * s->s_count, o, s->s_count * 4, cudaMemcpyHostToDevice));
            o += s->s_count * 4;
        }
    });
}

yuuka_status yuuka_session_prefill_logits(yuuka_session * s, int32_t seq, const int32_t * tokens, int32_t n,
                                          float * logits) {
    return guard([&] { run_chain(s, seq, tokens, n, logits, nullptr); });
}

yuuka_status yuuka_session_forward(yuuka_session * s, int32_t seq, const int32_t * tokens, int32_t n,
                                   float * last_logits) {
    return guard([&] { run_chain(s, seq, tokens, n, nullptr, last_logits); });
}

yuuka_status yuuka_verify_stage(yuuka_session * s, const yuuka_verify_batch * b) {
    return guard([&] {
        validate_batch(s, b);
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "verify_stage: the previous step has not been fetched");
        set_device(s->model->dev);
        // staging again before a launch replaces the step; the earlier copy out of the page-locked mirror must have left it
        if (s->staged) YK_CUDA(cudaStreamSynchronize(s->stream.s));
        s->staged = false;  // a batch refused half way through must not leave the earlier step launchable over its rows
        stage_rows(s, 0, b->batch, b->nodes, b->tokens, b->parent, 0, b->seq_ids);
        s->st_seqs.resize((size_t)b->batch);
        for (int i = 0; i < b->batch; i++) s->st_seqs[(size_t)i] = b->seq_ids ? b->seq_ids[i] : i;
        if (b->mode == YUUKA_ACCEPT_REJECTION) {
            const int V = s->model->cfg.vocab;
            if (!s->reject_residual) s->reject_residual = dalloc<unsigned long long>((size_t)s->cfg.max_batch * V, s->owned, false);
            for (int i = 0; i < b->batch * b->nodes * 2; i++)
                YK_REQUIRE(b->uniforms[i] >= 0.0f && b->uniforms[i] < 1.0f, YUUKA_ERR_INVALID_ARGUMENT,
                           "verify: uniform draw %d is outside [0, 1)", i);
            YK_CUDA(cudaMemcpyAsync(s->d_uniforms, b->uniforms, sizeof(float) * (size_t)b->batch * b->nodes * 2,
                                    cudaMemcpyHostToDevice, s->stream.s));
            YK_CUDA(cudaStreamSynchronize(s->stream.s));  // the host array may go away after this call
            s->st_draft_probs = (const float *)b->draft_probs->ptr;
            s->st_temperature = b->temperature;
        }
        s->st_seq0 = 0;
        s->st_batch = b->batch;
        s->st_nodes = b->nodes;
        s->st_mode = b->mode;
        s->staged = true;
    });
}

yuuka_status yuuka_verify_launch(yuuka_session * s, yuuka_event * completion) {
    return guard([&] {
        YK_REQUIRE(s && s->staged, YUUKA_ERR_INVALID_ARGUMENT, "verify_launch: no staged step");
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "verify_launch: the staged step is already running; fetch it first");
        set_device(s->model->dev);
        enqueue_staged_step(s);
        if (s->st_mode != YUUKA_ACCEPT_NONE)
            for (int b = 0; b < s->st_batch; b++) s->h_pos_upper[s->st_seqs[(size_t)b]] += s->st_nodes;
        s->launched = true;
        if (completion) YK_CUDA(cudaEventRecord(completion->e, s->stream.s));
    });
}

yuuka_status yuuka_verify_launch_profiled(yuuka_session * s, uint32_t * op_codes, uint64_t * op_times_ns,
                                          uint64_t capacity, uint64_t * op_count) {
    return guard([&] {
        YK_REQUIRE(s && s->staged && op_codes && op_times_ns && op_count, YUUKA_ERR_INVALID_ARGUMENT,
                   "verify_launch_profiled: null argument or no staged step");
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "verify_launch_profiled: the staged step is already running; fetch it first");
        set_device(s->model->dev);
        s->launches = 0;
        s->profiling = true;
        s->prof.clear();
        try {
            run_step(s, s->st_seq0, s->st_batch, s->st_nodes, s->st_mode, LOGITS_ALL,
                     max_total_keys(s, s->st_seq0, s->st_batch, s->st_nodes), 0, true);
            mark(s, 0);
        } catch (...) {
            s->profiling = false;
            for (auto & pe : s->prof) cudaEventDestroy(pe.second);
            s->prof.clear();
            throw;
        }
        s->profiling = false;
        if (s->st_mode != YUUKA_ACCEPT_NONE)
            for (int b = 0; b < s->st_batch; b++) s->h_pos_upper[s->st_seqs[(size_t)b]] += s->st_nodes;
        s->launched = true;
        cudaError_t err = cudaStreamSynchronize(s->stream.s);
        uint64_t n = s->prof.empty() ? 0 : s->prof.size() - 1;
        for (uint64_t i = 0; i < n && i < capacity && err == cudaSuccess; i++) {
            float ms = 0;
            err = cudaEventElapsedTime(&ms, s->prof[i].second, s->prof[i + 1].second);
            op_codes[i] = s->prof[i].first;
            op_times_ns[i] = (uint64_t)((double)ms * 1e6);
        }
        for (auto & pe : s->prof) cudaEventDestroy(pe.second);
        s->prof.clear();
        YK_CUDA(err);
        *op_count = n;
    });
}

yuuka_status yuuka_verify_fetch(yuuka_session * s, const yuuka_verify_batch * b) {
    return guard([&] {
        YK_REQUIRE(s && b && s->launched, YUUKA_ERR_INVALID_ARGUMENT, "verify_fetch: no launched step");
        YK_REQUIRE(b->batch == s->st_batch && b->nodes == s->st_nodes, YUUKA_ERR_INVALID_ARGUMENT,
                   "verify_fetch: batch shape differs from the staged step");
        set_device(s->model->dev);
        s->launched = false;
        s->staged = false;
        // results and the device error flags come back behind the step's kernels; one synchronization for all
        const int B = s->st_batch, N = s->st_nodes;
        const int maxB = s->cfg.max_batch, cap = s->rows_cap;
        int32_t * err2 = s->h_results + maxB + 2 * cap;
        if (s->st_mode != YUUKA_ACCEPT_NONE)
            YK_CUDA(cudaMemcpyAsync(s->h_results, s->d_results, sizeof(int32_t) * ((size_t)maxB + 2 * cap), cudaMemcpyDeviceToHost,
                                    s->stream.s));
        enqueue_device_error_read(s->stream.s, err2);
        YK_CUDA(cudaStreamSynchronize(s->stream.s));
        if ((err2[0] | err2[1]) != 0) clear_device_error(s->model->dev);  // reported once; later steps are judged on their own
        YK_REQUIRE((err2[0] | err2[1]) == 0, YUUKA_ERR_DEVICE, "a bounded wait inside a kernel expired (code %d); results are invalid",
                   err2[0] | err2[1]);
        const int32_t * acc = s->h_results;
        if (s->st_mode != YUUKA_ACCEPT_NONE) {
            if (b->accepted) memcpy(b->accepted, acc, sizeof(int32_t) * B);
            if (b->path) memcpy(b->path, s->h_results + maxB, sizeof(int32_t) * B * N);
            if (b->emitted) memcpy(b->emitted, s->h_results + maxB + cap, sizeof(int32_t) * B * N);
            for (int i = 0; i < B; i++) {
                const int sq = s->st_seqs[(size_t)i];
                s->h_pos[sq] += acc[i] + 1;
                s->h_pos_upper[sq] = s->h_pos[sq];
            }
        }
        if (b->logits)
            YK_CUDA(cudaMemcpy(b->logits, s->logits, sizeof(float) * (size_t)B * N * s->model->cfg.vocab, cudaMemcpyDeviceToHost));
    });
}

yuuka_status yuuka_verify_step(yuuka_session * s, const yuuka_verify_batch * b) {
    yuuka_status st = yuuka_verify_stage(s, b);
    if (st != YUUKA_OK) return st;
    st = yuuka_verify_launch(s, nullptr);
    if (st != YUUKA_OK) {
        if (s) s->staged = false;
        return st;
    }
    return yuuka_verify_fetch(s, b);
}

// generateSpeculative (engine/speculative.go:68-251) with the drafting on the device: every step has
// max_draft + 1 rows, a kernel behind each step appends what it emitted to a device-resident history, looks up
// the next draft there (lookupDraft, speculative.go:39-66) and writes the next step's token rows, so `burst`
// steps are enqueued back to back and the host synchronizes once per burst. Rows the draft does not fill
// repeat the pending token; the greedy walk accepts a row only if it is the model's own next token, so the
// emitted stream is the greedy stream whatever the rows hold. Stop tokens and max_tokens are applied by the
// host when a burst returns: the sequence may have run up to one burst past the end (its state is not
// rewound; the reference resets the state before the next request).
yuuka_status yuuka_spec_generate_device(yuuka_session * s, int32_t seq, const int32_t * prompt, int32_t n_prompt,
                                        const yuuka_spec_request * req, int32_t burst, int32_t * tokens,
                                        yuuka_spec_result * result) {
    return guard([&] {
        YK_REQUIRE(s && prompt && req && tokens && result, YUUKA_ERR_INVALID_ARGUMENT, "spec_generate_device: null argument");
        *result = yuuka_spec_result{};
        check_seq(s, seq);
        YK_REQUIRE(n_prompt > 0, YUUKA_ERR_INVALID_ARGUMENT, "prompt is empty");
        YK_REQUIRE(req->max_tokens > 0, YUUKA_ERR_INVALID_ARGUMENT, "max tokens must be positive");
        YK_REQUIRE(burst >= 1 && burst <= 64, YUUKA_ERR_INVALID_ARGUMENT, "spec_generate_device: burst %d is outside 1..64", burst);
        YK_REQUIRE(!s->launched, YUUKA_ERR_INVALID_ARGUMENT, "a launched verify step has not been fetched");
        YK_REQUIRE(s->logits, YUUKA_ERR_INVALID_ARGUMENT, "the session was created without want_logits");
        const int cap = s->cfg.capacity, V = s->model->cfg.vocab;
        YK_REQUIRE(n_prompt <= cap, YUUKA_ERR_INVALID_ARGUMENT, "prompt length %d exceeds context capacity %d", n_prompt, cap);
        const int max_tokens = req->max_tokens < cap - n_prompt ? req->max_tokens : cap - n_prompt;
        YK_REQUIRE(max_tokens > 0, YUUKA_ERR_INVALID_ARGUMENT, "no context space remains for generated tokens");
        YK_REQUIRE(req->n_stop >= 0 && (req->n_stop == 0 || req->stop_tokens), YUUKA_ERR_INVALID_ARGUMENT,
                   "spec_generate_device: stop token list is null");
        yuuka_spec_options so = req->options;
        yuuka_spec_options_normalize(&so);
        if (so.max_draft > s->cfg.max_nodes - 1) so.max_draft = s->cfg.max_nodes - 1;
        const int nodes = so.max_draft + 1;
        set_device(s->model->dev);
        cudaStream_t st = s->stream.s;
        if (!s->d_hist) {
            s->hist_cap = cap + 2;
            s->d_hist = dalloc<int32_t>((size_t)s->hist_cap, s->owned);
            s->d_hist_len = dalloc<int32_t>(1, s->owned);
            s->d_spec_stats = dalloc<int32_t>(4, s->owned);
        }
        auto is_stop = [&](int32_t t) {
            for (int i = 0; i < req->n_stop; i++)
                if (req->stop_tokens[i] == t) return true;
            return false;
        };
        result->prompt_tokens = n_prompt;
        result->finish_reason = YUUKA_FINISH_LENGTH;

        // prompt, first token (argmaxLogit, engine/speculative.go:263-271: first index of the maximum)
        if (yuuka_session_reset(s, seq) != YUUKA_OK) throw StatusError{YUUKA_ERR_DEVICE};
        std::vector<float> logits((size_t)V);
        run_chain(s, seq, prompt, n_prompt, nullptr, logits.data());
        int32_t pending = 0;
        for (int i = 1; i < V; i++)
            if (logits[(size_t)i] > logits[(size_t)pending]) pending = i;
        int n_out = 0;
        bool done = false;
        auto emit = [&](int32_t t) {
            if (is_stop(t)) {
                result->finish_reason = YUUKA_FINISH_STOP;
                return true;
            }
            tokens[n_out++] = t;
            return n_out >= max_tokens;
        };
        done = emit(pending);
        if (done) {
            result->output_tokens = n_out;
            return;
        }
        // history on the device: the prompt and the pending token
        std::vector<int32_t> hist(prompt, prompt + n_prompt);
        hist.push_back(pending);
        int hist_len = (int)hist.size();
        YK_CUDA(cudaMemcpyAsync(s->d_hist, hist.data(), hist.size() * sizeof(int32_t), cudaMemcpyHostToDevice, st));
        YK_CUDA(cudaMemcpyAsync(s->d_hist_len, &hist_len, sizeof(int32_t), cudaMemcpyHostToDevice, st));
        YK_CUDA(cudaMemsetAsync(s->d_spec_stats, 0, 4 * sizeof(int32_t), st));
        // chain metadata of a step (parents, depths, ancestor masks, the slot's sequence); the token rows are
        // written by the draft kernel
        if (s->h_pos_upper[seq] + nodes > cap) {
            // fewer than max_draft + 1 positions remain: generation ends here (the host loop would go on with
            // shorter steps)
            result->output_tokens = n_out;
            return;
        }
        std::vector<int32_t> zeros((size_t)nodes, 0);
        stage_rows(s, 0, 1, nodes, zeros.data(), nullptr, 0, &seq);
        s->st_seq0 = 0;
        s->st_batch = 1;
        s->st_nodes = nodes;
        s->st_mode = YUUKA_ACCEPT_GREEDY;
        s->st_seqs.assign(1, seq);
        DraftParams dp{};
        dp.hist = s->d_hist;
        dp.hist_len = s->d_hist_len;
        dp.hist_cap = s->hist_cap;
        dp.rows_tokens = s->d_tokens;
        dp.nodes = nodes;
        dp.max_draft = so.max_draft;
        dp.min_match = so.min_match;
        dp.stats = s->d_spec_stats;
        launch_spec_draft(st, dp);
        dp.accepted = s->acc.accepted;
        dp.emitted = s->acc.emitted;
        int32_t stats[4] = {0, 0, 0, 0};
        while (!done) {
            int enq = 0;
            for (; enq < burst && s->h_pos_upper[seq] + nodes <= cap; enq++) {
                enqueue_staged_step(s);
                launch_spec_draft(st, dp);
                s->h_pos_upper[seq] += nodes;
            }
            if (enq == 0) break;  // the context is full
            int new_len = 0, pos = 0;
            YK_CUDA(cudaMemcpyAsync(&new_len, s->d_hist_len, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
            YK_CUDA(cudaMemcpyAsync(&pos, s->d_pos0 + seq, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
            YK_CUDA(cudaMemcpyAsync(stats, s->d_spec_stats, sizeof stats, cudaMemcpyDeviceToHost, st));
            sync_and_check(s);
            s->h_pos[seq] = s->h_pos_upper[seq] = pos;
            if (new_len > hist_len) {
                hist.resize((size_t)new_len);
                YK_CUDA(cudaMemcpy(hist.data() + hist_len, s->d_hist + hist_len, (size_t)(new_len - hist_len) * sizeof(int32_t),
                                   cudaMemcpyDeviceToHost));
                for (int i = hist_len; i < new_len && !done; i++) done = emit(hist[(size_t)i]);
                hist_len = new_len;
            }
        }
        result->output_tokens = n_out;
        result->steps = stats[0];
        result->draft_tokens = stats[1];
        result->accepted_draft = stats[2];
    });
}

yuuka_stream * yuuka_session_stream(yuuka_session * s) { return s ? &s->stream : nullptr; }

uint32_t yuuka_session_last_launch_count(const yuuka_session * s) { return s ? s->launches : 0; }

}  // extern "C"
