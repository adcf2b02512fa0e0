// Prompt-lookup drafting on the device (lookupDraft, engine/speculative.go:39-66), so that consecutive verify
// steps of one sequence can be enqueued without the host looking at the tokens in between.
//
// The reference searches, for n from min(8, len - 1) down to min_match, the latest earlier occurrence of the
// history's last n tokens and returns what followed it. Equivalently: for every end position e <= len - 2 let
// c(e) be the number of tokens ending at e that equal the tokens ending at len - 1 (capped at min(8, len - 1));
// the draft follows the e with the largest c(e) >= min_match, the largest such e among equals. One CTA takes
// the maximum of (c(e), e) over all e.
#include "layers.cuh"

namespace yk {

constexpr int DRAFT_THREADS = 256;

__global__ void __launch_bounds__(DRAFT_THREADS) spec_draft_kernel(const DraftParams p) {
    pdl_entry();
    __shared__ int n_s;
    __shared__ unsigned long long best_s[DRAFT_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int n = *p.hist_len;
        if (p.accepted) {
            // the step that just ran: its emitted tokens join the history, its counts the statistics
            const int a = *p.accepted, k_prev = p.stats[3];
            for (int i = 0; i <= a && n < p.hist_cap; i++) p.hist[n++] = p.emitted[i];
            p.stats[0] += 1;
            p.stats[1] += k_prev;
            p.stats[2] += a < k_prev ? a : k_prev;
            *p.hist_len = n;
        }
        n_s = n;
    }
    __syncthreads();
    const int n = n_s;
    unsigned long long best = 0ull;  // (c << 32) | e, 0: nothing found
    if (p.max_draft > 0 && p.min_match > 0 && n > p.min_match) {
        const int longest = n - 1 < 8 ? n - 1 : 8;
        for (int e = tid; e <= n - 2; e += DRAFT_THREADS) {
            int c = 0;
            while (c < longest && e - c >= 0 && p.hist[e - c] == p.hist[n - 1 - c]) c++;
            if (c >= p.min_match) {
                const unsigned long long key = ((unsigned long long)c << 32) | (unsigned)e;
                if (key > best) best = key;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        if (other > best) best = other;
    }
    if (lane == 0) best_s[warp] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < DRAFT_THREADS / 32; w++)
            if (best_s[w] > best) best = best_s[w];
        int k = 0;
        const int32_t pending = n > 0 ? p.hist[n - 1] : 0;
        if (p.rows_tokens) p.rows_tokens[0] = pending;
        if (best) {
            const int e = (int)(best & 0xffffffffull);
            k = n - (e + 1) < p.max_draft ? n - (e + 1) : p.max_draft;
            for (int i = 0; i < k; i++) {
                if (p.rows_tokens) p.rows_tokens[1 + i] = p.hist[e + 1 + i];
                if (p.draft_out) p.draft_out[i] = p.hist[e + 1 + i];
            }
        }
        // rows beyond the draft repeat the pending token: a greedy walk accepts a row only if its token is the
        // model's own choice, so padding can add correct tokens but never a wrong one
        if (p.rows_tokens)
            for (int i = 1 + k; i < p.nodes; i++) p.rows_tokens[i] = pending;
        if (p.stats) p.stats[3] = k;
        if (p.k_out) *p.k_out = k;
    }
}

void launch_spec_draft(cudaStream_t s, const DraftParams & p) {
    launch_k(spec_draft_kernel, 1, DRAFT_THREADS, 0, s, p);
    YK_CUDA(cudaGetLastError());
}

}  // namespace yk

// Stand-alone form of the device draft, for tests and for hosts that keep token histories on the device:
// out[0] = number of draft tokens, out[1..] = the tokens (yuuka_spec_lookup_draft is the host form).
extern "C" yuuka_status yuuka_spec_lookup_draft_device(yuuka_stream * stream, const yuuka_buffer * history, int32_t n,
                                                       int32_t max_draft, int32_t min_match, yuuka_buffer * out) {
    using namespace yk;
    return guard([&] {
        YK_REQUIRE(stream && history && out, YUUKA_ERR_INVALID_ARGUMENT, "lookup_draft_device: null argument");
        YK_REQUIRE(n >= 0 && (uint64_t)n * 4 <= history->bytes, YUUKA_ERR_INVALID_ARGUMENT,
                   "lookup_draft_device: history of %d tokens exceeds the buffer", n);
        YK_REQUIRE(max_draft >= 0 && max_draft <= 64 && (uint64_t)(1 + max_draft) * 4 <= out->bytes, YUUKA_ERR_INVALID_ARGUMENT,
                   "lookup_draft_device: output buffer holds fewer than 1 + max_draft ids");
        set_device(stream->dev);
        // the history length travels in the first word of out until the kernel overwrites it with the count
        YK_CUDA(cudaMemcpyAsync(out->ptr, &n, sizeof(int32_t), cudaMemcpyHostToDevice, stream->s));
        DraftParams p{};
        p.hist = (int32_t *)history->ptr;
        p.hist_len = (int32_t *)out->ptr;
        p.hist_cap = n;
        p.nodes = 0;
        p.max_draft = max_draft;
        p.min_match = min_match;
        p.draft_out = (int32_t *)out->ptr + 1;
        p.k_out = (int32_t *)out->ptr;
        launch_spec_draft(stream->s, p);
        YK_CUDA(cudaStreamSynchronize(stream->s));
    });
}
