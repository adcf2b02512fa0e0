// Host side of exact greedy speculative decoding over a verify session: the
// counterpart of engine/speculative.go, written for the k+1-row verify step.
//
// The reference keeps `logits` for the position after the last fed token,
// verifies k draft rows, and on a miss restores a state snapshot and replays
// the accepted prefix plus the correction (engine/speculative.go:181-239).
// Here the last emitted token is held back as `pending`; one verify step feeds
// [pending, d1..dk], accepts the longest prefix whose tokens equal the argmax
// of the row before them, emits the accepted drafts plus the correction or
// bonus token, and commits only the accepted rows on the device: no snapshot,
// no replay. The emitted stream is the greedy continuation either way.
#include <algorithm>
#include <vector>

#include "common.cuh"

using namespace yk;

namespace {
// a failed inner call has already recorded its message; pass its status through
void inner(yuuka_status st) {
    if (st != YUUKA_OK) throw StatusError{st};
}
}  // namespace

extern "C" {

// SpeculativeOptions.normalize, engine/speculative.go:21-34
void yuuka_spec_options_normalize(yuuka_spec_options * o) {
    if (!o) return;
    if (o->max_draft <= 0) o->max_draft = 4;
    if (o->max_draft > 16) o->max_draft = 16;
    if (o->min_match <= 0) o->min_match = 2;
    if (o->min_match > 8) o->min_match = 8;
}

// lookupDraft, engine/speculative.go:39-66: the longest history suffix (at most
// 8 tokens, at least min_match) that occurred earlier; of its earlier
// occurrences the latest one that is followed by at least one token; returns
// the tokens that followed it, at most max_draft.
int32_t yuuka_spec_lookup_draft(const int32_t * history, int32_t n, int32_t max_draft, int32_t min_match, int32_t * out) {
    if (!history || !out || max_draft <= 0 || min_match <= 0 || n <= min_match) return 0;
    const int longest = std::min(8, n - 1);
    for (int len = longest; len >= min_match; len--) {
        const int32_t * suffix = history + (n - len);
        for (int start = n - len - 1; start >= 0; start--) {
            if (!std::equal(suffix, suffix + len, history + start)) continue;
            const int follow = start + len;
            const int take = std::min(max_draft, n - follow);
            if (take <= 0) continue;
            std::copy(history + follow, history + follow + take, out);
            return take;
        }
    }
    return 0;
}

yuuka_status yuuka_spec_generate(yuuka_session * s, int32_t seq, const int32_t * prompt, int32_t n_prompt,
                                 const yuuka_spec_request * req, int32_t * tokens, yuuka_spec_result * result) {
    return guard([&] {
        YK_REQUIRE(s && prompt && req && tokens && result, YUUKA_ERR_INVALID_ARGUMENT, "spec_generate: null argument");
        *result = yuuka_spec_result{};
        YK_REQUIRE(n_prompt > 0, YUUKA_ERR_INVALID_ARGUMENT, "prompt is empty");
        YK_REQUIRE(req->max_tokens > 0, YUUKA_ERR_INVALID_ARGUMENT, "max tokens must be positive");
        yuuka_session_info info{};
        inner(yuuka_session_info_get(s, &info));
        YK_REQUIRE(n_prompt <= info.capacity, YUUKA_ERR_INVALID_ARGUMENT, "prompt length %d exceeds context capacity %d",
                   n_prompt, info.capacity);
        int max_tokens = std::min(req->max_tokens, info.capacity - n_prompt);
        YK_REQUIRE(max_tokens > 0, YUUKA_ERR_INVALID_ARGUMENT, "no context space remains for generated tokens");
        YK_REQUIRE(req->n_stop >= 0 && (req->n_stop == 0 || req->stop_tokens), YUUKA_ERR_INVALID_ARGUMENT,
                   "spec_generate: stop token list is null");
        yuuka_spec_options so = req->options;
        yuuka_spec_options_normalize(&so);
        so.max_draft = std::min(so.max_draft, info.max_nodes - 1);

        auto is_stop = [&](int32_t t) {
            return std::find(req->stop_tokens, req->stop_tokens + req->n_stop, t) != req->stop_tokens + req->n_stop;
        };
        std::vector<int32_t> history(prompt, prompt + n_prompt);
        history.reserve((size_t)n_prompt + max_tokens);
        std::vector<float> logits((size_t)info.vocab);
        std::vector<int32_t> rows((size_t)info.max_nodes), emitted((size_t)info.max_nodes);
        int n_out = 0;
        result->prompt_tokens = n_prompt;
        result->finish_reason = YUUKA_FINISH_LENGTH;

        inner(yuuka_session_reset(s, seq));
        inner(yuuka_session_forward(s, seq, prompt, n_prompt, logits.data()));
        // argmaxLogit, engine/speculative.go:263-271: first index of the maximum
        int32_t pending = 0;
        for (int i = 1; i < info.vocab; i++)
            if (logits[(size_t)i] > logits[(size_t)pending]) pending = i;

        // returns true when generation has to stop
        auto emit = [&](int32_t t) {
            if (is_stop(t)) {
                result->finish_reason = YUUKA_FINISH_STOP;
                return true;
            }
            tokens[n_out++] = t;
            history.push_back(t);
            return n_out >= max_tokens;
        };
        bool done = emit(pending);
        while (!done) {
            // pending is emitted but not run: a step of k drafts runs k + 1 rows and emits at most k + 1 tokens
            const int fed = (int)history.size() - 1;
            int limit = std::min(so.max_draft, max_tokens - n_out - 1);
            limit = std::min(limit, info.capacity - fed - 1);
            if (info.capacity - fed < 1) break;
            rows[0] = pending;
            const int k = limit > 0 ? yuuka_spec_lookup_draft(history.data(), (int32_t)history.size(), limit, so.min_match,
                                                              rows.data() + 1)
                                    : 0;
            int32_t accepted = 0;
            yuuka_verify_batch vb{};
            vb.batch = 1;
            vb.nodes = k + 1;
            vb.tokens = rows.data();
            vb.mode = YUUKA_ACCEPT_GREEDY;
            vb.accepted = &accepted;
            vb.emitted = emitted.data();
            vb.seq_ids = &seq;
            inner(yuuka_verify_step(s, &vb));
            result->steps++;
            result->draft_tokens += k;
            result->accepted_draft += accepted;
            for (int i = 0; i <= accepted && !done; i++) done = emit(emitted[(size_t)i]);
            pending = emitted[(size_t)accepted];
        }
        result->output_tokens = n_out;
    });
}

}  // extern "C"
