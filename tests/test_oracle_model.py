"""Oracle model-level properties: the reference's speculative loop emits the
greedy token stream (engine/speculative_test.go:103-137,180-215), and the
k+1-row verify formulation and tree verification agree with it."""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import synth


@pytest.fixture(scope="module")
def tiny():
    cfg = synth.tiny_config()
    tensors = synth.make_model(cfg, "q8_0", seed=7)
    return cfg, tensors, yo.Model(cfg, tensors)


def greedy_tokens(model, prompt, n, kv=yo.KV_F32):
    st = yo.State(model, 256, kv)
    logits = st.forward(prompt)
    out = []
    for _ in range(n):
        t = yo.argmax(logits)
        out.append(t)
        logits = st.step(t)
    st.close()
    return out


def test_quantizers_round_trip():
    x = synth.normal_f32(8 * 512, 0.02, 3).reshape(8, 512)
    for dtype, tol in ((synth.Q8_0, 0.02 * 4 / 127), (synth.Q6_K, 0.02 * 5 / 31),
                       (synth.Q5_K, 0.02 * 8 / 31), (synth.Q4_K, 0.02 * 8 / 15)):
        packed = synth.quantize(x, dtype)
        rb = synth.row_bytes(dtype, 512)
        back = np.stack([yo.dequantize_row(dtype, packed[r * rb:(r + 1) * rb]) for r in range(8)])
        assert np.max(np.abs(back - x)) < tol, dtype
    # the seeded stream does not depend on how it is consumed
    a = synth.normal_quant(4, 512, synth.Q4_K, 0.02, 11)
    b = synth.quantize(synth.normal_f32(4 * 512, 0.02, 11).reshape(4, 512), synth.Q4_K)
    assert np.array_equal(a, b)


def test_snapshot_restore_round_trip(tiny):
    cfg, _, model = tiny
    st = yo.State(model, 64, yo.KV_F32)
    st.forward([1, 2, 3, 4, 5])
    snap = st.snapshot()
    # state.go:211-234: conv then s for each recurrent layer, f32 LE
    S, G, R = cfg["state_size"], cfg["group_count"], cfg["time_step_rank"]
    conv_dim = 2 * G * S + cfg["inner_size"]
    per_layer = (cfg["conv_kernel"] - 1) * conv_dim + R * S * S
    assert snap.size == 3 * per_layer * 4
    assert np.array_equal(snap[:12 * conv_dim].view(np.float32), st.rec_conv(0))
    a = st.step(9)
    st.restore(snap)
    st.set_pos(5)
    b = st.step(9)
    assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        st.restore(snap[:-4])
    st.close()


def test_reference_speculative_loop_matches_greedy(tiny):
    cfg, _, model = tiny
    prompt = synth.uniform_i32(24, 0, cfg["vocab"], 5).tolist()
    want = greedy_tokens(model, prompt, 20)
    drafts = synth.corrupt_draft(np.array(want, np.int32), cfg["vocab"], 0.3, 99)
    st = yo.State(model, 256, yo.KV_F32)
    logits = st.forward(prompt)
    out, i, n_draft, n_acc = [], 0, 0, 0
    while len(out) < 16:
        draft = drafts[len(out):len(out) + 4]
        acc, emitted, logits = st.spec_verify_reference(logits, draft)
        n_draft += len(draft)
        n_acc += acc
        out.extend(emitted.tolist())
    assert out[:16] == want[:16]
    assert 0 < n_acc < n_draft
    st.close()


def test_k_plus_one_rows_match_reference_formulation(tiny):
    cfg, _, model = tiny
    prompt = synth.uniform_i32(24, 0, cfg["vocab"], 6).tolist()
    want = greedy_tokens(model, prompt, 24)
    drafts = synth.corrupt_draft(np.array(want, np.int32), cfg["vocab"], 0.3, 100)
    # the k+1-row path holds a pending token instead of its logits
    st = yo.State(model, 256, yo.KV_F32)
    logits = st.forward(prompt)
    pending = yo.argmax(logits)
    out = [pending]
    while len(out) < 20:
        draft = drafts[len(out):len(out) + 4]
        acc, emitted, _ = st.verify_chain(pending, draft)
        assert st.pos == len(prompt) + len(out) + acc
        out.extend(emitted.tolist())
        pending = out[-1]
    assert out[:20] == want[:20]
    st.close()


def test_tree_verify_equals_chain_on_a_chain(tiny):
    cfg, _, model = tiny
    prompt = synth.uniform_i32(16, 0, cfg["vocab"], 8).tolist()
    want = greedy_tokens(model, prompt, 6)
    draft = [want[1], want[2], 17, want[4]]
    a = yo.State(model, 128, yo.KV_F32)
    a.forward(prompt)
    acc_c, em_c, log_c = a.verify_chain(want[0], draft, want_logits=True)
    b = yo.State(model, 128, yo.KV_F32)
    b.forward(prompt)
    acc_t, path, em_t, log_t = b.verify_tree_greedy([want[0]] + draft, [-1, 0, 1, 2, 3], want_logits=True)
    assert acc_c == acc_t == 2 and em_c.tolist() == em_t.tolist() == [want[1], want[2], want[3]]
    assert path.tolist() == [1, 2]
    assert np.array_equal(log_c, log_t)
    assert np.array_equal(a.snapshot(), b.snapshot()) and a.pos == b.pos
    a.close(); b.close()


def test_tree_verify_takes_the_matching_branch(tiny):
    cfg, _, model = tiny
    prompt = synth.uniform_i32(16, 0, cfg["vocab"], 9).tolist()
    want = greedy_tokens(model, prompt, 5)
    parent = synth.tree_16()
    tokens = np.full(17, 3, np.int32)
    tokens[0] = want[0]
    tokens[1:5] = [5, want[1], 6, 7]          # branch 2 matches
    tokens[7:9] = [8, want[2]]                # children of node 2: second matches
    tokens[12] = want[3]                      # child of node 8
    tokens[16] = 11                           # child of node 12: wrong
    st = yo.State(model, 128, yo.KV_F32)
    st.forward(prompt)
    acc, path, emitted, _ = st.verify_tree_greedy(tokens, parent)
    assert acc == 3 and path.tolist() == [2, 8, 12]
    assert emitted.tolist() == [want[1], want[2], want[3], want[4]]
    # committed state equals plain decoding of the accepted tokens
    ref = yo.State(model, 128, yo.KV_F32)
    ref.forward(prompt + want[:4])
    assert np.array_equal(ref.snapshot(), st.snapshot()) and ref.pos == st.pos
    st.close(); ref.close()


def test_permuted_block_table_gives_identical_logits(tiny):
    cfg, _, model = tiny
    prompt = synth.uniform_i32(40, 0, cfg["vocab"], 10).tolist()
    a = yo.State(model, 64, yo.KV_F16)
    b = yo.State(model, 64, yo.KV_F16, pool_blocks=9, block_size=16, table=[5, 0, 8, 2])
    assert np.array_equal(a.forward(prompt), b.forward(prompt))
    a.close(); b.close()


def test_moe_forward_runs_and_uses_top_k():
    cfg = synth.tiny_moe_config()
    model = yo.Model(cfg, synth.make_model(cfg, "q8_0", seed=3))
    st = yo.State(model, 32, yo.KV_F32)
    logits = st.forward([1, 2, 3])
    assert np.all(np.isfinite(logits)) and float(np.std(logits)) > 0
    st.close()


def test_rejection_sampling_properties():
    rng = np.random.default_rng(0)
    V, k = 512, 4
    logits = (rng.standard_normal((k + 1, V)) * 3).astype(np.float32)
    parent = np.arange(-1, k, dtype=np.int32)
    q = np.exp(logits + rng.standard_normal((k + 1, V)).astype(np.float32))
    q = (q / q.sum(-1, keepdims=True)).astype(np.float32)
    # draft distribution of node c is the one its token was drawn from: row parent[c]
    Q = np.zeros_like(q)
    Q[1:] = q[:-1]
    tokens = np.zeros(k + 1, np.int32)
    tokens[1:] = [int(np.argmax(Q[c])) for c in range(1, k + 1)]
    U = rng.random(2 * (k + 1)).astype(np.float32)
    # T -> 0 degenerates to greedy
    greedy_tokens_ = tokens.copy()
    greedy_tokens_[1] = int(np.argmax(logits[0]))
    greedy_tokens_[2] = int(np.argmax(logits[1]))
    greedy_tokens_[3] = (int(np.argmax(logits[2])) + 1) % V
    a_g, _, em_g = yo.accept_greedy_tree(logits, greedy_tokens_, parent)
    a_r, _, em_r = yo.accept_rejection_tree(logits, Q, greedy_tokens_, parent, 1e-4, U)
    assert a_g == a_r == 2 and em_g.tolist() == em_r.tolist()
    # q == p: every draft is accepted whatever the uniforms
    p = np.exp((logits - logits.max(-1, keepdims=True)) / np.float32(0.7))
    p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
    Qp = np.zeros_like(p)
    Qp[1:] = p[:-1] * np.float32(0.999)
    a, _, em = yo.accept_rejection_tree(logits, Qp, tokens, parent, 0.7, U)
    assert a == k and 0 <= em[-1] < V
    # empirical acceptance probability of the first draft ~ min(1, p/q)
    x = int(np.argsort(Q[1])[-3])
    toks = tokens.copy()
    toks[1] = x
    p0 = np.exp((logits[0] - logits[0].max()) / 0.7)
    p0 /= p0.sum()
    want = min(1.0, p0[x] / Q[1][x])
    hits = 0
    for s in range(400):
        Us = np.random.default_rng(s).random(2 * (k + 1)).astype(np.float32)
        a, _, _ = yo.accept_rejection_tree(logits, Q, toks, parent, 0.7, Us)
        hits += a >= 1
    assert abs(hits / 400 - want) < 0.08


def test_exp_det_accuracy():
    xs = np.linspace(-80, 0, 4001, dtype=np.float32)
    got = np.array([yo.lib().yo_exp_det(float(x)) for x in xs])
    assert np.max(np.abs(got - np.exp(xs.astype(np.float64))) / np.exp(xs.astype(np.float64))) < 3e-7
    assert yo.lib().yo_exp_det(0.0) == 1.0 and yo.lib().yo_exp_det(-100.0) == 0.0
