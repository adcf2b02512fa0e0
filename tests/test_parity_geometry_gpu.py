"""GPU-vs-oracle parity at the per-head geometry of the graded configurations, through the C ABI.

The tiny model of the other parity tests has head_dim 64 with a full rotary, delta-net state 64 and as
many value heads as key groups, so it instantiates different kernels from the ones the 4B-shaped
configurations run. The models here keep those configurations' per-head shapes and shrink only the
widths that do not select a kernel (hidden size, layer count, vocabulary), so that the CPU oracle
finishes in seconds:

* head_dim 256 with a partial rotary (64 of 256 dimensions, model/qwen35/forward.go:181-182,495-514),
  several query heads per KV head, delta-net state 128 with more value heads than key groups
  (kh = h % groups, model/qwen35/recurrent.go:62), Q4_K / Q6_K weights: prompt passes in the three KV
  formats, 9-row chain steps with partial accepts, the 17-row tree, committed state;
* rejection-sampling acceptance over the full 248,320-token vocabulary at temperature 0.7;
* the qwen35moe block with 256 experts of which 8 are used (selectExperts, forward.go:393-439) on
  160 rows, so that every expert group of the router and a full segment list take part.

Bars as in test_verify_gpu.py: integers bit-exact (outside documented near-ties), logits within
max-abs 2e-2 and cosine >= 0.9999 of the fp32 CPU path, recurrent state within 2e-3.
"""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2
STATE_TOL = 2e-3


def cosine(a, b):
    a, b = a.ravel().astype(np.float64), b.ravel().astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def head_geometry_config(**over) -> dict:
    """Four layers (three Gated-DeltaNet, one gated attention) with the 4B configuration's head shapes."""
    cfg = dict(block_count=4, context_length=512, hidden=512, ffn=1536, heads=8, kv_heads=2, head_dim=256,
               rope_dim=64, rope_freq_base=1.0e7, rms_eps=1e-6, vocab=4096, conv_kernel=4, state_size=128,
               group_count=2, time_step_rank=4, inner_size=512, full_attention_interval=4, expert_count=0,
               expert_used=0, expert_ffn=0, shared_ffn=0)
    cfg.update(over)
    return cfg


@pytest.fixture(scope="module")
def geo():
    cfg = head_geometry_config()
    tensors = synth.make_model(cfg, "q4_k_m", seed=41, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    yield cfg, gm, om
    gm.close()
    dev.close()


def greedy(om, prompt, n, kv=yo.KV_F32, capacity=256):
    st = yo.State(om, capacity, kv)
    logits = st.forward(prompt)
    out = []
    for _ in range(n):
        t = yo.argmax(logits)
        out.append(t)
        logits = st.step(t)
    st.close()
    return out


def top2_gap(logits):
    part = np.partition(logits, -2, axis=-1)
    return part[..., -1] - part[..., -2]


@pytest.mark.parametrize("kv", [cuda.KV_F32, cuda.KV_F16, cuda.KV_Q8_0])
def test_prompt_pass_matches_oracle(geo, kv):
    cfg, gm, om = geo
    prompt = synth.uniform_i32(40, 0, cfg["vocab"], 121)
    st = yo.State(om, 128, kv)
    want = st.prefill_logits(prompt)
    sess = cuda.Session(gm, max_batch=1, max_nodes=16, capacity=128, kv_format=kv)
    got = sess.prefill_logits(prompt)
    assert sess.position() == st.pos == 40
    err = float(np.max(np.abs(got - want)))
    assert err <= LOGIT_TOL and cosine(got, want) >= 0.9999, (err, cosine(got, want))
    snap_g, snap_o = sess.snapshot().view(np.float32), st.snapshot().view(np.float32)
    assert snap_g.size == snap_o.size and float(np.max(np.abs(snap_g - snap_o))) <= STATE_TOL
    sess.close(); st.close()


def test_single_row_decode_matches_oracle_tightly(geo):
    """One row per step takes the fp32 routes: the head-to-group map, the rotary split and the query-head
    grouping show up undiluted by fp16 operands."""
    cfg, gm, om = geo
    prompt = synth.uniform_i32(10, 0, cfg["vocab"], 122)
    st = yo.State(om, 64, yo.KV_F32)
    sess = cuda.Session(gm, max_batch=1, max_nodes=1, capacity=64, kv_format=cuda.KV_F32)
    for t in prompt:
        want = st.step(int(t))
        got = sess.forward([int(t)])
    assert float(np.max(np.abs(got - want))) <= 5e-4
    assert float(np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32)))) <= 1e-4
    sess.close(); st.close()


def decisive(gap, err):
    """A row decides a token safely when its top-2 gap is outside the documented near-tie band (1e-3) and
    clear of the logit error measured on this very step."""
    return gap >= max(1e-3, 3.0 * err)


def test_chain_steps_with_partial_accepts_match_oracle(geo):
    cfg, gm, om = geo
    V, K = cfg["vocab"], 8
    prompt = synth.uniform_i32(48, 0, V, 136).tolist()
    want = greedy(om, prompt, 56, yo.KV_F16)
    drafts = synth.corrupt_draft(np.array(want, np.int32), V, 0.3, 17)
    st = yo.State(om, 256, yo.KV_F16)
    sess = cuda.Session(gm, max_batch=1, max_nodes=K + 1, capacity=256, kv_format=cuda.KV_F16)
    lo = st.forward(prompt)
    lg = sess.forward(prompt)
    assert float(np.max(np.abs(lg - lo))) <= LOGIT_TOL
    pending = yo.argmax(lo)
    out = [pending]
    n_acc = n_draft = compared = 0
    while len(out) < 40:
        draft = drafts[len(out):len(out) + K]
        acc_o, em_o, log_o = st.verify_chain(pending, draft, want_logits=True)
        res = sess.verify([[pending] + draft.tolist()], want_logits=True)
        acc_g = int(res.accepted[0])
        err = float(np.max(np.abs(res.logits[0] - log_o)))
        assert err <= LOGIT_TOL and cosine(res.logits[0], log_o) >= 0.9999, err
        if not decisive(float(top2_gap(log_o[:acc_o + 1]).min()), err):
            break                               # a near-tie may resolve either way; the two states part here
        assert acc_g == acc_o
        assert res.emitted[0, :acc_g + 1].tolist() == em_o.tolist()
        assert res.path[0, :acc_g].tolist() == list(range(1, acc_g + 1))
        assert sess.position() == st.pos
        compared += 1
        n_acc += acc_o
        n_draft += len(draft)
        out.extend(em_o.tolist())
        pending = out[-1]
    # (the oracle alone: gaps of at least 1.1e-2 on every deciding row of this seed, 17 steps)
    assert compared >= 8 and out == want[:len(out)]
    assert 0 < n_acc < n_draft
    assert float(np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32)))) <= STATE_TOL
    sess.close(); st.close()


def test_tree_step_matches_oracle(geo):
    cfg, gm, om = geo
    V = cfg["vocab"]
    prompt = synth.uniform_i32(37, 0, V, 127).tolist()   # top-2 gaps >= 6e-2 on the path's rows
    want = greedy(om, prompt, 6)
    parent = synth.tree_16()
    tokens = synth.uniform_i32(17, 0, V, 125)
    tokens[0] = want[0]
    tokens[2], tokens[8], tokens[12] = want[1], want[2], want[3]
    for kv in (cuda.KV_F32, cuda.KV_F16):
        st = yo.State(om, 128, kv)
        st.forward(prompt)
        acc_o, path_o, em_o, log_o = st.verify_tree_greedy(tokens, parent, want_logits=True)
        assert acc_o == 3 and path_o.tolist() == [2, 8, 12]
        sess = cuda.Session(gm, max_batch=1, max_nodes=17, capacity=128, kv_format=kv)
        sess.forward(prompt, want_logits=False)
        res = sess.verify([tokens], parent=parent, want_logits=True)
        err = float(np.max(np.abs(res.logits[0] - log_o)))
        assert err <= LOGIT_TOL and cosine(res.logits[0], log_o) >= 0.9999, err
        assert int(res.accepted[0]) == 3 and res.path[0, :3].tolist() == [2, 8, 12]
        assert res.emitted[0, :4].tolist() == em_o.tolist()
        assert sess.position() == st.pos == 37 + 4
        assert float(np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32)))) <= STATE_TOL
        # the moved KV rows and the committed state carry plain decoding on
        nxt = int(em_o[-1])
        assert float(np.max(np.abs(sess.forward([nxt]) - st.step(nxt)))) <= LOGIT_TOL
        sess.close(); st.close()


def test_batched_trees_with_permuted_block_tables(geo):
    """Four sequences x 16-row trees = 64 query rows per KV head (the widest attention tile) over permuted
    block tables, contexts of different lengths, a different accepted branch in every sequence. 64 rows would
    take the tensor-memory GEMM route with its fp16-rounded weights; the session asks for the exact route so
    that every deciding row is clear of the logit error."""
    cfg, gm, om = geo
    V, B, cap, bs = cfg["vocab"], 4, 96, 16
    per = cap // bs
    parent = synth.tree_16()[:16].copy()
    N = parent.size
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=cap, kv_format=cuda.KV_F16, block_size=bs,
                        flags=cuda.SESSION_EXACT_WIDE)
    perm = np.random.default_rng(13).permutation(B * per).astype(np.int32)
    tokens = np.zeros((B, N), np.int32)
    states = []
    for b in range(B):
        table = perm[b * per:(b + 1) * per]
        sess.set_block_table(b, table)
        prompt = synth.uniform_i32(9 + 13 * b, 0, V, 130 + b).tolist()
        want = greedy(om, prompt, 4, yo.KV_F16)
        st = yo.State(om, cap, yo.KV_F16, pool_blocks=B * per, block_size=bs, table=table)
        st.forward(prompt)
        sess.forward(prompt, seq=b, want_logits=False)
        tokens[b] = synth.uniform_i32(N, 0, V, 140 + b)
        tokens[b, 0] = want[0]
        # the greedy continuation along root -> row 1 + b -> its first child (rows 1 and 2 have children) -> ...
        row = 1 + b
        for depth in range(1, 4):
            tokens[b, row] = want[depth]
            kids = [i for i in range(N) if parent[i] == row]
            if not kids:
                break
            row = kids[0]
        states.append(st)
    res = sess.verify(tokens, parent=parent, want_logits=True)
    accepted = []
    for b in range(B):
        acc_o, path_o, em_o, log_o = states[b].verify_tree_greedy(tokens[b], parent, want_logits=True)
        err = float(np.max(np.abs(res.logits[b] - log_o)))
        assert err <= LOGIT_TOL and cosine(res.logits[b], log_o) >= 0.9999, (b, err)
        if decisive(float(top2_gap(log_o[[0] + path_o.tolist()]).min()), err):
            assert int(res.accepted[b]) == acc_o
            assert res.path[b, :acc_o].tolist() == path_o.tolist()
            assert res.emitted[b, :acc_o + 1].tolist() == em_o.tolist()
            assert sess.position(b) == states[b].pos
            accepted.append(acc_o)
        states[b].close()
    assert len(accepted) >= 3 and max(accepted) >= 2
    sess.close()


def softmax32(x):
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def test_rejection_sampling_over_the_full_vocabulary():
    """Four sequences x 9-row chains, 248,320 tokens, temperature 0.7, draft distributions from the softmax of
    the logits plus unit noise: accepted counts, paths and emitted tokens equal the oracle's on the same
    logits, draft probabilities and uniforms, bit for bit."""
    V, B, N, T = 248320, 4, 9, 0.7
    cfg = dict(synth.tiny_config(), block_count=2, full_attention_interval=2, vocab=V)
    tensors = synth.make_model(cfg, "q8_0", seed=43, unit_norms=False, std=0.05)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    del tensors
    rng = np.random.default_rng(77)
    parent = np.arange(-1, N - 1, dtype=np.int32)
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=64, kv_format=cuda.KV_F16)
    tokens = np.zeros((B, N), np.int32)
    for b in range(B):
        prompt = synth.uniform_i32(6 + 3 * b, 0, V, 150 + b)
        tokens[b, 0] = int(np.argmax(sess.forward(prompt, seq=b)))
    q = np.zeros((B, N, V), np.float32)
    for c in range(1, N):
        res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True)
        for b in range(B):
            q[b, c] = softmax32(res.logits[b, c - 1].astype(np.float64) / T + rng.standard_normal(V))
            p64 = q[b, c].astype(np.float64)
            tokens[b, c] = rng.choice(V, p=p64 / p64.sum())
    logits = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits
    uniforms = np.minimum(rng.random((B, N, 2), dtype=np.float32), np.float32(0.99999994))
    qbuf = dev.upload(q)
    before = [sess.position(b) for b in range(B)]
    res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_REJECTION, temperature=T, draft_probs=qbuf,
                      uniforms=uniforms, want_logits=True)
    assert np.array_equal(res.logits.view(np.uint32), logits.view(np.uint32))
    for b in range(B):
        a, path, emitted = yo.accept_rejection_tree(logits[b], q[b], tokens[b], parent, T, uniforms[b])
        assert int(res.accepted[b]) == a, b
        assert res.path[b, :a].tolist() == path.tolist()
        assert res.emitted[b, :a + 1].tolist() == emitted.tolist()
        assert sess.position(b) == before[b] + a + 1
    qbuf.free()
    sess.close(); gm.close(); dev.close()


def test_rejection_walk_on_scaled_logits_full_vocabulary():
    """The same rule on logits with the spread the microbenchmark names (N(0, 3), so that a handful of tokens
    carry the mass and both the accept and the residual branch run): a one-layer model cannot produce such
    logits, so the temperature is lowered until its logits have that spread after the division."""
    V, B, N = 248320, 4, 9
    cfg = dict(synth.tiny_config(), block_count=2, full_attention_interval=2, vocab=V)
    tensors = synth.make_model(cfg, "q8_0", seed=44, unit_norms=False, std=0.05)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    del tensors
    rng = np.random.default_rng(78)
    parent = np.arange(-1, N - 1, dtype=np.int32)
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=64, kv_format=cuda.KV_F16)
    tokens = np.zeros((B, N), np.int32)
    for b in range(B):
        prompt = synth.uniform_i32(5 + 2 * b, 0, V, 160 + b)
        tokens[b, 0] = int(np.argmax(sess.forward(prompt, seq=b)))
    probe = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits
    T = float(probe[:, 0].std() / 3.0)          # logits / T ~ N(0, 3)
    q = np.zeros((B, N, V), np.float32)
    for c in range(1, N):
        res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True)
        for b in range(B):
            q[b, c] = softmax32(res.logits[b, c - 1].astype(np.float64) / T + rng.standard_normal(V))
            p64 = q[b, c].astype(np.float64)
            tokens[b, c] = rng.choice(V, p=p64 / p64.sum())
    logits = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits
    uniforms = np.minimum(rng.random((B, N, 2), dtype=np.float32), np.float32(0.99999994))
    qbuf = dev.upload(q)
    res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_REJECTION, temperature=T, draft_probs=qbuf,
                      uniforms=uniforms)
    total = 0
    for b in range(B):
        a, path, emitted = yo.accept_rejection_tree(logits[b], q[b], tokens[b], parent, T, uniforms[b])
        assert int(res.accepted[b]) == a, b
        assert res.path[b, :a].tolist() == path.tolist()
        assert res.emitted[b, :a + 1].tolist() == emitted.tolist()
        total += a
    assert 0 < total < B * (N - 1)            # accepts and rejections both occurred
    qbuf.free()
    sess.close(); gm.close(); dev.close()


def test_moe_block_with_256_experts_top_8():
    """32 sequences x 5-row chains = 160 rows through a two-layer qwen35moe model with 256 routed experts,
    8 used, plus the shared expert. The router picks experts by comparing logits, so a row whose eighth and
    ninth logits are closer than the error of its input changes expert and moves far; the session therefore
    runs the dense matrices on the exact route (the tensor-memory route's fp16 rounding flips a few per cent
    of the rows of such a step)."""
    cfg = dict(synth.tiny_config(), block_count=2, full_attention_interval=2, ffn=0, expert_count=256, expert_used=8,
               expert_ffn=256, shared_ffn=256)
    tensors = synth.make_model(cfg, "q4_k_m", seed=45, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    V, B, N = cfg["vocab"], 32, 5
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=64, kv_format=cuda.KV_F16, flags=cuda.SESSION_EXACT_WIDE)
    tokens = np.zeros((B, N), np.int32)
    states = []
    for b in range(B):
        prompt = synth.uniform_i32(3 + (b % 7), 0, V, 170 + b).tolist()
        st = yo.State(om, 64, yo.KV_F16)
        lo = st.forward(prompt)
        sess.forward(prompt, seq=b, want_logits=False)
        tokens[b] = synth.uniform_i32(N, 0, V, 210 + b)
        tokens[b, 0] = yo.argmax(lo)
        states.append(st)
    res = sess.verify(tokens, want_logits=True)
    worst = 0.0
    for b in range(B):
        acc_o, em_o, log_o = states[b].verify_chain(int(tokens[b, 0]), tokens[b, 1:], want_logits=True)
        err = float(np.max(np.abs(res.logits[b] - log_o)))
        worst = max(worst, err)
        assert err <= LOGIT_TOL and cosine(res.logits[b], log_o) >= 0.9999, (b, err)
        if decisive(float(top2_gap(log_o[:acc_o + 1]).min()), err):
            assert int(res.accepted[b]) == acc_o
            assert res.emitted[b, :acc_o + 1].tolist() == em_o.tolist()
            assert sess.position(b) == states[b].pos
        states[b].close()
    # the experts the router picked, for a few rows, against selectExperts on the oracle's router logits is
    # covered end to end by the logits above: a wrong expert or weight moves them by far more than the bar
    assert worst > 0.0
    sess.close(); gm.close(); dev.close()
