"""Rejection-sampling acceptance over a draft tree: the CUDA kernel against the
CPU oracle's statement of the same rule, through the C ABI.

The reference verifies greedily only (engine/speculative.go:73-75), so nothing in
it pins this rule; the pins are the oracle (integer-exact rule, bit-exact match
demanded here) and two properties: a temperature near zero with one-hot draft
distributions reproduces the greedy walk, and the committed position advances
by accepted + 1.
"""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    cfg = synth.tiny_config()
    tensors = synth.make_model(cfg, "q8_0", seed=7, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    yield cfg, gm, dev
    gm.close()
    dev.close()


def softmax32(x):
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def draft_tree(rng, logits, parent, temperature, noise):
    """Draft distributions q[c] = softmax((L[parent c] + noise) / T) and tokens drawn from them."""
    n, V = logits.shape
    q = np.zeros((n, V), np.float32)
    tokens = np.zeros(n, np.int32)
    for c in range(1, n):
        q[c] = softmax32((logits[parent[c]] + noise * rng.standard_normal(V).astype(np.float32)) / temperature)
        tokens[c] = rng.choice(V, p=q[c].astype(np.float64) / q[c].astype(np.float64).sum())
    return q, tokens


@pytest.mark.parametrize("temperature,noise", [(0.8, 1.0), (0.7, 0.0), (1.5, 3.0)])
def test_rejection_walk_matches_oracle_bit_for_bit(tiny, temperature, noise):
    cfg, gm, dev = tiny
    V, B = cfg["vocab"], 3
    parent = np.array(synth.tree_16(), np.int32)
    N = parent.size
    rng = np.random.default_rng(int(temperature * 100) + int(noise * 10))
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=128, kv_format=cuda.KV_F16)
    prompts = [synth.uniform_i32(20 + 7 * b, 0, V, 60 + b) for b in range(B)]
    pend = [int(np.argmax(sess.forward(prompts[b], seq=b))) for b in range(B)]
    # a first pass that commits nothing gives the logits of the root rows; drafts are drawn level by level
    tokens = np.zeros((B, N), np.int32)
    tokens[:, 0] = pend
    q = np.zeros((B, N, V), np.float32)
    depth = np.zeros(N, np.int32)
    for c in range(1, N):
        depth[c] = depth[parent[c]] + 1
    for level in range(1, int(depth.max()) + 1):
        res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True)
        for b in range(B):
            for c in np.nonzero(depth == level)[0]:
                q[b, c] = softmax32((res.logits[b, parent[c]] + noise * rng.standard_normal(V).astype(np.float32)) / temperature)
                p64 = q[b, c].astype(np.float64)
                tokens[b, c] = rng.choice(V, p=p64 / p64.sum())
    logits = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits
    uniforms = rng.random((B, N, 2), dtype=np.float32)
    uniforms = np.minimum(uniforms, np.float32(0.99999994))
    qbuf = dev.upload(q)
    pos_before = [sess.position(b) for b in range(B)]
    res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_REJECTION, temperature=temperature, draft_probs=qbuf,
                      uniforms=uniforms, want_logits=True)
    assert np.array_equal(res.logits.view(np.uint32), logits.view(np.uint32))  # the step is deterministic
    total_accepted = 0
    for b in range(B):
        a, path, emitted = yo.accept_rejection_tree(logits[b], q[b], tokens[b], parent, temperature, uniforms[b])
        assert int(res.accepted[b]) == a
        assert res.path[b, :a].tolist() == path.tolist()
        assert res.emitted[b, :a + 1].tolist() == emitted.tolist()
        assert sess.position(b) == pos_before[b] + a + 1
        total_accepted += a
    if noise <= 1.0:
        assert total_accepted > 0  # the case exercises the accept branch, not only the residual draw
    qbuf.free()
    sess.close()


def test_cold_temperature_with_one_hot_drafts_is_the_greedy_walk(tiny):
    cfg, gm, dev = tiny
    V = cfg["vocab"]
    parent = np.array(synth.tree_16(), np.int32)
    N = parent.size
    prompt = synth.uniform_i32(33, 0, V, 91)
    outs = []
    for mode in (cuda.ACCEPT_GREEDY, cuda.ACCEPT_REJECTION):
        sess = cuda.Session(gm, max_batch=1, max_nodes=N, capacity=128, kv_format=cuda.KV_F32)
        pend = int(np.argmax(sess.forward(prompt)))
        tokens = synth.uniform_i32(N, 0, V, 92)
        tokens[0] = pend
        # make a three-deep greedy path exist in the tree: rows 2, 8, 12
        for row in (2, 8, 12):
            lg = sess.verify([tokens], parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits[0]
            tokens[row] = int(np.argmax(lg[parent[row]]))
        if mode == cuda.ACCEPT_GREEDY:
            res = sess.verify([tokens], parent=parent)
        else:
            q = np.zeros((1, N, V), np.float32)
            q[0, np.arange(N), tokens] = 1.0
            qbuf = dev.upload(q)
            u = np.full((1, N, 2), 0.5, np.float32)
            res = sess.verify([tokens], parent=parent, mode=mode, temperature=0.01, draft_probs=qbuf, uniforms=u)
            qbuf.free()
        a = int(res.accepted[0])
        outs.append((a, res.path[0, :a].tolist(), res.emitted[0, :a + 1].tolist(), sess.position()))
        sess.close()
    assert outs[0] == outs[1]
    assert outs[0][0] == 3 and outs[0][1] == [2, 8, 12]


def test_rejection_arguments_are_validated(tiny):
    cfg, gm, dev = tiny
    V = cfg["vocab"]
    sess = cuda.Session(gm, max_batch=1, max_nodes=4, capacity=64, kv_format=cuda.KV_F32)
    sess.forward([1, 2, 3], want_logits=False)
    toks = [[5, 6, 7, 8]]
    q = dev.upload(np.zeros((1, 4, V), np.float32))
    small = dev.upload(np.zeros(16, np.float32))
    u = np.full((1, 4, 2), 0.5, np.float32)
    bad = [dict(temperature=0.0, draft_probs=q, uniforms=u), dict(temperature=0.8, draft_probs=None, uniforms=u),
           dict(temperature=0.8, draft_probs=small, uniforms=u), dict(temperature=0.8, draft_probs=q, uniforms=None),
           dict(temperature=0.8, draft_probs=q, uniforms=np.full((1, 4, 2), 1.0, np.float32))]
    for kw in bad:
        with pytest.raises(cuda.YuukaError) as e:
            sess.verify(toks, mode=cuda.ACCEPT_REJECTION, **kw)
        assert e.value.status == 1
    assert sess.position() == 3  # nothing ran
    q.free(); small.free()
    sess.close()


def test_acceptance_case_of_the_kernel_microbenchmark_matches_the_oracle():
    """fp32 logits N(0, 3) over 248,320 tokens for 16 sequences x 9 positions (the microbenchmark names 64
    sequences; 16 keep the CPU side of the test to seconds), draft probabilities = softmax of the logits plus
    N(0, 1) noise, temperature 0.7, seeded uniforms: yuuka_accept_tree returns the oracle's accepted counts,
    paths and emitted tokens bit for bit, for the rejection walk and for the greedy walk."""
    V, B, N, T = 248320, 16, 9, 0.7
    dev = cuda.Device(0)
    stream = dev.stream()
    rng = np.random.default_rng(2026)
    logits = (3.0 * rng.standard_normal((B, N, V), dtype=np.float32)).astype(np.float32)
    parent = np.arange(-1, N - 1, dtype=np.int32)
    q = np.zeros((B, N, V), np.float32)
    tokens = np.zeros((B, N), np.int32)
    tokens[:, 0] = rng.integers(0, V, B)
    for b in range(B):
        for c in range(1, N):
            q[b, c] = softmax32(logits[b, c - 1] / T + rng.standard_normal(V, dtype=np.float32))
            # half of the drafts are the draft model's most likely token, half are drawn from it
            if (b + c) % 2:
                tokens[b, c] = int(np.argmax(q[b, c]))
            else:
                p64 = q[b, c].astype(np.float64)
                tokens[b, c] = rng.choice(V, p=p64 / p64.sum())
    uniforms = np.minimum(rng.random((B, N, 2), dtype=np.float32), np.float32(0.99999994))
    lb, qb = dev.upload(logits), dev.upload(q)
    acc, em, path = cuda.accept_tree(stream, lb, tokens, V, parent=parent, mode=cuda.ACCEPT_REJECTION, temperature=T,
                                     draft_probs=qb, uniforms=uniforms)
    total = 0
    for b in range(B):
        a, p_o, e_o = yo.accept_rejection_tree(logits[b], q[b], tokens[b], parent, T, uniforms[b])
        assert int(acc[b]) == a, b
        assert path[b, :a].tolist() == p_o.tolist() and em[b, :a + 1].tolist() == e_o.tolist()
        total += a
    assert 0 < total < B * (N - 1)
    # greedy walk over the same logits, with the first three drafts of every other sequence set to the argmax chain
    for b in range(0, B, 2):
        for c in range(1, 4):
            tokens[b, c] = int(np.argmax(logits[b, c - 1]))
    acc, em, path = cuda.accept_tree(stream, lb, tokens, V, parent=parent)
    for b in range(B):
        a, p_o, e_o = yo.accept_greedy_tree(logits[b], tokens[b], parent)
        assert int(acc[b]) == a and path[b, :a].tolist() == p_o.tolist() and em[b, :a + 1].tolist() == e_o.tolist()
        assert a >= 3 or b % 2
    lb.free(); qb.free()
    stream.destroy()
    dev.close()
