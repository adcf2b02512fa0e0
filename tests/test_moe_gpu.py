"""qwen35moe feed-forward block (router, top-k, grouped expert GEMM, shared expert) on the GPU
against the CPU oracle (model/qwen35/forward.go:320-458), through the C ABI, on the tiny MoE
model (hidden 256, 8 experts, 2 used, expert FFN 256, shared FFN 256, Q8_0)."""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth

pytestmark = pytest.mark.gpu
LOGIT_TOL = 8e-3


def cosine(a, b):
    a, b = a.ravel().astype(np.float64), b.ravel().astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.fixture(scope="module")
def moe():
    cfg = synth.tiny_moe_config()
    tensors = synth.make_model(cfg, "q8_0", seed=11, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    yield cfg, gm, om
    gm.close()
    dev.close()


@pytest.mark.parametrize("n", [1, 2, 5, 23])
def test_prefill_logits_match_oracle(moe, n):
    cfg, gm, om = moe
    prompt = synth.uniform_i32(n, 0, cfg["vocab"], 40 + n)
    st = yo.State(om, 64, yo.KV_F32)
    want = st.prefill_logits(prompt)
    sess = cuda.Session(gm, max_batch=1, max_nodes=16, capacity=64, kv_format=cuda.KV_F32)
    got = sess.prefill_logits(prompt)
    err = float(np.max(np.abs(got - want)))
    assert err <= LOGIT_TOL and cosine(got, want) >= 0.9999, err
    sess.close(); st.close()


def test_chain_verify_and_following_decode(moe):
    cfg, gm, om = moe
    V = cfg["vocab"]
    prompt = synth.uniform_i32(30, 0, V, 51).tolist()
    st = yo.State(om, 128, yo.KV_F32)
    logits = st.forward(prompt)
    greedy = []
    probe = yo.State(om, 128, yo.KV_F32)
    lg = probe.forward(prompt)
    for _ in range(7):
        t = yo.argmax(lg); greedy.append(t); lg = probe.step(t)
    probe.close()
    draft = np.array(greedy[1:7], np.int32)
    draft[3] = (draft[3] + 5) % V
    acc_o, em_o, log_o = st.verify_chain(greedy[0], draft, want_logits=True)
    assert acc_o == 3
    sess = cuda.Session(gm, max_batch=1, max_nodes=7, capacity=128, kv_format=cuda.KV_F32)
    sess.forward(prompt, want_logits=False)
    res = sess.verify([[greedy[0]] + draft.tolist()], want_logits=True)
    assert float(np.max(np.abs(res.logits[0] - log_o))) <= LOGIT_TOL
    assert int(res.accepted[0]) == acc_o and res.emitted[0, :acc_o + 1].tolist() == em_o.tolist()
    assert sess.position() == st.pos
    nxt = int(em_o[-1])
    assert float(np.max(np.abs(sess.forward([nxt]) - st.step(nxt)))) <= LOGIT_TOL
    # the same step twice from the same state gives the same bits
    sess2 = cuda.Session(gm, max_batch=1, max_nodes=7, capacity=128, kv_format=cuda.KV_F32)
    sess2.forward(prompt, want_logits=False)
    res2 = sess2.verify([[greedy[0]] + draft.tolist()], want_logits=True)
    assert np.array_equal(res.logits.view(np.uint32), res2.logits.view(np.uint32))
    sess.close(); sess2.close(); st.close()


def test_batched_tree_rows_spread_over_experts(moe):
    cfg, gm, om = moe
    V, B = cfg["vocab"], 3
    parent = np.array(synth.tree_16(), np.int32)
    N = parent.size
    sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=96, kv_format=cuda.KV_F16)
    tokens = np.zeros((B, N), np.int32)
    states = []
    for b in range(B):
        prompt = synth.uniform_i32(10 + 9 * b, 0, V, 70 + b)
        sess.forward(prompt, seq=b, want_logits=False)
        st = yo.State(om, 96, yo.KV_F16)
        st.forward(prompt)
        states.append(st)
        tokens[b] = synth.uniform_i32(N, 0, V, 80 + b)
    res = sess.verify(tokens, parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True)  # 51 rows x 2 experts
    for b in range(B):
        _, _, _, log_o = states[b].verify_tree_greedy(tokens[b], parent, want_logits=True)
        err = float(np.max(np.abs(res.logits[b] - log_o)))
        assert err <= LOGIT_TOL and cosine(res.logits[b], log_o) >= 0.9999, (b, err)
        states[b].close()
    sess.close()
