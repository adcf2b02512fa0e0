"""End-to-end parity of the verify path against the CPU oracle on the tiny
qwen35 model (hidden 256, 3 Gated-DeltaNet + 1 gated-attention layers, vocab
4096, Q8_0 weights), through the C ABI.

Bars: integer results (accepted counts, emitted tokens, committed positions,
block-table addressing) bit-exact; logits within max-abs 2e-2 and cosine >=
0.9999 of the fp32 CPU path. The reference's own GPU-vs-CPU test bound for
all-logits rows on a tiny model is 5e-3 (engine/gpu/spec_fixture_test.go:70).
Steps of up to 47 rows run on the exact register-fed GEMM route (integer
weights, two-half activations) and land far inside that; prompts of 48 rows
and more pass through the tensor-memory route with fp16-rounded operands and
leave state and KV between 3e-3 and 6e-3 from the fp32 path depending on how
the prompt was chunked, so the tests that follow such a prompt are held to
8e-3 and single-row steps to a tight bound of their own.
"""
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
def tiny():
    cfg = synth.tiny_config()
    tensors = synth.make_model(cfg, "q8_0", seed=7, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    yield cfg, gm, om
    gm.close()
    dev.close()


def greedy(om, prompt, n, kv=yo.KV_F32):
    st = yo.State(om, 256, kv)
    logits = st.forward(prompt)
    out = []
    for _ in range(n):
        t = yo.argmax(logits)
        out.append(t)
        logits = st.step(t)
    st.close()
    return out


def top2_gaps(logits):
    part = np.partition(logits, -2, axis=-1)
    return (part[..., -1] - part[..., -2]).ravel().tolist()


@pytest.mark.parametrize("kv", [cuda.KV_F32, cuda.KV_F16, cuda.KV_Q8_0])
def test_prefill_logits_match_oracle(tiny, kv):
    cfg, gm, om = tiny
    prompt = synth.uniform_i32(40, 0, cfg["vocab"], 21)
    st = yo.State(om, 128, kv)
    want = st.prefill_logits(prompt)
    sess = cuda.Session(gm, max_batch=1, max_nodes=16, capacity=128, kv_format=kv)
    got = sess.prefill_logits(prompt)          # chunks of 16, 16, 8
    assert sess.position() == 40
    err = float(np.max(np.abs(got - want)))
    # a Q8_0 pool re-quantizes K/V rows: one flipped int8 step moves a value by max/127, so that
    # format is held to the path's stated bound (2e-2) rather than the tiny-model bound
    tol = 2e-2 if kv == cuda.KV_Q8_0 else LOGIT_TOL
    assert err <= tol and cosine(got, want) >= 0.9999, (err, cosine(got, want))
    # recurrent state and conv history after 40 tokens
    snap_g = sess.snapshot().view(np.float32)
    snap_o = st.snapshot().view(np.float32)
    assert snap_g.size == snap_o.size
    assert np.max(np.abs(snap_g - snap_o)) <= 2e-3
    sess.close(); st.close()


def test_single_row_steps_match_tightly(tiny):
    cfg, gm, om = tiny
    prompt = synth.uniform_i32(12, 0, cfg["vocab"], 22)
    st = yo.State(om, 64, yo.KV_F32)
    sess = cuda.Session(gm, max_batch=1, max_nodes=1, capacity=64, kv_format=cuda.KV_F32)
    for t in prompt:
        want = st.step(int(t))
        got = sess.forward([int(t)])
    # one row per step: the exact register-fed route (integer weights, two-half activations, fp32 accumulation)
    assert float(np.max(np.abs(got - want))) <= 2e-4
    sess.close(); st.close()


def test_chain_verify_matches_oracle(tiny):
    cfg, gm, om = tiny
    V = cfg["vocab"]
    prompt = synth.uniform_i32(64, 0, V, 23).tolist()
    want = greedy(om, prompt, 40)
    drafts = synth.corrupt_draft(np.array(want, np.int32), V, 0.3, 5)
    st = yo.State(om, 256, yo.KV_F32)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=256, kv_format=cuda.KV_F32)
    lo = st.forward(prompt)
    lg = sess.forward(prompt)
    assert yo.argmax(lo) == yo.argmax(lg)
    pending = yo.argmax(lo)
    out = [pending]
    n_acc = n_draft = 0
    while len(out) < 32:
        draft = drafts[len(out):len(out) + 4]
        acc_o, em_o, log_o = st.verify_chain(pending, draft, want_logits=True)
        res = sess.verify([[pending] + draft.tolist()], want_logits=True)
        acc_g = int(res.accepted[0])
        gap = np.sort(log_o, -1)[:, -1] - np.sort(log_o, -1)[:, -2]
        if gap[:acc_o + 1].min() >= 1e-3:       # documented near-tie exemption
            assert acc_g == acc_o
            assert res.emitted[0, :acc_g + 1].tolist() == em_o.tolist()
            assert res.path[0, :acc_g].tolist() == list(range(1, acc_g + 1))
        err = float(np.max(np.abs(res.logits[0] - log_o)))
        assert err <= LOGIT_TOL and cosine(res.logits[0], log_o) >= 0.9999, err
        assert sess.position() == st.pos
        n_acc += acc_o
        n_draft += len(draft)
        out.extend(em_o.tolist())
        pending = out[-1]
    assert out[:32] == want[:32]
    assert 0 < n_acc < n_draft
    # committed recurrent state equals the oracle's after the same accepted tokens
    assert np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32))) <= 2e-3
    sess.close(); st.close()


def test_tree_verify_matches_oracle(tiny):
    cfg, gm, om = tiny
    V = cfg["vocab"]
    prompt = synth.uniform_i32(48, 0, V, 24).tolist()
    want = greedy(om, prompt, 6)
    parent = synth.tree_16()
    tokens = synth.uniform_i32(17, 0, V, 25)
    tokens[0] = want[0]
    tokens[1:5] = [tokens[1], want[1], tokens[3], tokens[4]]
    tokens[7:9] = [tokens[7], want[2]]
    tokens[12] = want[3]
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
        assert int(res.accepted[0]) == 3
        assert res.path[0, :3].tolist() == [2, 8, 12]
        assert res.emitted[0, :4].tolist() == em_o.tolist()
        assert sess.position() == st.pos == 48 + 4
        assert np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32))) <= 2e-3
        # the moved KV rows and committed state reproduce plain decoding afterwards
        nxt = int(em_o[-1])
        assert float(np.max(np.abs(sess.forward([nxt]) - st.step(nxt)))) <= LOGIT_TOL
        sess.close(); st.close()


def test_batched_sequences_with_permuted_block_tables(tiny):
    cfg, gm, om = tiny
    V = cfg["vocab"]
    B, cap, bs = 3, 96, 16
    per = cap // bs
    sess = cuda.Session(gm, max_batch=B, max_nodes=5, capacity=cap, kv_format=cuda.KV_F16, block_size=bs)
    perm = np.random.default_rng(3).permutation(B * per).astype(np.int32)
    states, pend, drafts = [], [], []
    for b in range(B):
        table = perm[b * per:(b + 1) * per]
        sess.set_block_table(b, table)
        prompt = synth.uniform_i32(20 + 7 * b, 0, V, 30 + b).tolist()
        st = yo.State(om, cap, yo.KV_F16, pool_blocks=B * per, block_size=bs, table=table)
        lo = st.forward(prompt)
        sess.forward(prompt, seq=b, want_logits=False)
        states.append(st)
        p = yo.argmax(lo)
        pend.append(p)
        g = greedy(om, prompt + [p], 4, yo.KV_F16)
        drafts.append(synth.corrupt_draft(np.array(g, np.int32), V, 0.4, 40 + b))
    toks = np.array([[pend[b]] + drafts[b].tolist() for b in range(B)], np.int32)
    res = sess.verify(toks, want_logits=True)
    for b in range(B):
        acc_o, em_o, log_o = states[b].verify_chain(pend[b], drafts[b], want_logits=True)
        assert float(np.max(np.abs(res.logits[b] - log_o))) <= LOGIT_TOL
        assert int(res.accepted[b]) == acc_o
        assert res.emitted[b, :acc_o + 1].tolist() == em_o.tolist()
        assert sess.position(b) == states[b].pos
        states[b].close()
    sess.close()


def test_steps_of_33_to_47_rows_on_the_wide_route_on_request(tiny):
    """Four sequences x nine rows: three exact 16-row passes by default, one pass of the tensor-memory route with
    YUUKA_SESSION_WIDE_FROM_33. Both stay inside the path's logit bound; the flag changes the kernels that run."""
    cfg, gm, om = tiny
    V, B = cfg["vocab"], 4
    states, pend, drafts, prompts = [], [], [], []
    for b in range(B):
        prompt = synth.uniform_i32(18 + 5 * b, 0, V, 60 + b).tolist()
        st = yo.State(om, 96, yo.KV_F32)
        p = yo.argmax(st.forward(prompt))
        g = greedy(om, prompt + [p], 8, yo.KV_F32)
        states.append(st); pend.append(p); prompts.append(prompt)
        drafts.append(synth.corrupt_draft(np.array(g, np.int32), V, 0.3, 70 + b))
    toks = np.array([[pend[b]] + drafts[b].tolist() for b in range(B)], np.int32)
    want = [states[b].verify_chain(pend[b], drafts[b], want_logits=True) for b in range(B)]
    counts = {}
    for flags in (0, cuda.SESSION_WIDE_FROM_33):
        sess = cuda.Session(gm, max_batch=B, max_nodes=9, capacity=96, kv_format=cuda.KV_F32, flags=flags)
        for b in range(B):
            sess.forward(prompts[b], seq=b, want_logits=False)
        res = sess.verify(toks, want_logits=True)
        counts[flags] = sess.last_launch_count
        for b in range(B):
            acc_o, em_o, log_o = want[b]
            err = float(np.max(np.abs(res.logits[b] - log_o)))
            assert err <= (5e-4 if flags == 0 else LOGIT_TOL), (flags, err)
            if all(g >= max(1e-3, 3 * err) for g in top2_gaps(log_o)):
                assert int(res.accepted[b]) == acc_o and res.emitted[b, :acc_o + 1].tolist() == em_o.tolist()
        sess.close()
    assert counts[0] != counts[cuda.SESSION_WIDE_FROM_33]
    for st in states:
        st.close()


def test_snapshot_restore_round_trip_and_legacy_rollback(tiny):
    """engine/speculative.go:181-216 through the legacy trio: snapshot, all-position
    logits, restore + replay."""
    cfg, gm, om = tiny
    V = cfg["vocab"]
    prompt = synth.uniform_i32(24, 0, V, 50).tolist()
    sess = cuda.Session(gm, max_batch=1, max_nodes=8, capacity=128, kv_format=cuda.KV_F32)
    st = yo.State(om, 128, yo.KV_F32)
    sess.forward(prompt, want_logits=False)
    st.forward(prompt)
    snap, pos = sess.snapshot(), sess.position()
    assert snap.size == st.snapshot().size
    draft = [5, 6, 7]
    a = sess.prefill_logits(draft)
    sess.restore(snap)
    sess.set_position(0, pos)
    b = sess.prefill_logits(draft)
    assert np.array_equal(a, b)                       # rollback is exact and the kernels are deterministic
    assert float(np.max(np.abs(a - st.prefill_logits(draft)))) <= LOGIT_TOL
    with pytest.raises(cuda.YuukaError):
        sess.restore(snap[:-4])
    sess.close(); st.close()


def test_argument_validation(tiny):
    cfg, gm, om = tiny
    sess = cuda.Session(gm, max_batch=1, max_nodes=4, capacity=32)
    with pytest.raises(cuda.YuukaError):              # token id out of range (forward.go:30-32)
        sess.forward([cfg["vocab"]])
    with pytest.raises(cuda.YuukaError):              # exceeds remaining context (forward.go:25-28)
        sess.forward(list(range(33)))
    with pytest.raises(cuda.YuukaError):              # parent must precede the row
        sess.verify([[1, 2, 3]], parent=[-1, 2, 0])
    with pytest.raises(cuda.YuukaError):              # more rows than the session holds
        sess.verify([[1, 2, 3, 4, 5]])
    with pytest.raises(cuda.YuukaError):
        sess.set_block_table(0, [999, 0])
    with pytest.raises(cuda.YuukaError):
        cuda.Session(gm, capacity=cfg["context_length"] + 1)
    bad = dict(cfg, kv_heads=3)
    with pytest.raises(cuda.YuukaError):
        cuda.Model(gm.dev, bad)
    sess.close()


def _verify_rows(gm, prompt, rows):
    sess = cuda.Session(gm, max_batch=1, max_nodes=len(rows), capacity=128, kv_format=cuda.KV_F32)
    sess.forward(prompt, want_logits=False)
    res = sess.verify([rows], want_logits=True)
    logits = res.logits[0].copy()
    sess.close()
    return logits


def test_folded_epilogues_match_their_own_kernels(tiny, monkeypatch):
    """RMSNorm folded into the neighbouring GEMMs and silu(gate) * up finished in the gate|up GEMM's
    epilogue, against the same step with the row-wise kernels launched on their own."""
    cfg, gm, om = tiny
    prompt = synth.uniform_i32(20, 0, cfg["vocab"], 61).tolist()
    rows = synth.uniform_i32(9, 0, cfg["vocab"], 62).tolist()
    folded = _verify_rows(gm, prompt, rows)
    monkeypatch.setenv("YUUKA_CUDA_NO_FOLD_SWIGLU", "1")
    own_silu = _verify_rows(gm, prompt, rows)
    # the epilogue evaluates the expression of the silu kernel on the same sums: identical bits
    assert np.array_equal(folded, own_silu)
    monkeypatch.setenv("YUUKA_CUDA_NO_FOLD_NORM", "1")
    plain = _verify_rows(gm, prompt, rows)
    # the folded norm rounds x * w * pre to fp16 before the scale is known: close, not identical
    assert float(np.max(np.abs(folded - plain))) <= 4e-3


def test_wide_hidden_narrow_ffn_model_matches_oracle():
    """hidden 4096 with FFN 256: few row tiles and a long K, so the gate|up GEMM splits K across CTAs and
    the SwiGLU epilogue runs in the CTA that sums the parts."""
    cfg = dict(synth.tiny_config(), block_count=2, full_attention_interval=2, hidden=4096, ffn=256, vocab=1024)
    tensors = synth.make_model(cfg, "q4_k_m", seed=11, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(12, 0, cfg["vocab"], 63).tolist()
    rows = synth.uniform_i32(9, 0, cfg["vocab"], 64).tolist()
    st = yo.State(om, 64, yo.KV_F32)
    st.forward(prompt)
    _, _, want = st.verify_chain(rows[0], np.array(rows[1:], np.int32), want_logits=True)
    got = _verify_rows(gm, prompt, rows)
    err = float(np.max(np.abs(got - want)))
    assert err <= 2e-2 and cosine(got, want) >= 0.9999, (err, cosine(got, want))
    st.close(); gm.close(); dev.close()


@pytest.mark.parametrize("kv", [cuda.KV_F32, cuda.KV_F16])
def test_long_prompts_run_as_wide_passes_with_mixer_sub_chunks(tiny, kv):
    """Prompts beyond 64 tokens: one pass of up to 512 rows for the GEMMs (two tensor-memory accumulators
    beyond 256 rows), 64-row sub-chunks for the delta-net scan, its state commit and the attention, ragged
    tails (300 = 4 x 64 + 44, 150 = 64 + 64 + 22)."""
    cfg, gm, om = tiny
    V = cfg["vocab"]
    prompt = synth.uniform_i32(300, 0, V, 71)
    st = yo.State(om, 512, kv)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=512, kv_format=kv)
    lo = st.forward(prompt.tolist())
    lg = sess.forward(prompt)
    assert sess.position() == st.pos == 300
    err = float(np.max(np.abs(lg - lo)))
    assert err <= 2e-2 and cosine(lg, lo) >= 0.9999, (err, cosine(lg, lo))
    assert np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32))) <= 4e-3
    # decoding continues from the committed state and KV rows
    nxt = yo.argmax(lo)
    err = float(np.max(np.abs(sess.forward([nxt]) - st.step(nxt))))
    assert err <= 2e-2, err
    sess.close(); st.close()
    # all-position logits over 150 tokens
    st = yo.State(om, 256, kv)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=256, kv_format=kv)
    want = st.prefill_logits(prompt[:150])
    got = sess.prefill_logits(prompt[:150])
    err = float(np.max(np.abs(got - want)))
    assert got.shape == (150, V) and err <= 2e-2 and cosine(got, want) >= 0.9999, (err, cosine(got, want))
    sess.close(); st.close()


def test_prompt_longer_than_one_pass():
    """600 tokens = a 512-row pass and an 88-row pass (64 + 24): state, conv history and KV rows carry over."""
    cfg = dict(synth.tiny_config(), context_length=1024)
    tensors = synth.make_model(cfg, "q8_0", seed=7, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(600, 0, cfg["vocab"], 72)
    st = yo.State(om, 640, yo.KV_F16)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=640, kv_format=cuda.KV_F16)
    lo = st.forward(prompt.tolist())
    lg = sess.forward(prompt)
    assert sess.position() == st.pos == 600
    err = float(np.max(np.abs(lg - lo)))
    assert err <= 2e-2 and cosine(lg, lo) >= 0.9999, (err, cosine(lg, lo))
    assert np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32))) <= 4e-3
    sess.close(); st.close(); gm.close(); dev.close()


def test_mixed_tensor_types_take_the_unfused_routes():
    """A file whose small projections stayed in F32 / F16 and whose gate and up differ in type: the fused
    matrices (qkv|gate|beta|alpha, q|k, gate|up) cannot be built, untiled matrices take the generic kernel,
    the norm is not folded, and the step still matches the oracle."""
    cfg = synth.tiny_config()
    tensors = synth.make_model(cfg, "q4_k", seed=21, unit_norms=False)
    H, R = cfg["hidden"], cfg["time_step_rank"]
    kv_dim = cfg["kv_heads"] * cfg["head_dim"]
    n = 0
    for name in list(tensors):
        n += 1
        if name.endswith("ssm_beta.weight") or name.endswith("ssm_alpha.weight"):
            tensors[name] = (synth.F32, synth.normal_f32(R * H, 0.02, 900 + n), R, H)
        elif name.endswith("attn_k.weight"):
            k16 = synth.normal_f32(kv_dim * H, 0.02, 900 + n).astype(np.float16)
            tensors[name] = (synth.F16, k16.view(np.uint8).copy(), kv_dim, H)
        elif name.endswith("ffn_up.weight"):
            tensors[name] = (synth.Q8_0, synth.normal_quant(cfg["ffn"], H, synth.Q8_0, 0.02, 900 + n), cfg["ffn"], H)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(70, 0, cfg["vocab"], 81).tolist()     # one wide pass with two sub-chunks
    rows = synth.uniform_i32(9, 0, cfg["vocab"], 82).tolist()
    st = yo.State(om, 128, yo.KV_F32)
    st.forward(prompt)
    _, _, want = st.verify_chain(rows[0], np.array(rows[1:], np.int32), want_logits=True)
    got = _verify_rows(gm, prompt, rows)
    err = float(np.max(np.abs(got - want)))
    assert err <= 2e-2 and cosine(got, want) >= 0.9999, (err, cosine(got, want))
    # one-row decode (fp32 routes everywhere) after the same prompt
    sess = cuda.Session(gm, max_batch=1, max_nodes=2, capacity=128, kv_format=cuda.KV_F32)
    sess.forward(prompt, want_logits=False)
    st2 = yo.State(om, 128, yo.KV_F32)
    st2.forward(prompt)
    err = float(np.max(np.abs(sess.forward([rows[0]]) - st2.step(rows[0]))))
    assert err <= 2e-2, err
    sess.close(); st.close(); st2.close(); gm.close(); dev.close()


@pytest.mark.parametrize("scheme", ["q4_k", "q5_k", "q6_k"])
def test_every_k_quant_through_the_folded_step(scheme):
    """The 9-row step (folded norms, SwiGLU epilogue, split-free and K-split GEMMs) with all matrices in one
    K-quant type, against the oracle."""
    cfg = dict(synth.tiny_config(), block_count=4)
    tensors = synth.make_model(cfg, scheme, seed=31, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(30, 0, cfg["vocab"], 91).tolist()
    rows = synth.uniform_i32(9, 0, cfg["vocab"], 92).tolist()
    st = yo.State(om, 64, yo.KV_F32)
    st.forward(prompt)
    _, _, want = st.verify_chain(rows[0], np.array(rows[1:], np.int32), want_logits=True)
    got = _verify_rows(gm, prompt, rows)
    err = float(np.max(np.abs(got - want)))
    assert err <= 2e-2 and cosine(got, want) >= 0.9999, (scheme, err, cosine(got, want))
    st.close(); gm.close(); dev.close()


def test_widest_tree_and_single_row_steps(tiny):
    """The limits of a step: 64 rows per sequence in a bushy random tree (the ancestor masks use all 64 bits,
    branches rebuild their parents' recurrent state from the delta log), and the one-row step."""
    cfg, gm, om = tiny
    V = cfg["vocab"]
    rng = np.random.default_rng(5)
    parent = np.array([-1] + [int(rng.integers(max(0, i - 6), i)) for i in range(1, 64)], np.int32)
    prompt = synth.uniform_i32(33, 0, V, 95).tolist()
    tokens = synth.uniform_i32(64, 0, V, 96)
    st = yo.State(om, 128, yo.KV_F32)
    lo = st.forward(prompt)
    tokens[0] = yo.argmax(lo)
    # seed a greedy path three levels deep along existing children of the tree
    sess = cuda.Session(gm, max_batch=1, max_nodes=64, capacity=128, kv_format=cuda.KV_F32)
    sess.forward(prompt, want_logits=False)
    node = 0
    for _ in range(3):
        kids = [i for i in range(1, 64) if parent[i] == node]
        if not kids:
            break
        lg = sess.verify([tokens], parent=parent, mode=cuda.ACCEPT_NONE, want_logits=True).logits[0]
        tokens[kids[-1]] = int(np.argmax(lg[node]))
        node = kids[-1]
    acc_o, path_o, em_o, log_o = st.verify_tree_greedy(tokens, parent, want_logits=True)
    res = sess.verify([tokens], parent=parent, want_logits=True)
    err = float(np.max(np.abs(res.logits[0] - log_o)))
    assert err <= LOGIT_TOL and cosine(res.logits[0], log_o) >= 0.9999, err
    gap = np.sort(log_o, -1)[:, -1] - np.sort(log_o, -1)[:, -2]
    if gap.min() >= 1e-3:
        a = int(res.accepted[0])
        assert a == acc_o >= 1
        assert res.path[0, :a].tolist() == path_o.tolist() and res.emitted[0, :a + 1].tolist() == em_o.tolist()
        assert sess.position() == st.pos
        assert np.max(np.abs(sess.snapshot().view(np.float32) - st.snapshot().view(np.float32))) <= 2e-3
    with pytest.raises(cuda.YuukaError):              # a 65th row does not fit the 64-bit ancestor masks
        cuda.Session(gm, max_batch=1, max_nodes=65, capacity=128)
    # one row: nothing to accept, the bonus token is the argmax
    one = sess.verify([[int(res.emitted[0, int(res.accepted[0])])]], want_logits=True)
    assert int(one.accepted[0]) == 0 and int(one.emitted[0, 0]) == int(np.argmax(one.logits[0, 0]))
    sess.close(); st.close()


def test_batch_over_a_list_of_sequences_equals_the_sequences_alone(tiny):
    """A scheduler verifies whichever runs are ready: sequences {5, 1, 6} of an eight-sequence session as one
    batch (seq_ids) give the integers and the logits, bit for bit, of the same three sequences stepped one by
    one, leave the other sequences untouched, and the next step may list them in another order."""
    cfg, gm, om = tiny
    V, B, N = cfg["vocab"], 8, 5
    ids = [5, 1, 6]

    def fresh():
        sess = cuda.Session(gm, max_batch=B, max_nodes=N, capacity=96, kv_format=cuda.KV_F16)
        pend = {}
        for sq in range(B):
            prompt = synth.uniform_i32(11 + 3 * sq, 0, V, 500 + sq)
            pend[sq] = int(np.argmax(sess.forward(prompt, seq=sq)))
        return sess, pend

    toks = {sq: [0] + synth.uniform_i32(N - 1, 0, V, 600 + sq).tolist() for sq in range(B)}
    a, pend = fresh()
    for sq in ids:
        toks[sq][0] = pend[sq]
    alone = {}
    for sq in ids:
        r = a.verify([toks[sq]], want_logits=True, seq_ids=[sq])
        alone[sq] = (int(r.accepted[0]), r.emitted[0].copy(), r.logits[0].copy(), a.position(sq))
    b, _ = fresh()
    before = {sq: (b.position(sq), b.snapshot(sq).copy()) for sq in range(B) if sq not in ids}
    r = b.verify([toks[sq] for sq in ids], want_logits=True, seq_ids=ids)
    for slot, sq in enumerate(ids):
        acc, em, lg, pos = alone[sq]
        assert int(r.accepted[slot]) == acc and np.array_equal(r.emitted[slot, :acc + 1], em[:acc + 1])
        assert np.array_equal(r.logits[slot].view(np.uint32), lg.view(np.uint32))
        assert b.position(sq) == pos
        assert np.array_equal(b.snapshot(sq), a.snapshot(sq))
    for sq, (pos, snap) in before.items():
        assert b.position(sq) == pos and np.array_equal(b.snapshot(sq), snap)
    # next step, other order and another subset; against the oracle for one of them
    st = yo.State(om, 96, yo.KV_F16)
    prompt = synth.uniform_i32(11 + 3 * 6, 0, V, 506).tolist()
    lo = st.forward(prompt)
    acc6, em6, _ = st.verify_chain(yo.argmax(lo), np.array(toks[6][1:], np.int32))
    assert alone[6][0] == acc6 and alone[6][1][:acc6 + 1].tolist() == em6.tolist()
    nxt6 = [int(em6[-1])] + synth.uniform_i32(N - 1, 0, V, 700).tolist()
    nxt2 = [pend[2]] + synth.uniform_i32(N - 1, 0, V, 701).tolist()
    r2 = b.verify([nxt6, nxt2], want_logits=True, seq_ids=[6, 2])
    acc_o, em_o, log_o = st.verify_chain(nxt6[0], np.array(nxt6[1:], np.int32), want_logits=True)
    assert float(np.max(np.abs(r2.logits[0] - log_o))) <= LOGIT_TOL
    assert int(r2.accepted[0]) == acc_o and r2.emitted[0, :acc_o + 1].tolist() == em_o.tolist()
    with pytest.raises(cuda.YuukaError):
        b.verify([nxt6, nxt2], seq_ids=[3, 3])           # a sequence twice
    with pytest.raises(cuda.YuukaError):
        b.verify([nxt6, nxt2], seq_ids=[3, 8])           # outside the session
    a.close(); b.close(); st.close()


def test_copy_block_gives_a_private_copy_of_a_shared_prefix(tiny):
    """KVPool.CopyBlock (model/qwen35/kv_pool.go:156-170): sequence 1 adopts sequence 0's prefix by pointing its
    table at 0's full blocks and at a copy of the partly filled one; its logits then equal sequence 0's, and
    what it appends lands in its own copy."""
    cfg, gm, om = tiny
    V, bs, cap = cfg["vocab"], 16, 64
    per = cap // bs
    sess = cuda.Session(gm, max_batch=2, max_nodes=4, capacity=cap, kv_format=cuda.KV_F16, block_size=bs)
    prompt = synth.uniform_i32(24, 0, V, 800)            # one full block and half of the next
    sess.forward(prompt, seq=0, want_logits=False)
    # sequence 1: blocks of sequence 0 are 0..3, its own are 4..7
    sess.copy_block(5, 1)
    sess.set_block_table(1, [0, 5, 6, 7])
    sess.restore(sess.snapshot(0), seq=1)
    sess.set_position(1, 24)
    nxt = synth.uniform_i32(3, 0, V, 801)
    a = sess.forward(nxt, seq=0)
    b = sess.forward(nxt, seq=1)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # the two sequences now diverge without disturbing one another
    a2 = sess.forward([7], seq=0)
    b2 = sess.forward([9], seq=1)
    a3 = sess.forward([11], seq=0)
    st = yo.State(om, cap, yo.KV_F16)
    st.forward(prompt.tolist() + nxt.tolist() + [7])
    assert float(np.max(np.abs(a3 - st.step(11)))) <= LOGIT_TOL
    assert not np.array_equal(a2, b2)
    with pytest.raises(cuda.YuukaError):
        sess.copy_block(99, 0)
    sess.close(); st.close()


def test_a_step_cannot_be_launched_twice_before_it_is_fetched(tiny):
    cfg, gm, om = tiny
    sess = cuda.Session(gm, max_batch=1, max_nodes=4, capacity=32)
    sess.forward([1, 2, 3], want_logits=False)
    sess.stage([[5, 6, 7]])
    sess.launch()
    with pytest.raises(cuda.YuukaError):
        sess.launch()                                    # would run and commit the same step again
    snap = sess.snapshot()                               # reading the state behind the step is fine
    for call in (lambda: sess.reset(0), lambda: sess.set_position(0, 2), lambda: sess.restore(snap)):
        with pytest.raises(cuda.YuukaError):
            call()                                       # the fetch would add to positions these calls replace
    res = sess.fetch()
    assert sess.position() == 3 + int(res.accepted[0]) + 1
    sess.close()


def test_a_refused_batch_does_not_leave_the_earlier_staged_step_launchable(tiny):
    cfg, gm, om = tiny
    sess = cuda.Session(gm, max_batch=1, max_nodes=4, capacity=32)
    sess.forward([1, 2, 3], want_logits=False)
    sess.stage([[5, 6, 7]])
    with pytest.raises(cuda.YuukaError):
        sess.stage([[5, 6, cfg["vocab"]]])               # refused after two of its rows replaced the staged ones
    with pytest.raises(cuda.YuukaError):
        sess.launch()                                    # nothing is staged any more
    res = sess.verify([[5, 6, 7]])
    assert sess.position() == 3 + int(res.accepted[0]) + 1
    sess.close()


def test_more_step_shapes_than_the_session_keeps_captured(tiny):
    """A session replays a captured launch sequence per step shape and keeps a bounded number of them (48,
    least recently used dropped first). 60 shapes (4 batch sizes x 15 row counts) run through one session; the
    first shape, whose capture has been dropped by then, must give the same bits when it runs again."""
    cfg, gm, om = tiny
    V = cfg["vocab"]
    sess = cuda.Session(gm, max_batch=4, max_nodes=15, capacity=64, kv_format=cuda.KV_F32)
    for b in range(4):
        sess.forward(synth.uniform_i32(6 + b, 0, V, 950 + b).tolist(), seq=b, want_logits=False)
    rows = synth.uniform_i32(4 * 15, 0, V, 960).reshape(4, 15)

    def run(batch, nodes):
        return sess.verify([rows[b, :nodes].tolist() for b in range(batch)], mode=cuda.ACCEPT_NONE,
                           want_logits=True).logits.copy()

    first = run(1, 1)
    mid = run(3, 7)
    for batch in range(1, 5):
        for nodes in range(1, 16):
            run(batch, nodes)
    assert np.array_equal(run(1, 1).view(np.uint32), first.view(np.uint32))
    assert np.array_equal(run(3, 7).view(np.uint32), mid.view(np.uint32))
    sess.close()


def test_an_expired_device_wait_is_reported_once_and_the_path_keeps_working(tiny):
    """Every wait inside a kernel is bounded; when one runs out the kernel sets a device error word and
    carries on, and the step that sees the word fails with YUUKA_ERR_DEVICE. The wait is made to run out in
    the safe way: a test flag makes the GEMM kernels of the session never issue the copies of their
    activations (nothing is in flight when a CTA exits) and give up after a short limit. The failing step is
    reported once, the word is cleared, and the same session then verifies correctly again."""
    cfg, gm, om = tiny
    V = cfg["vocab"]
    prompt = synth.uniform_i32(20, 0, V, 901).tolist()
    rows = synth.uniform_i32(5, 0, V, 902).tolist()
    st = yo.State(om, 64, yo.KV_F32)
    st.forward(prompt)
    _, _, want = st.verify_chain(rows[0], np.array(rows[1:], np.int32), want_logits=True)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=64, kv_format=cuda.KV_F32)
    sess.forward(prompt, want_logits=False)
    snap, pos = sess.snapshot(), sess.position()
    good = sess.verify([rows], mode=cuda.ACCEPT_NONE, want_logits=True).logits[0].copy()
    assert float(np.max(np.abs(good - want))) <= LOGIT_TOL
    sess.set_flags(cuda.SESSION_TEST_DROP_COPIES)
    with pytest.raises(cuda.YuukaError) as e:
        sess.verify([rows], mode=cuda.ACCEPT_NONE, want_logits=True)
    assert e.value.status == cuda.ERR_DEVICE and "bounded wait" in str(e.value)
    # the flag off again: the word was cleared when it was reported, the session and the device still answer
    sess.set_flags(0)
    sess.restore(snap)
    sess.set_position(0, pos)
    again = sess.verify([rows], mode=cuda.ACCEPT_NONE, want_logits=True).logits[0]
    assert np.array_equal(again.view(np.uint32), good.view(np.uint32))
    # the kernel-level entry point carries the same hook; the next step of any session reports it
    dev = gm.dev
    stream = dev.stream()
    n_out, n_in = 64, 256
    w = synth.normal_quant(n_out, n_in, synth.Q8_0, 0.02, 3)
    raw = dev.upload(w)
    wb = dev.alloc(cuda.tiled_bytes(synth.Q8_0, n_out, n_in) + 256)
    cuda.tile_weights(stream, wb, raw, synth.Q8_0, n_out, n_in)
    xb = dev.upload(synth.normal_f32(4 * n_in, 1.0, 4))
    ob = dev.alloc(4 * n_out * 4)
    cuda.gemm_quant(stream, ob, xb, wb, n_in, n_out, 4, synth.Q8_0, cuda.F32, cuda.PATH_MMA,
                    flags=cuda.GEMM_TILED | cuda.GEMM_TEST_DROP_COPIES)
    stream.synchronize()
    with pytest.raises(cuda.YuukaError) as e:
        sess.verify([rows], mode=cuda.ACCEPT_NONE)
    assert e.value.status == cuda.ERR_DEVICE
    ok = sess.verify([rows], mode=cuda.ACCEPT_NONE, want_logits=True).logits[0]
    assert np.array_equal(ok.view(np.uint32), good.view(np.uint32))
    for b in (raw, wb, xb, ob):
        b.free()
    stream.destroy()
    sess.close(); st.close()
