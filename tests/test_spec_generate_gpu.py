"""yuuka_spec_generate (host loop of engine/speculative.go over the k+1-row verify
step) on the tiny model: the emitted stream must equal plain greedy decoding by
the CPU oracle, which is the property the reference's own
TestSpeculative*MatchesGreedy tests assert (engine/speculative_test.go:103-137)."""
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
    om = yo.Model(cfg, tensors)
    yield cfg, gm, om
    gm.close()
    dev.close()


def oracle_greedy(om, prompt, n, capacity=256):
    st = yo.State(om, capacity, yo.KV_F32)
    logits = st.forward(prompt)
    out, gaps = [], []
    for _ in range(n):
        top2 = np.partition(logits, -2)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        t = yo.argmax(logits)
        out.append(t)
        if len(out) < n:
            logits = st.step(t)
    st.close()
    return out, gaps


def agree(got, want, gaps):
    """Identical tokens, except that a near-tie (top-2 gap < 1e-3) may legitimately fork the stream."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert gaps[i] < 1e-3, f"token {i}: got {g}, want {w}, top-2 gap {gaps[i]}"
            return i
    return len(want)


def damped_model(cfg, dev, scale):
    """The tiny model with its mixer output projections scaled down: at 0 the next token depends on
    the current token only, so greedy decoding falls into a cycle that prompt lookup predicts; at
    0.1 the cycle is broken often enough that most drafts are wrong."""
    tensors = synth.make_model(cfg, "q8_0", seed=7, unit_norms=False)
    for name, (d, arr, r, c) in list(tensors.items()):
        if name.endswith("ssm_out.weight") or name.endswith("attn_output.weight"):
            tensors[name] = (d, synth.normal_quant(r, c, d, 0.02 * scale, 999 + r), r, c)
    return cuda.Model(dev, cfg, tensors), yo.Model(cfg, tensors)


@pytest.mark.parametrize("scale,min_match", [(0.0, 2), (0.1, 1)])
def test_generate_matches_greedy_decoding(tiny, scale, min_match):
    cfg, gm0, om0 = tiny
    gm, om = damped_model(cfg, gm0.dev, scale)
    V = cfg["vocab"]
    prompt = synth.uniform_i32(12, 0, V, 70).tolist()
    n = 300
    want, gaps = oracle_greedy(om, prompt, n, capacity=512)
    sess = cuda.Session(gm, max_batch=1, max_nodes=9, capacity=512, kv_format=cuda.KV_F32)
    got, res = cuda.spec_generate(sess, prompt, n, max_draft=8, min_match=min_match)
    same = agree(got, want, gaps)
    assert same >= 150, f"stream forked at a near-tie after {same} tokens; pick another seed"
    assert len(got) == n and res.output_tokens == n and res.prompt_tokens == len(prompt)
    assert res.finish_reason == cuda.FINISH_LENGTH
    assert res.draft_tokens > 50 and 0 <= res.accepted_draft <= res.draft_tokens
    if scale == 0.0:
        assert res.accepted_draft > res.draft_tokens // 2 and res.steps < n // 2   # the cycle is predicted
    else:
        assert res.accepted_draft < res.draft_tokens // 2                          # mostly corrections
    assert res.steps + res.accepted_draft == n - 1  # every step emits its accepted drafts plus one token
    assert sess.position() == len(prompt) + n - 1   # the last emitted token is pending, not run
    # the same request again (the call resets the sequence) gives the same stream
    again, res2 = cuda.spec_generate(sess, prompt, n, max_draft=8, min_match=min_match)
    assert again == got and (res2.steps, res2.draft_tokens, res2.accepted_draft) == (res.steps, res.draft_tokens, res.accepted_draft)
    sess.close()
    gm.close()


def test_generate_stops_on_stop_token_and_on_capacity(tiny):
    cfg, gm, om = tiny
    V = cfg["vocab"]
    base = synth.uniform_i32(10, 0, V, 71).tolist()
    prompt = base + base
    want, gaps = oracle_greedy(om, prompt, 24)
    sess = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=64, kv_format=cuda.KV_F16)
    stop = want[9]
    first = want.index(stop)
    got, res = cuda.spec_generate(sess, prompt, 24, max_draft=4, stop_tokens=[stop, V - 1])
    assert res.finish_reason == cuda.FINISH_STOP and got == want[:first]
    # max_tokens is clipped to the free context: capacity 64 - 20 prompt tokens = 44
    got, res = cuda.spec_generate(sess, prompt, 1000, max_draft=16)
    assert res.finish_reason == cuda.FINISH_LENGTH and len(got) == 44
    assert sess.position() <= 64
    want44, gaps44 = oracle_greedy(om, prompt, 44, capacity=64)
    assert agree(got, want44, gaps44) >= 24
    # a session of one row per step cannot draft and still decodes
    one = cuda.Session(gm, max_batch=1, max_nodes=1, capacity=64, kv_format=cuda.KV_F32)
    got1, res1 = cuda.spec_generate(one, prompt, 12)
    assert agree(got1, want[:12], gaps[:12]) == 12 and res1.draft_tokens == 0 and res1.steps == 11
    one.close()
    sess.close()


def test_generate_argument_errors(tiny):
    cfg, gm, om = tiny
    sess = cuda.Session(gm, max_batch=1, max_nodes=4, capacity=32, kv_format=cuda.KV_F32)
    for prompt, n in (([], 4), ([1, 2, 3], 0), (list(range(33)), 4), (list(range(32)), 4)):
        with pytest.raises(cuda.YuukaError) as e:
            cuda.spec_generate(sess, prompt, n)
        assert e.value.status == 1
    sess.close()


def test_generate_after_a_long_prompt(tiny):
    """A 200-token prompt goes in as one wide pass (GEMMs over all rows, mixers in 64-row sub-chunks) before
    the verify loop starts; the stream still equals greedy decoding."""
    cfg, gm0, om0 = tiny
    gm, om = damped_model(cfg, gm0.dev, 0.0)
    prompt = synth.uniform_i32(200, 0, cfg["vocab"], 71).tolist()
    n = 80
    want, gaps = oracle_greedy(om, prompt, n, capacity=512)
    sess = cuda.Session(gm, max_batch=1, max_nodes=9, capacity=512, kv_format=cuda.KV_F16)
    got, res = cuda.spec_generate(sess, prompt, n, max_draft=8, min_match=2)
    same = agree(got, want, gaps)
    assert same >= 40, f"stream forked at a near-tie after {same} tokens; pick another seed"
    assert res.prompt_tokens == 200 and res.output_tokens == n and sess.position() >= 200 + n - 1
    sess.close(); gm.close()


def test_generation_on_another_sequence_of_the_session(tiny):
    """Sequence 2 of a three-sequence session generates the stream sequence 0 would, and leaves the others alone."""
    cfg, gm, om = tiny
    prompt = synth.uniform_i32(20, 0, cfg["vocab"], 31).tolist()
    want, gaps = oracle_greedy(om, prompt, 24)
    sess = cuda.Session(gm, max_batch=3, max_nodes=5, capacity=128, kv_format=cuda.KV_F32)
    sess.forward([3, 4, 5], seq=0, want_logits=False)
    got, res = cuda.spec_generate(sess, prompt, 24, max_draft=4, min_match=2, seq=2)
    n = agree(got, want, gaps)
    assert n >= 8
    assert sess.position(0) == 3 and sess.position(1) == 0
    assert sess.position(2) == len(prompt) + res.output_tokens - 1 or sess.position(2) == len(prompt) + res.output_tokens
    sess.close()


def test_device_lookup_draft_equals_the_host_lookup():
    """lookupDraft on the device against yuuka_spec_lookup_draft: the reference's three vectors
    (engine/speculative_test.go:139-151) and random histories over a small alphabet (many repeats)."""
    dev = cuda.Device(0)
    cases = [([1, 2, 3, 4, 1, 2], 3, 2), ([1, 2, 3, 4], 3, 2), ([5, 6, 7, 5, 6, 8, 5, 6], 2, 2)]
    wants = [[3, 4, 1], [], [8, 5]]
    for (h, md, mm), want in zip(cases, wants):
        assert cuda.spec_lookup_draft(h, md, mm) == want
        assert cuda.spec_lookup_draft_device(dev, h, md, mm) == want
    rng = np.random.default_rng(9)
    for trial in range(60):
        n = int(rng.integers(1, 700))
        alphabet = int(rng.integers(2, 12))
        h = rng.integers(0, alphabet, n).astype(np.int32)
        md, mm = int(rng.integers(1, 17)), int(rng.integers(1, 9))
        assert cuda.spec_lookup_draft_device(dev, h, md, mm) == cuda.spec_lookup_draft(h, md, mm), (trial, n, md, mm)
    dev.close()


@pytest.mark.parametrize("scale,burst,min_match", [(0.0, 4, 2), (0.1, 3, 1), (1.0, 1, 2)])
def test_device_drafted_generation_emits_the_greedy_stream(tiny, scale, burst, min_match):
    """Steps of max_draft + 1 rows with the drafting between them on the device, `burst` steps per host
    synchronization: same tokens as the host loop and as greedy decoding by the oracle, with drafts that
    mostly hit (scale 0: the stream falls into a cycle), mostly miss (0.1) or hardly occur (the plain model)."""
    cfg, gm0, om0 = tiny
    if scale == 1.0:
        gm, om, owned = gm0, om0, False
    else:
        gm, om = damped_model(cfg, gm0.dev, scale)
        owned = True
    prompt = synth.uniform_i32(12, 0, cfg["vocab"], 70).tolist()
    n = 200
    want, gaps = oracle_greedy(om, prompt, n, capacity=512)
    a = cuda.Session(gm, max_batch=2, max_nodes=9, capacity=512, kv_format=cuda.KV_F32)
    host, res_h = cuda.spec_generate(a, prompt, n, max_draft=8, min_match=min_match)
    b = cuda.Session(gm, max_batch=2, max_nodes=9, capacity=512, kv_format=cuda.KV_F32)
    got, res_d = cuda.spec_generate_device(b, prompt, n, max_draft=8, min_match=min_match, seq=1, burst=burst)
    agreed = agree(got, want, gaps)
    assert agreed >= 100, f"stream forked at a near-tie after {agreed} tokens; pick another seed"
    assert len(got) == n and res_d.prompt_tokens == len(prompt) and res_d.finish_reason == cuda.FINISH_LENGTH
    if agreed == n:
        assert got == host
    assert 0 <= res_d.accepted_draft <= res_d.draft_tokens
    if scale == 0.0:
        # the cycle is predicted: most drafts are accepted and far fewer steps than tokens run
        assert res_d.accepted_draft > res_d.draft_tokens // 2 and res_d.steps < n // 2
        assert res_d.draft_tokens == res_h.draft_tokens or res_d.steps <= res_h.steps + burst
    elif scale == 0.1:
        assert res_d.draft_tokens > 20 and res_d.accepted_draft < res_d.draft_tokens // 2
    # a stop token ends the stream before it
    stop = got[30]
    cut, res_s = cuda.spec_generate_device(b, prompt, n, max_draft=8, min_match=min_match, seq=1, burst=burst, stop_tokens=[stop])
    assert cut == got[:got.index(stop)] and res_s.finish_reason == cuda.FINISH_STOP
    # capacity: generation ends when fewer than max_draft + 1 positions remain
    small = cuda.Session(gm, max_batch=1, max_nodes=5, capacity=40, kv_format=cuda.KV_F32)
    tail, res_c = cuda.spec_generate_device(small, prompt, 1000, max_draft=4, min_match=min_match, burst=burst)
    assert 40 - 12 - 5 <= len(tail) <= 40 - 12 and tail == got[:len(tail)] and small.position() <= 40
    a.close(); b.close(); small.close()
    if owned:
        gm.close(); om.close()
