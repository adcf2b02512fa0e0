"""The chunkwise (WY-form) Gated-DeltaNet scan of the prompt path against the oracle and against the row-by-row scan.

gdnChunkedScan (model/qwen35/recurrent.go:107-351) and gdnPerTokenScan (recurrent.go:56-105) are two forms of one
recurrence; the reference holds them to 1e-4 of each other, relative to the largest magnitude
(model/qwen35/recurrent_test.go:9-126). Prompts longer than 64 tokens run their delta-net layers in sub-chunks of
64 rows through the chunkwise kernel, which rewrites the state in place; YUUKA_CUDA_NO_GDN_CHUNK=1 (read when a
session is created) sends them through the row-by-row scan and the state commit instead.
"""
import os

import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth
from tests.test_parity_geometry_gpu import cosine, head_geometry_config

pytestmark = pytest.mark.gpu


def rel_diff(a, b):
    peak = float(np.max(np.abs(a)))
    diff = float(np.max(np.abs(a - b)))
    return diff if peak == 0 else diff / peak


def run_prompt(gm, prompt, capacity, chunked):
    if chunked:
        os.environ.pop("YUUKA_CUDA_NO_GDN_CHUNK", None)
    else:
        os.environ["YUUKA_CUDA_NO_GDN_CHUNK"] = "1"
    try:
        sess = cuda.Session(gm, max_batch=1, max_nodes=16, capacity=capacity, kv_format=cuda.KV_F32)
    finally:
        os.environ.pop("YUUKA_CUDA_NO_GDN_CHUNK", None)
    logits = sess.forward(prompt)
    snap = sess.snapshot().view(np.float32).copy()
    launches = sess.last_launch_count
    sess.close()
    return logits, snap, launches


@pytest.mark.parametrize("name,n_prompt", [("geometry", 200), ("geometry", 65), ("geometry", 128), ("tiny", 150)])
def test_prompt_through_the_chunkwise_scan(name, n_prompt):
    # geometry: state 128, 4 value heads over 2 key groups; tiny: state 64
    cfg = head_geometry_config() if name == "geometry" else synth.tiny_config()
    tensors = synth.make_model(cfg, "q4_k_m", seed=43, unit_norms=False)
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(n_prompt, 0, cfg["vocab"], 7 + n_prompt)
    st = yo.State(om, 256, yo.KV_F32)
    want = st.forward(prompt)
    want_snap = st.snapshot().view(np.float32).copy()
    st.close()
    got_c, snap_c, _ = run_prompt(gm, prompt, 256, True)
    got_r, snap_r, _ = run_prompt(gm, prompt, 256, False)
    # the two forms on the GPU. The first delta-net layer sees identical inputs in both runs: the reference's own
    # bar for the two forms applies to its state. Later layers inherit the first one's differences through GEMMs
    # with fp16-rounded operands (passes of 48 rows and more), hence the wider bar on the whole snapshot.
    def first_layer_state(snap):
        probe = yo.State(om, 256, yo.KV_F32)
        probe.restore(snap.view(np.uint8))
        out = probe.rec_s(0).copy()
        probe.close()
        return out
    assert rel_diff(first_layer_state(snap_r), first_layer_state(snap_c)) <= 1e-4
    assert rel_diff(snap_r, snap_c) <= 2e-3, rel_diff(snap_r, snap_c)
    assert float(np.max(np.abs(got_c - got_r))) <= 5e-3
    # and the chunkwise path against the oracle, bars of the other prompt tests
    err = float(np.max(np.abs(got_c - want)))
    assert err <= 2e-2 and cosine(got_c, want) >= 0.9999, (err, cosine(got_c, want))
    # (over 150-200 tokens the GEMMs' fp16-rounded operands move the state further from the fp32 path than over the
    # 40-token prompts of the other tests; the bar is the row-by-row path's own distance on the same prompt)
    err_r = float(np.max(np.abs(snap_r - want_snap)))
    assert float(np.max(np.abs(snap_c - want_snap))) <= max(2e-3, 1.25 * err_r)
    gm.close()
    dev.close()


def test_strong_decay_stays_finite():
    """Heads whose decay is strong enough for exp(-g) over a 64-row chunk to overflow in the reference's scaling:
    the kernel works with ratios exp(g_r - g_s) <= 1 only."""
    cfg = head_geometry_config()
    tensors = synth.make_model(cfg, "q4_k_m", seed=44, unit_norms=False)
    for name in [n for n in tensors if n.endswith("ssm_a")]:
        dtype, data, rows, cols = tensors[name]
        tensors[name] = (dtype, (data * np.float32(40.0)).astype(np.float32), rows, cols)  # log decay about -11 per row
    dev = cuda.Device(0)
    gm = cuda.Model(dev, cfg, tensors)
    om = yo.Model(cfg, tensors)
    prompt = synth.uniform_i32(130, 0, cfg["vocab"], 5)
    st = yo.State(om, 256, yo.KV_F32)
    want = st.forward(prompt)
    want_snap = st.snapshot().view(np.float32).copy()
    st.close()
    got, snap, _ = run_prompt(gm, prompt, 256, True)
    got_r, snap_r, _ = run_prompt(gm, prompt, 256, False)
    assert np.isfinite(got).all() and np.isfinite(snap).all()
    # with the state wiped at every row the layers pass the GEMMs' rounding straight on: the bar is the row-by-row
    # path's own distance from the fp32 path on this model
    err_r, serr_r = float(np.max(np.abs(got_r - want))), float(np.max(np.abs(snap_r - want_snap)))
    assert float(np.max(np.abs(got - want))) <= max(2e-2, 1.25 * err_r) and cosine(got, want) >= 0.9999
    assert float(np.max(np.abs(snap - want_snap))) <= max(2e-3, 1.25 * serr_r)
    assert rel_diff(snap_r, snap) <= 2e-3
    gm.close()
    dev.close()
