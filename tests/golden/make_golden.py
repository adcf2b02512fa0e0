#!/usr/bin/env python
"""Regenerates tests/golden/c0_tiny.npz from the CPU oracle.

The reference is Go and cannot run where this repository is built, so these
vectors are outputs of the oracle (the C restatement of model/qwen35 and
engine/speculative.go), frozen so that a later change of the oracle or of the
kernels shows up as a diff. They pin the C0 configuration: tiny qwen35 model
(hidden 256, 4 layers, vocab 4096, Q8_0 weights, seed 7), 48-token prompt, a
chain verify with k=4, and a 17-row tree verify.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import pyoracle as yo  # noqa: E402
from yuuka_b200 import synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "c0_tiny.npz")
SAMPLE = np.arange(0, 4096, 61)  # logit columns kept per row


def build():
    cfg = synth.tiny_config()
    tensors = synth.make_model(cfg, "q8_0", seed=7, unit_norms=False)
    om = yo.Model(cfg, tensors)
    V = cfg["vocab"]
    prompt = synth.uniform_i32(48, 0, V, 24)
    out = {"prompt": prompt, "sample_cols": SAMPLE}
    for kv_name, kv in (("f32", yo.KV_F32), ("f16", yo.KV_F16), ("q8_0", yo.KV_Q8_0)):
        st = yo.State(om, 128, kv)
        rows = st.prefill_logits(prompt)
        out[f"prefill_argmax_{kv_name}"] = np.array([yo.argmax(r) for r in rows], np.int32)
        out[f"prefill_logits_{kv_name}"] = rows[:, SAMPLE].astype(np.float32)
        st.close()
    # greedy continuation and the chain verify of a draft whose third token is wrong
    st = yo.State(om, 128, yo.KV_F32)
    logits = st.forward(prompt)
    greedy = []
    for _ in range(8):
        t = yo.argmax(logits)
        greedy.append(t)
        logits = st.step(t)
    st.close()
    out["greedy"] = np.array(greedy, np.int32)
    draft = np.array(greedy[1:5], np.int32)
    draft[2] = (draft[2] + 7) % V
    st = yo.State(om, 128, yo.KV_F32)
    st.forward(prompt)
    acc, emitted, allv = st.verify_chain(greedy[0], draft, want_logits=True)
    out["chain_draft"] = draft
    out["chain_accepted"] = np.array([acc], np.int32)
    out["chain_emitted"] = emitted
    out["chain_logits"] = allv[:, SAMPLE].astype(np.float32)
    out["chain_position"] = np.array([st.pos], np.int32)
    out["chain_state_sum"] = np.array([np.abs(st.snapshot().view(np.float32)).astype(np.float64).sum()])
    st.close()
    # tree verify: the greedy path is rows 2, 8, 12
    parent = np.array(synth.tree_16(), np.int32)
    tokens = synth.uniform_i32(17, 0, V, 25)
    tokens[0] = greedy[0]
    tokens[2], tokens[8], tokens[12] = greedy[1], greedy[2], greedy[3]
    st = yo.State(om, 128, yo.KV_F16)
    st.forward(prompt)
    acc, path, emitted, allv = st.verify_tree_greedy(tokens, parent, want_logits=True)
    out["tree_parent"] = parent
    out["tree_tokens"] = tokens
    out["tree_accepted"] = np.array([acc], np.int32)
    out["tree_path"] = path
    out["tree_emitted"] = emitted
    out["tree_logits"] = allv[:, SAMPLE].astype(np.float32)
    st.close()
    # prompt lookup on a history with repeats
    hist = np.array([5, 6, 7, 5, 6, 8, 5, 6, 7, 5, 6], np.int32)
    out["lookup_history"] = hist
    out["lookup_draft"] = np.array(yo.lookup_draft(hist, 4, 2), np.int32)
    om.close()
    return out


if __name__ == "__main__":
    data = build()
    np.savez_compressed(OUT, **data)
    print(OUT, os.path.getsize(OUT), "bytes")
