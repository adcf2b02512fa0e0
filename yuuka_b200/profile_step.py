"""A short run of verify steps on the 4B-shaped model, for profilers.

    python -m yuuka_b200.profile_step [--layers 32] [--prompt 64] [--steps 3] [--rows 9]

Builds the synthetic Q4_K_M model, feeds a short prompt and runs a few 9-row
verify steps with dummy drafts. Set YUUKA_CUDA_NO_GRAPH=1 to launch the kernels
directly instead of replaying a captured graph (profilers then list them one
by one). Prints the per-step time measured with CUDA events.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import cuda, synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--rows", type=int, default=9)
    ap.add_argument("--vocab", type=int, default=248320)
    args = ap.parse_args()
    cfg = synth.dense4b_config(layers=args.layers, vocab=args.vocab, context=4096)
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    dev = cuda.Device(0)
    model = cuda.Model(dev, cfg, tensors)
    del tensors
    cap = args.prompt + (args.steps + 2) * args.rows + 32
    sess = cuda.Session(model, max_batch=1, max_nodes=args.rows, capacity=cap, kv_format=cuda.KV_F16)
    prompt = synth.uniform_i32(args.prompt, 0, cfg["vocab"], 3)
    logits = sess.forward(prompt)
    pending = int(np.argmax(logits))
    e0, e1 = dev.event(), dev.event()
    times = []
    for _ in range(args.steps):
        sess.stage([[pending] + [1] * (args.rows - 1)])
        sess.record(e0)
        sess.launch(e1)
        res = sess.fetch()
        times.append(e0.elapsed_ms(e1))
        pending = int(res.emitted[0, int(res.accepted[0])])
    print(json.dumps({"ms_per_step": times, "launches_per_step": sess.last_launch_count,
                      "weight_bytes": model.weight_bytes}))
    sess.close()
    model.close()
    dev.close()


if __name__ == "__main__":
    main()
