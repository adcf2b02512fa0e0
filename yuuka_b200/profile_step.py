"""A short run of verify steps on the 4B-shaped model, for profilers.

    python -m yuuka_b200.profile_step [--layers 32] [--prompt 64] [--steps 3] [--rows 9]

Builds the synthetic Q4_K_M model (dense 4B shape, or the qwen35moe shape with
--moe), feeds a short prompt to each of --batch sequences and runs a few verify
steps of --rows rows per sequence with dummy drafts. Set YUUKA_CUDA_NO_GRAPH=1 to launch the kernels
directly instead of replaying a captured graph (profilers then list them one
by one). With --profiler-range the steps (not the model set-up or the prompt), or with
--profiler-range prompt the prompt passes, run between cuProfilerStart and cuProfilerStop, for
`ncu --profile-from-start off`.
Prints the per-step time measured with CUDA events.
"""
from __future__ import annotations

import argparse
import ctypes
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
    ap.add_argument("--batch", type=int, default=1, help="sequences per step")
    ap.add_argument("--per-op", action="store_true", help="one more step with an event pair around every operation")
    ap.add_argument("--moe", action="store_true", help="qwen35moe shape (256 experts, 8 used) instead of the dense 4B shape")
    ap.add_argument("--profiler-range", nargs="?", const="steps", default=None, choices=["steps", "prompt"],
                    help="cuProfilerStart / Stop around the verify steps (default) or around the prompt passes")
    args = ap.parse_args()
    if args.moe:
        cfg = synth.moe_config(layers=args.layers, vocab=args.vocab, context=4096)
    else:
        cfg = synth.dense4b_config(layers=args.layers, vocab=args.vocab, context=4096)
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    dev = cuda.Device(0)
    model = cuda.Model(dev, cfg, tensors)
    del tensors
    cap = args.prompt + (args.steps + 2) * args.rows + 32
    B = args.batch
    sess = cuda.Session(model, max_batch=B, max_nodes=args.rows, capacity=cap, kv_format=cuda.KV_F16)
    pending = []
    driver = ctypes.CDLL("libcuda.so.1") if args.profiler_range else None
    if args.profiler_range == "prompt":
        driver.cuProfilerStart()
    for b in range(B):
        prompt = synth.uniform_i32(args.prompt, 0, cfg["vocab"], 3 + b)
        pending.append(int(np.argmax(sess.forward(prompt, seq=b))))
    if args.profiler_range == "prompt":
        driver.cuProfilerStop()
    e0, e1 = dev.event(), dev.event()
    times = []
    if args.profiler_range == "steps":
        driver.cuProfilerStart()
    for _ in range(args.steps):
        sess.stage([[pending[b]] + [1 + b] * (args.rows - 1) for b in range(B)])
        sess.record(e0)
        sess.launch(e1)
        res = sess.fetch()
        times.append(e0.elapsed_ms(e1))
        pending = [int(res.emitted[b, int(res.accepted[b])]) for b in range(B)]
    if args.profiler_range == "steps":
        driver.cuProfilerStop()
    per_op = {}
    if args.per_op:
        sess.stage([[pending[b]] + [1 + b] * (args.rows - 1) for b in range(B)])
        for code, ns in sess.launch_profiled():
            name = cuda.OP_NAMES.get(code, str(code))
            per_op[name] = round(per_op.get(name, 0.0) + ns / 1e6, 4)
        sess.fetch()
    print(json.dumps({"per_op_ms": per_op, "ms_per_step": times, "launches_per_step": sess.last_launch_count,
                      "weight_bytes": model.weight_bytes}))
    sess.close()
    model.close()
    dev.close()


if __name__ == "__main__":
    main()
