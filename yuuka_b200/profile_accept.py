"""A short run of the acceptance stage on its own, for profilers.

    python -m yuuka_b200.profile_accept [--batch 8] [--nodes 9] [--vocab 248320] [--iters 3]

Uploads fp32 logits N(0, 3) and draft distributions (softmax of the parent row's logits / T plus N(0, 1)
noise), draws the drafts from them and runs yuuka_accept_tree in both modes (rejection sampling at T = 0.7,
greedy). Prints the time of the acceptance kernels measured with CUDA events.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import cuda


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--nodes", type=int, default=9)
    ap.add_argument("--vocab", type=int, default=248320)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    B, N, V, T = args.batch, args.nodes, args.vocab, 0.7
    rng = np.random.default_rng(1)
    logits = (3.0 * rng.standard_normal((B, N, V), dtype=np.float32)).astype(np.float32)
    q = np.empty_like(logits)
    q[:, 0] = 0.0
    q[:, 1:] = logits[:, :-1] / T + rng.standard_normal((B, N - 1, V), dtype=np.float32)
    q -= q.max(axis=-1, keepdims=True)
    np.exp(q, out=q)
    q /= q.sum(axis=-1, keepdims=True)
    tokens = np.zeros((B, N), np.int32)
    tokens[:, 0] = rng.integers(0, V, B)
    for b in range(B):
        for c in range(1, N):
            cdf = np.cumsum(q[b, c], dtype=np.float64)
            tokens[b, c] = min(int(np.searchsorted(cdf, rng.random() * cdf[-1])), V - 1)
    uniforms = np.minimum(rng.random((B, N, 2), dtype=np.float32), np.float32(0.99999994))
    dev = cuda.Device(0)
    lb, qb = dev.upload(logits), dev.upload(q)
    stream = dev.stream()
    e0, e1 = dev.event(), dev.event()
    out = {}
    for mode, name in ((cuda.ACCEPT_REJECTION, "rejection"), (cuda.ACCEPT_GREEDY, "greedy")):
        times = []
        for _ in range(args.iters):
            acc, _, _ = cuda.accept_tree(stream, lb, tokens, V, mode=mode, temperature=T, draft_probs=qb, uniforms=uniforms,
                                         begin=e0, end=e1)
            times.append(e0.elapsed_ms(e1))
        out[name] = {"ms": times, "mean_accepted": float(acc.mean())}
    print(json.dumps({"batch": B, "nodes": N, "vocab": V, "logit_bytes": B * N * V * 4, **out}))
    lb.free(); qb.free()
    stream.destroy()
    dev.close()


if __name__ == "__main__":
    main()
