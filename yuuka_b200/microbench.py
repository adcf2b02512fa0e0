"""Kernel-level verify microbench (random data).

GEMM shapes: packed weights K=2560 x N in {9216, 2560, 248320} (the last stored
as Q6_K, the others Q4_K), plus the 4B model's other shapes; activations bf16
N(0,1) with M in {1, 2, 4, 9, 16, 64, 576} rows. Each timed launch reads a
different copy of the weights (copies rotate through > 2x the L2 size), so the
reported GB/s are HBM reads, not L2 hits. Times are CUDA events on the
launching stream, mean over the timed launches after warm-up.

    python -m yuuka_b200.microbench [--shape N,K,dtype] [--rows 9] [--path auto|fp32|mma] [--iters 20]
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import cuda, synth

DTYPES = {"q4_k": synth.Q4_K, "q5_k": synth.Q5_K, "q6_k": synth.Q6_K, "q8_0": synth.Q8_0}
PATHS = {"auto": cuda.PATH_AUTO, "fp32": cuda.PATH_FP32, "mma": cuda.PATH_MMA}
DEFAULT_SHAPES = [(9216, 2560, "q4_k"), (2560, 2560, "q4_k"), (248320, 2560, "q6_k"), (18432, 2560, "q4_k"),
                  (12352, 2560, "q4_k"), (2560, 9216, "q6_k"), (2560, 4096, "q4_k")]
DEFAULT_ROWS = [1, 2, 4, 9, 16, 64, 576]


def bench_gemm(dev, n_out, n_in, dtype_name, rows, path, iters, warmup=3, l2_bytes=126 << 20):
    dtype = DTYPES[dtype_name]
    rb = synth.row_bytes(dtype, n_in)
    wbytes = n_out * rb
    tbytes = cuda.tiled_bytes(dtype, n_out, n_in)
    stride = (tbytes + 255) // 256 * 256
    copies = max(2, min(iters + warmup, -(-2 * l2_bytes // wbytes) + 1))
    # one generated matrix, replicated: the values do not matter for timing
    w = synth.normal_quant(min(n_out, 4096), n_in, dtype, 0.02, 1)
    reps = -(-n_out // min(n_out, 4096))
    w = np.tile(w, reps)[:wbytes]
    wb = dev.alloc(copies * stride + 256)
    raw = dev.upload(w)
    st0 = dev.stream()
    for c in range(copies):
        cuda.tile_weights(st0, wb, raw, dtype, n_out, n_in, dst_offset=c * stride)
    st0.synchronize()
    st0.destroy()
    raw.free()
    x = synth.normal_f32(rows * n_in, 1.0, 2)
    xb = dev.upload(cuda.to_bf16(x))
    ob = dev.alloc(rows * n_out * 4)
    stream = dev.stream()
    e0, e1 = dev.event(), dev.event()
    times = []
    for it in range(warmup + iters):
        off = (it % copies) * stride
        stream.record(e0)
        cuda.gemm_quant(stream, ob, xb, wb, n_in, n_out, rows, dtype, cuda.BF16, path, flags=cuda.GEMM_TILED,
                        w_offset=off, completion=e1)
        e1.wait()
        if it >= warmup:
            times.append(e0.elapsed_ms(e1))
    for b in (wb, xb, ob):
        b.free()
    stream.destroy()
    ms = float(np.mean(times))
    return {"n_out": n_out, "n_in": n_in, "dtype": dtype_name, "rows": rows, "path": path, "ms": ms,
            "ms_min": float(np.min(times)), "weight_gbs": wbytes / ms / 1e6,
            "tflops": 2.0 * rows * n_out * n_in / ms / 1e9, "copies": copies}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", help="N,K,dtype (repeatable)")
    ap.add_argument("--rows", action="append", type=int)
    ap.add_argument("--path", default="auto", choices=list(PATHS))
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    shapes = DEFAULT_SHAPES
    if args.shape:
        shapes = []
        for s in args.shape:
            n, k, d = s.split(",")
            shapes.append((int(n), int(k), d))
    rows = args.rows or DEFAULT_ROWS
    dev = cuda.Device(0)
    for n_out, n_in, d in shapes:
        for m in rows:
            r = bench_gemm(dev, n_out, n_in, d, m, PATHS[args.path], args.iters)
            r["path"] = args.path
            print(json.dumps(r), flush=True)
    dev.close()


if __name__ == "__main__":
    main()
