#!/usr/bin/env python
"""Benchmark of the speculative-decoding verify step.

Workload (N=1): the dense 4B-shaped qwen35 model with Q4_K_M-style mixed
quantization, batch 1, 512-token random prompt, chain draft k=8 whose tokens are
the model's own greedy continuation with each position replaced by a uniform
random id with probability 0.3, greedy acceptance. One "step" is one verify
step: k+1 = 9 rows through all layers and the LM head, on-device acceptance and
KV / recurrent-state commit. Data are synthetic (seeded random weights and
tokens).

N>1: one model replica and one sequence per GPU, no collective on the data
path (weak scaling); launched by torch.distributed.run, which is used only for
the barrier and the max-over-ranks reduction.

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "accepted_tokens_per_second"
UNIT = "tok/s"
K_DRAFT = 8
PROMPT_LEN = 512
P_CORRUPT = 0.3
# expected emitted tokens per step at per-token acceptance 0.7, k = 8: sum_{i=0..8} 0.7^i
EXPECTED_EMITTED = sum(0.7 ** i for i in range(K_DRAFT + 1))


def workload_config(args) -> dict:
    return {
        "workload": "configs[2]: dense 4B-shaped qwen35 (hidden 2560, 32 layers 3 GDN:1 attention, FFN 9216, "
                    "vocab 248320), Q4_K_M-style quantization, batch 1 per GPU, 512-token prompt, chain k=8, "
                    "greedy, drafts = greedy continuation corrupted with p=0.3",
        "layers": args.layers, "rows_per_step": K_DRAFT + 1, "kv_format": "F16", "prompt_len": PROMPT_LEN,
        "l2": "no flush needed: each step streams 2.7 GB of weights, 21x the 126 MB L2",
        "parallelism": f"replicas x{args.gpus}, one sequence per GPU, no collective",
    }


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c > 0]
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm

def cpu_reference_sample(steps: int, warmup: int, threads: int = 0) -> dict:
    """Times the CPU reference algorithm (oracle port: one forwardOne per draft
    row, row-parallel matvec) on a bounded sample of the workload: one row
    through the first 4 layers (3 GDN + 1 attention) and the full LM head. The
    reference runs the 9 rows of a step one after the other and the eight layer
    groups are identical in shape, so a step costs 9 x (8 x layer-group + head)."""
    from oracle import pyoracle as yo
    from yuuka_b200 import synth

    # all host cores, whatever OMP_NUM_THREADS says (torch.distributed.run sets it to 1)
    yo.lib().yo_set_threads(threads if threads > 0 else (os.cpu_count() or 1))
    cores = yo.lib().yo_get_threads()
    cfg = synth.dense4b_config(layers=4, context=64)
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    model = yo.Model(cfg, tensors)
    rows = K_DRAFT + 1
    toks = synth.uniform_i32(1, 0, cfg["vocab"], 5)
    _, out_w, out_rows, out_cols = tensors["output.weight"]
    out_dtype = tensors["output.weight"][0]
    x = synth.normal_f32(cfg["hidden"], 1.0, 9).reshape(1, -1)
    times = []
    for it in range(warmup + steps):
        st = yo.State(model, 64, yo.KV_F16)
        t0 = time.perf_counter()
        st.prefill_logits(toks)                      # one forwardOne incl. the LM head
        t1 = time.perf_counter()
        yo.matmul(out_w, out_dtype, out_rows, out_cols, x)
        t2 = time.perf_counter()
        st.close()
        head = t2 - t1
        group = (t1 - t0) - head
        if it >= warmup:
            times.append(rows * (8 * group + head))
    model.close()
    step_s = float(np.mean(times))
    return {"value": EXPECTED_EMITTED / step_s, "unit": UNIT, "cores": cores, "kind": "port",
            "ms_per_step": step_s * 1e3,
            "sample": f"{steps} x [one row through layers 0-3 + full LM head on the CPU oracle]; step time = "
                      f"9 rows x (8 x layer-group + head); emitted tokens per step taken as {EXPECTED_EMITTED:.3f} (p=0.7, k=8)"}


def run_reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    base = cpu_reference_sample(args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference is Go and cannot be built here (no Go toolchain); this arm times this "
                    "repository's C restatement of its CPU path on the host cores"}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm

def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def run_gpu_arm(args, rank: int, local_rank: int, world: int) -> None:
    from yuuka_b200 import cuda, synth

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    cfg = synth.dense4b_config(layers=args.layers, context=4096)
    t_gen = time.perf_counter()
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    t_gen = time.perf_counter() - t_gen
    dev = cuda.Device(local_rank)
    model = cuda.Model(dev, cfg, tensors)
    weight_bytes = model.weight_bytes
    del tensors
    rows = K_DRAFT + 1
    total_steps = args.warmup + args.steps
    capacity = PROMPT_LEN + total_steps * rows + 64
    sess = cuda.Session(model, max_batch=1, max_nodes=rows, capacity=capacity, kv_format=cuda.KV_F16)

    # prompt, then the model's own greedy continuation (single-row steps), then rewind
    prompt = synth.uniform_i32(PROMPT_LEN, 0, cfg["vocab"], 100 + rank)
    logits = sess.forward(prompt)
    snap, pos = sess.snapshot(), sess.position()
    n_cont = total_steps * rows + rows
    # greedy continuation through the same 9-row kernels the timed steps use (row 0 of a step whose
    # drafts are dummies), so that near-ties resolve the same way in both passes
    cont_list: list[int] = []
    first = int(np.argmax(logits))
    pend = first
    dummy = [0] * K_DRAFT
    while len(cont_list) < n_cont:
        r0 = sess.verify([[pend] + dummy])
        a0 = int(r0.accepted[0])
        cont_list.extend(int(t) for t in r0.emitted[0, :a0 + 1])
        pend = cont_list[-1]
    cont = np.array(cont_list[:n_cont], np.int32)
    sess.restore(snap)
    sess.set_position(0, pos)
    drafts = synth.corrupt_draft(cont, cfg["vocab"], P_CORRUPT, 7 + rank)

    ev0, ev1 = dev.event(), dev.event()
    pending, idx = first, 0
    emitted_total, accepted_total, dev_ms = 0, 0, 0.0
    sampler = ClockSampler(local_rank)
    launches = 0

    def barrier():
        sess_stream_sync()
        if dist is not None:
            dist.barrier()

    def sess_stream_sync():
        cuda.check(cuda.lib().yuuka_stream_synchronize(sess.stream_handle()))

    t_e2e = 0.0
    for step in range(total_steps):
        if step == 0:
            sampler.start()
        if step == args.warmup:
            barrier()
            emitted_total = accepted_total = 0
            dev_ms = 0.0
            t_e2e = time.perf_counter()
        toks = np.concatenate(([pending], drafts[idx:idx + K_DRAFT])).astype(np.int32)
        sess.stage(toks)                       # host -> device: tokens and row metadata
        sess.record(ev0)
        sess.launch(ev1)                       # kernels only, no host synchronisation
        res = sess.fetch()                     # device -> host: accepted count and tokens
        dev_ms += ev0.elapsed_ms(ev1)
        a = int(res.accepted[0])
        emitted_total += a + 1
        accepted_total += a
        idx += a + 1
        pending = int(res.emitted[0, a])
        launches = sess.last_launch_count
    barrier()
    t_e2e = time.perf_counter() - t_e2e
    clocks = sampler.stop()

    # per-op attribution on three more steps (events around every op; not part of the timed region)
    per_op: dict[str, float] = {}
    prof_steps = 3
    for _ in range(prof_steps):
        toks = np.concatenate(([pending], drafts[idx:idx + K_DRAFT])).astype(np.int32)
        sess.stage(toks)
        for code, ns in sess.launch_profiled():
            name = cuda.OP_NAMES.get(code, str(code))
            per_op[name] = per_op.get(name, 0.0) + ns / 1e6 / prof_steps
        res = sess.fetch()
        a = int(res.accepted[0])
        idx += a + 1
        pending = int(res.emitted[0, a])
    gemm_ms = per_op.get("gemm", 0.0) + per_op.get("lm_head", 0.0)
    ctx_mid = PROMPT_LEN + (idx // 2)

    # max over ranks of the timed region, sum of tokens
    from yuuka_b200 import replicas
    tot = replicas.reduce_totals(dist, "cuda", dev_ms, t_e2e, float(emitted_total), float(accepted_total))
    dev_ms, t_e2e, emitted_all = tot.device_ms, tot.wall_s, tot.emitted

    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_per_step = dev_ms / args.steps
        kv_bytes = ctx_mid * 2 * cfg["kv_heads"] * cfg["head_dim"] * 2 * (args.layers // 4)
        state_bytes = 2 * (args.layers - args.layers // 4) * (cfg["time_step_rank"] * cfg["state_size"] ** 2 * 4)
        step_bytes = weight_bytes + kv_bytes + state_bytes
        # GEMM time inside the timed region: the timed steps run as one graph replay with dependent launches, so
        # single kernels cannot be bracketed there; the event pairs of the profiled steps (serialised, each op
        # with its launch latency) give the GEMM family's SHARE of a step, which is applied to the timed step
        prof_total = sum(per_op.values())
        gemm_share = gemm_ms / prof_total if prof_total > 0 else 0.0
        gemm_timed_ms = gemm_share * ms_per_step
        gemm_gbs = weight_bytes / (gemm_timed_ms * 1e-3) / 1e9 if gemm_timed_ms > 0 else 0.0
        line = {
            "metric": METRIC, "value": emitted_all / (dev_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate (weights Q4_K/Q6_K)",
            "data": "synthetic", "config": workload_config(args),
            "accepted_per_step": accepted_total / args.steps, "emitted_per_step": emitted_total / args.steps,
            "e2e": {"value": emitted_all / t_e2e, "unit": UNIT, "ms_per_step": t_e2e / args.steps * 1e3,
                    # one copy in: ancestor masks, tokens, parents, depths; one copy out: accepted count, path, emitted
                    # tokens, plus the two device error words
                    "h2d_bytes_per_step": rows * (8 + 4 + 4 + 4), "d2h_bytes_per_step": 4 + 2 * rows * 4 + 8},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "gemm_tiled_mma_kernel (every quantized GEMM launch of a step, LM head included)",
                         "achieved": gemm_gbs, "peak": peak, "unit": "GB/s", "frac": gemm_gbs / peak,
                         "peak_source": peak_kind, "bytes_per_step": weight_bytes, "ms_per_step": gemm_timed_ms,
                         "share_of_step": gemm_share, "profiled_ms_per_step": gemm_ms,
                         # DRAM read / algorithmic ratio of the ncu captures under profiles/ (1.004 Q4_K, 1.002 Q6_K)
                         "traffic": int(weight_bytes * 1.003), "traffic_source": "ncu dram__bytes_read of two GEMM "
                         "shapes, scaled by bytes processed",
                         "launches_per_step": 137},
            "step_roofline": {"bytes_per_step": step_bytes, "weights": weight_bytes, "kv": kv_bytes,
                              "recurrent_state": state_bytes, "achieved_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                              "frac_of_measured_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                              "frac_of_8tbs": step_bytes / (ms_per_step * 1e-3) / 1e9 / 8000.0},
            "per_op_ms": {k: round(v, 4) for k, v in sorted(per_op.items(), key=lambda kv: -kv[1])},
            "setup": {"weight_gen_s": round(t_gen, 1), "device": dev.info().name.decode()},
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_reference_sample(steps=8, warmup=2)
        print(json.dumps(line), flush=True)

    sess.close()
    model.close()
    dev.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
