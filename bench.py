#!/usr/bin/env python
"""Benchmark of the speculative-decoding verify step.

Default workload (configs[2], "c2"): the dense 4B-shaped qwen35 model with Q4_K_M-style mixed quantization,
batch 1, 512-token random prompt, chain draft k=8 whose tokens are the model's own greedy continuation with
each position replaced by a uniform random id with probability 0.3, greedy acceptance. One "step" is one
verify step: k+1 = 9 rows through all layers and the LM head, on-device acceptance and KV / recurrent-state
commit. Data are synthetic (seeded random weights and tokens).

N>1: one model replica per GPU and the sequences split over the GPUs, no collective on the data path (weak
scaling); launched by torch.distributed.run, which is used only for the barrier and the reduction of the
per-rank results.

--impl reference times the CPU restatement of the reference's own path (the reference is Go; there is no
toolchain for it here) on the host cores: real verify steps of the full model, after a shortened prompt.

--config c1 | c3 | c4 run the other named configurations and print the same JSON shape:
  c1  kernel microbenchmark: quantized GEMM sweep (rows x shapes) and the acceptance stage on its own
  c3  256 sequences / N GPUs, 16-node draft trees, rejection sampling at T = 0.8, contexts 256-3072, permuted
      block tables
  c4  qwen35moe shape, 32 sequences per GPU, chain k=4, greedy

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import re
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
DTYPE = "f16 tensor-core operands (exact integer weights, two-half activations), f32 accumulate; weights Q4_K/Q6_K"


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


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profiled_traffic_ratio() -> tuple[float | None, str]:
    """DRAM bytes read per algorithmic weight byte of the register-fed GEMM kernel, as the ncu capture summarised
    under profiles/ measured it (a line `dram_read_over_algorithmic: <ratio>` with the capture's date beside it)."""
    path = os.path.join(ROOT, "profiles", "gemm_tiled_mma_exact_rows9_layer_shapes.md")
    try:
        text = open(path).read()
    except OSError:
        return None, "no ncu summary found"
    m = re.search(r"dram_read_over_algorithmic:\s*([0-9.]+)", text)
    d = re.search(r"captured:\s*([0-9-]+)", text)
    if not m:
        return None, "no ratio in " + os.path.relpath(path, ROOT)
    return float(m.group(1)), f"{os.path.relpath(path, ROOT)} (ncu dram__bytes_read, captured {d.group(1) if d else '?'})"


# --------------------------------------------------------------------------- CPU arm

def cpu_reference_steps(steps: int, warmup: int, layers: int, tensors: dict | None = None, prompt_len: int = 16,
                        threads: int = 0, budget_s: float | None = None) -> dict:
    """Real verify steps of the CPU path (oracle port of engine/speculative.go over model/qwen35: one forwardOne
    per row, row-parallel matvec) on all host cores: the 32-layer model, `warmup + steps` 9-row steps whose drafts
    are the path's own greedy continuation corrupted with p = 0.3. The bounded part is the prompt (16 tokens
    instead of 512: a step of the CPU path reads the same weights whatever the context) and the number of steps:
    with budget_s the loop ends after the first timed step (of at least three) that finishes past that many seconds
    of stepping, and the result says how many steps were timed."""
    from oracle import pyoracle as yo
    from yuuka_b200 import synth

    # all host cores, whatever OMP_NUM_THREADS says (torch.distributed.run sets it to 1)
    yo.lib().yo_set_threads(threads if threads > 0 else (os.cpu_count() or 1))
    cores = yo.lib().yo_get_threads()
    if budget_s is not None:
        steps = min(steps, 400)                   # (bounds the context the two states are created with)
    total = warmup + steps
    cap = prompt_len + (total + 2) * (K_DRAFT + 1) + 16
    cfg = synth.dense4b_config(layers=layers, context=max(cap, 64))
    if tensors is None:
        tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    model = yo.Model(cfg, tensors)
    V = cfg["vocab"]
    prompt = synth.uniform_i32(prompt_len, 0, V, 100).tolist()
    st = yo.State(model, cap, yo.KV_F16)
    probe = yo.State(model, cap, yo.KV_F16)      # runs ahead of `st` to supply the greedy continuation
    logits = st.forward(prompt)
    plog = probe.forward(prompt)
    cont: list[int] = []
    u = synth.uniform_f32(cap, 7)
    r = synth.uniform_i32(cap, 0, V, 8)

    def need(n):
        nonlocal plog
        while len(cont) < n:
            t = yo.argmax(plog)
            cont.append(t)
            plog = probe.step(t)

    pending = yo.argmax(logits)
    need(1)
    idx = 1                                       # cont[0] is the pending token
    times, emitted_total, accepted_total = [], 0, 0
    t_begin = time.perf_counter()
    for step in range(total):
        if budget_s is not None and len(times) >= 3 and time.perf_counter() - t_begin > budget_s:
            break
        need(idx + K_DRAFT)
        drafts = np.array([r[idx + i] if u[idx + i] < P_CORRUPT else cont[idx + i] for i in range(K_DRAFT)], np.int32)
        t0 = time.perf_counter()
        acc, em, _ = st.verify_chain(pending, drafts)
        dt = time.perf_counter() - t0
        if step >= warmup:
            times.append(dt)
            emitted_total += acc + 1
            accepted_total += acc
        idx += acc + 1
        pending = int(em[-1])
    st.close()
    probe.close()
    model.close()
    total_s = float(np.sum(times))
    return {"value": emitted_total / total_s, "unit": UNIT, "cores": cores, "kind": "port",
            "ms_per_step": total_s / max(len(times), 1) * 1e3, "emitted_per_step": emitted_total / max(len(times), 1),
            "accepted_per_step": accepted_total / max(len(times), 1), "steps": len(times),
            "sample": f"{len(times)} real 9-row verify steps (after {warmup} untimed) of the {layers}-layer model on the CPU "
                      f"oracle, {cores} threads; prompt shortened to {prompt_len} tokens; drafts = the path's own greedy "
                      f"continuation corrupted with p={P_CORRUPT}"}


def run_reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    # every step is a real step of the CPU path (seconds each): the run is bounded in time, and `steps` is the
    # number of steps that were timed (= the request when it fits)
    base = cpu_reference_steps(args.steps, args.warmup, args.layers, budget_s=240.0)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": base["steps"], "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "accepted_per_step": base["accepted_per_step"],
            "emitted_per_step": base["emitted_per_step"], "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference is Go and cannot be built here (no Go toolchain); this arm times this "
                    "repository's C restatement of its CPU path on the host cores"}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- helpers of the GPU arms

def profiler_range(args, start: bool) -> None:
    """cuProfilerStart / cuProfilerStop when --profiler-range was given: a profiler then sees the timed steps only."""
    if getattr(args, "profiler_range", False):
        import ctypes
        drv = ctypes.CDLL("libcuda.so.1")
        (drv.cuProfilerStart if start else drv.cuProfilerStop)()


def init_dist(world: int, local_rank: int):
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return dist


def finish_dist(dist):
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def per_op_profile(sess, stage_fn, on_result, n_steps: int = 3):
    """Event pairs around every operation of `n_steps` more steps (outside the timed region). The ops run
    serialised, each with its own launch latency, so the times are shares of a step, not a timeline. Returns
    (milliseconds per op kind and step, ops per kind and step)."""
    from yuuka_b200 import cuda
    per_op: dict[str, float] = {}
    counts: dict[str, int] = {}
    for _ in range(n_steps):
        stage_fn()
        for code, ns in sess.launch_profiled():
            name = cuda.OP_NAMES.get(code, str(code))
            per_op[name] = per_op.get(name, 0.0) + ns / 1e6 / n_steps
            counts[name] = counts.get(name, 0) + 1
        on_result(sess.fetch())
    return per_op, {k: v // n_steps for k, v in counts.items()}


# --------------------------------------------------------------------------- c2: the graded configuration

def run_c2(args, rank: int, local_rank: int, world: int) -> None:
    from yuuka_b200 import cuda, replicas, synth

    dist = init_dist(world, local_rank)
    cfg = synth.dense4b_config(layers=args.layers, context=4096)
    t_gen = time.perf_counter()
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    t_gen = time.perf_counter() - t_gen
    dev = cuda.Device(local_rank)
    model = cuda.Model(dev, cfg, tensors)
    weight_bytes = model.weight_bytes
    if not (world == 1 and not args.no_cpu_baseline):
        tensors = None
    rows = K_DRAFT + 1
    total_steps = args.warmup + args.steps
    capacity = PROMPT_LEN + total_steps * rows + 64
    sess = cuda.Session(model, max_batch=1, max_nodes=rows, capacity=capacity, kv_format=cuda.KV_F16)

    # prompt, then the model's own greedy continuation, then rewind
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

    def sess_stream_sync():
        cuda.check(cuda.lib().yuuka_stream_synchronize(sess.stream_handle()))

    def barrier():
        sess_stream_sync()
        if dist is not None:
            dist.barrier()

    t_e2e = 0.0
    for step in range(total_steps):
        if step == 0:
            sampler.start()
        if step == args.warmup:
            barrier()
            emitted_total = accepted_total = 0
            dev_ms = 0.0
            profiler_range(args, True)
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
    profiler_range(args, False)
    clocks = sampler.stop()

    # per-op attribution on three more steps (not part of the timed region)
    state = {"pending": pending, "idx": idx}

    def stage_next():
        toks = np.concatenate(([state["pending"]], drafts[state["idx"]:state["idx"] + K_DRAFT])).astype(np.int32)
        sess.stage(toks)

    def consume(res):
        a = int(res.accepted[0])
        state["idx"] += a + 1
        state["pending"] = int(res.emitted[0, a])

    per_op, op_counts = per_op_profile(sess, stage_next, consume)
    gemm_ms = per_op.get("gemm", 0.0) + per_op.get("lm_head", 0.0)
    ctx_mid = PROMPT_LEN + (state["idx"] // 2)

    tot = replicas.reduce_totals(dist, "cuda", dev_ms, t_e2e, float(emitted_total), float(accepted_total))
    dev_ms, t_e2e, emitted_all = tot.device_ms, tot.wall_s, tot.emitted

    if rank == 0:
        peaks = measured_peaks()
        peak = peaks["hbm_gbs"]
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
        ratio, ratio_src = profiled_traffic_ratio()
        line = {
            "metric": METRIC, "value": emitted_all / (dev_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": workload_config(args),
            "accepted_per_step": accepted_total / args.steps, "emitted_per_step": emitted_total / args.steps,
            "e2e": {"value": emitted_all / t_e2e, "unit": UNIT, "ms_per_step": t_e2e / args.steps * 1e3,
                    # one copy in: ancestor masks, tokens, parents, depths, the slot's sequence; one copy out:
                    # accepted count, path, emitted tokens, plus the two device error words
                    "h2d_bytes_per_step": rows * (8 + 4 + 4 + 4) + 4, "d2h_bytes_per_step": 4 + 2 * rows * 4 + 8},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "gemm_tiled_mma_kernel (every quantized GEMM launch of a step, LM head included)",
                         "achieved": gemm_gbs, "peak": peak, "unit": "GB/s", "frac": gemm_gbs / peak,
                         "peak_source": peaks["source"], "bytes_per_step": weight_bytes, "ms_per_step": gemm_timed_ms,
                         "share_of_step": gemm_share, "profiled_ms_per_step": gemm_ms,
                         "traffic": int(weight_bytes * ratio) if ratio else None, "traffic_source": ratio_src,
                         "launches_per_step": launches,
                         "gemm_ops_per_step": op_counts.get("gemm", 0) + op_counts.get("lm_head", 0)},
            "step_roofline": {"bytes_per_step": step_bytes, "weights": weight_bytes, "kv": kv_bytes,
                              "recurrent_state": state_bytes, "achieved_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                              "frac_of_measured_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                              "frac_of_8tbs": step_bytes / (ms_per_step * 1e-3) / 1e9 / 8000.0},
            "per_op_ms": {k: round(v, 4) for k, v in sorted(per_op.items(), key=lambda kv: -kv[1])},
            "per_op_note": "event pairs around every op of three extra steps, run serialised: shares of a step, "
                           "their sum exceeds ms_per_step (graph replay with dependent launches overlaps them)",
            "setup": {"weight_gen_s": round(t_gen, 1), "device": dev.info().name.decode()},
        }
        if world == 1 and not args.no_cpu_baseline:
            sess.close()
            model.close()
            line["cpu_baseline"] = cpu_reference_steps(steps=3, warmup=1, layers=args.layers, tensors=tensors)
        print(json.dumps(line), flush=True)

    sess.close()
    model.close()
    dev.close()
    finish_dist(dist)


# --------------------------------------------------------------------------- c1: kernel microbenchmark

def run_c1(args, rank: int, local_rank: int, world: int) -> None:
    """configs[1]: GEMM shapes K=2560 x N in {9216, 2560 (Q4_K), 248320 (Q6_K)} with bf16 activations of
    M in {1, 2, 4, 9, 16, 64, 576} rows, and the acceptance stage over fp32 logits N(0, 3), vocabulary 248320,
    64 sequences x 9 positions, temperature 0.7. Every rank runs the same sweep on its own GPU (replicas); rank
    0 prints its table."""
    from yuuka_b200 import cuda, microbench, synth

    dist = init_dist(world, local_rank)
    dev = cuda.Device(local_rank)
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank)
    sampler.start()
    table = []
    shapes = [(9216, 2560, "q4_k"), (2560, 2560, "q4_k"), (248320, 2560, "q6_k")]
    for n_out, n_in, d in shapes:
        for m in (1, 2, 4, 9, 16, 64, 576):
            r = microbench.bench_gemm(dev, n_out, n_in, d, m, cuda.PATH_AUTO, iters=max(args.steps, 10), warmup=max(args.warmup, 3))
            route = "register-fed mma.sync, exact" if m < 48 else "tcgen05 + tensor memory"
            table.append({"n_out": n_out, "n_in": n_in, "dtype": d, "rows": m, "route": route, "us": round(r["ms"] * 1e3, 2),
                          "weight_gbs": round(r["weight_gbs"], 1), "hbm_frac": round(r["weight_gbs"] / peaks["hbm_gbs"], 4),
                          "tflops": round(r["tflops"], 2), "tensor_frac": round(r["tflops"] / peaks["bf16_tflops"], 4)})
    # acceptance
    V, B, N, T = 248320, 64, 9, 0.7
    rng = np.random.default_rng(1)
    logits = (3.0 * rng.standard_normal((B, N, V), dtype=np.float32)).astype(np.float32)
    # the draft distribution of row c perturbs the target distribution of its parent row c - 1
    q = np.empty_like(logits)
    q[:, 0] = 0.0
    q[:, 1:] = logits[:, :-1] / T + rng.standard_normal((B, N - 1, V), dtype=np.float32)
    q -= q.max(axis=-1, keepdims=True)
    np.exp(q, out=q)
    q /= q.sum(axis=-1, keepdims=True)
    tokens = np.zeros((B, N), np.int32)
    tokens[:, 0] = rng.integers(0, V, B)
    # drafts drawn from the draft distributions (inverse CDF), so that rows are accepted and rejected
    for b in range(B):
        for c in range(1, N):
            cdf = np.cumsum(q[b, c], dtype=np.float64)
            tokens[b, c] = min(int(np.searchsorted(cdf, rng.random() * cdf[-1])), V - 1)
    uniforms = np.minimum(rng.random((B, N, 2), dtype=np.float32), np.float32(0.99999994))
    lb, qb = dev.upload(logits), dev.upload(q)
    stream = dev.stream()
    e0, e1 = dev.event(), dev.event()
    acc_times = {"rejection": [], "greedy": []}
    accepted = {}
    for it in range(max(args.warmup, 3) + max(args.steps, 10)):
        for mode, name in ((cuda.ACCEPT_REJECTION, "rejection"), (cuda.ACCEPT_GREEDY, "greedy")):
            acc, _, _ = cuda.accept_tree(stream, lb, tokens, V, mode=mode, temperature=T, draft_probs=qb, uniforms=uniforms,
                                         begin=e0, end=e1)
            accepted[name] = float(acc.mean())
            if it >= max(args.warmup, 3):
                acc_times[name].append(e0.elapsed_ms(e1))
    clocks = sampler.stop()
    logit_bytes = B * N * V * 4
    acceptance = {}
    for name, ts in acc_times.items():
        ms = float(np.mean(ts))
        acceptance[name] = {"ms": round(ms, 4), "logit_gbs": round(logit_bytes / ms / 1e6, 1),
                            "hbm_frac": round(logit_bytes / ms / 1e6 / peaks["hbm_gbs"], 4), "mean_accepted": accepted[name]}
    if rank == 0:
        ref = next(t for t in table if t["n_out"] == 9216 and t["rows"] == 9)
        line = {"metric": "weight_stream_GBps_9rows_9216x2560_q4k", "value": ref["weight_gbs"], "unit": "GB/s", "n_gpus": world,
                "steps": max(args.steps, 10), "warmup": max(args.warmup, 3), "ms_per_step": ref["us"] / 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
                "config": {"workload": "configs[1]: kernel-level verify microbenchmark, bf16 activations N(0,1), weights N(0,0.02) "
                                       "quantized; a step = one GEMM call through yuuka_gemm_quant (activation preparation "
                                       "kernel + GEMM kernel) on a weight copy not in L2 (copies rotate through > 2x L2); "
                                       "acceptance: yuuka_accept_tree over 64 x 9 x 248320 fp32 logits N(0,3), q = softmax(logits / T "
                                       "+ N(0,1)), T = 0.7, drafts drawn from q",
                           "l2": "weights rotate through more than twice the 126 MB L2; the 571 MB of logits exceed it"},
                "gemm_table": table, "acceptance": acceptance, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": "gemm_tiled_mma_kernel, 9216 x 2560 Q4_K, 9 rows", "achieved": ref["weight_gbs"],
                             "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ref["hbm_frac"], "peak_source": peaks["source"],
                             "traffic": None},
                "gpu_launches": 2 * max(args.steps, 10)}
        print(json.dumps(line), flush=True)
    lb.free(); qb.free()
    stream.destroy()
    dev.close()
    finish_dist(dist)


# --------------------------------------------------------------------------- c3: batched trees, rejection sampling

def run_c3(args, rank: int, local_rank: int, world: int) -> None:
    from yuuka_b200 import cuda, replicas, synth

    dist = init_dist(world, local_rank)
    n_total = args.seqs if args.seqs > 0 else 256
    mine = replicas.sequences_of_rank(n_total, world, rank)
    B = len(mine)
    cfg = synth.dense4b_config(layers=args.layers, context=4096)
    tensors = synth.make_model(cfg, "q4_k_m", seed=1)
    dev = cuda.Device(local_rank)
    model = cuda.Model(dev, cfg, tensors)
    weight_bytes = model.weight_bytes
    del tensors
    V = cfg["vocab"]
    parent = synth.tree_16()
    N = parent.size
    total_steps = args.warmup + args.steps
    cap, bs = 4096, 16
    per = cap // bs
    sess = cuda.Session(model, max_batch=B, max_nodes=N, capacity=cap, kv_format=cuda.KV_F16, block_size=bs)
    rng = np.random.default_rng(1000 + rank)
    perm = rng.permutation(B * per).astype(np.int32)
    lens = synth.uniform_i32(n_total, 256, 3073, 77)
    pend = np.zeros(B, np.int32)
    t_prompt = time.perf_counter()
    for b, sq in enumerate(mine):
        sess.set_block_table(b, perm[b * per:(b + 1) * per])
        prompt = synth.uniform_i32(int(lens[sq]), 0, V, 2000 + sq)
        pend[b] = int(np.argmax(sess.forward(prompt, seq=b)))
    t_prompt = time.perf_counter() - t_prompt
    # draft distributions: a perturbed softmax, one base row (softmax of N(0, 3) noise) rotated per (sequence, node)
    base = rng.standard_normal(V).astype(np.float32) * 3.0
    base = np.exp(base - base.max())
    base /= base.sum()
    q = np.empty((B, N, V), np.float32)
    tokens = synth.uniform_i32(B * N, 0, V, 300 + rank).reshape(B, N)
    shifts = rng.integers(0, V, (B, N))
    # (a random-init model spreads its mass almost evenly over the vocabulary, so a drafted token is accepted
    # unless the draft model was far surer of it than the target: 30 % of the drafts get q = 0.5, which rejects
    # them; the others keep the rotated base value, far below the target's probability, and are accepted)
    sure = rng.random((B, N)) < P_CORRUPT
    for b in range(B):
        for c in range(N):
            q[b, c] = np.roll(base, int(shifts[b, c]))
            q[b, c, tokens[b, c]] = 0.5 if sure[b, c] else min(float(q[b, c, tokens[b, c]]), 1e-7)
    qb = dev.upload(q)
    del q
    ev0, ev1 = dev.event(), dev.event()
    sampler = ClockSampler(local_rank)
    dev_ms, emitted_total, accepted_total, t_e2e = 0.0, 0, 0, 0.0

    def sync():
        cuda.check(cuda.lib().yuuka_stream_synchronize(sess.stream_handle()))
        if dist is not None:
            dist.barrier()

    for step in range(total_steps):
        if step == 0:
            sampler.start()
        if step == args.warmup:
            sync()
            dev_ms, emitted_total, accepted_total = 0.0, 0, 0
            profiler_range(args, True)
            t_e2e = time.perf_counter()
        tokens[:, 0] = pend
        uniforms = synth.uniform_f32(B * N * 2, 900 + step).reshape(B, N, 2)
        sess.stage(tokens, parent=parent, mode=cuda.ACCEPT_REJECTION, temperature=0.8, draft_probs=qb, uniforms=uniforms)
        sess.record(ev0)
        sess.launch(ev1)
        res = sess.fetch()
        dev_ms += ev0.elapsed_ms(ev1)
        emitted_total += int(res.accepted.sum()) + B
        accepted_total += int(res.accepted.sum())
        pend = res.emitted[np.arange(B), res.accepted].astype(np.int32)
        launches = sess.last_launch_count
    sync()
    t_e2e = time.perf_counter() - t_e2e
    profiler_range(args, False)
    clocks = sampler.stop()
    ctx_now = [sess.position(b) for b in range(B)]
    tot = replicas.reduce_totals(dist, "cuda", dev_ms, t_e2e, float(emitted_total), float(accepted_total))
    if rank == 0:
        peaks = measured_peaks()
        ms = tot.device_ms / args.steps
        R = B * N
        kv_bytes = int(np.sum(ctx_now)) * 2 * cfg["kv_heads"] * cfg["head_dim"] * 2 * (args.layers // 4)
        state_bytes = 2 * B * (args.layers - args.layers // 4) * (cfg["time_step_rank"] * cfg["state_size"] ** 2 * 4)
        logit_bytes = R * V * 4
        flops = 2.0 * R * (weight_bytes / 0.6)     # ~0.6 B per weight in the Q4_K / Q6_K mix
        line = {"metric": METRIC, "value": tot.emitted / (tot.device_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16 tensor-core operands (tcgen05, weights and activations rounded to fp16), f32 accumulate; weights Q4_K/Q6_K",
                "data": "synthetic",
                "config": {"workload": f"configs[3]: dense 4B-shaped qwen35, {n_total} sequences over {world} GPU(s) ({B} on rank 0), "
                                       "paged KV with 16-token blocks and permuted block tables, context 4096, prompts of uniform "
                                       "random length 256-3072, 16-node draft tree (4/2/1/1, 17 rows with the pending token), "
                                       "rejection sampling at T = 0.8 against a synthetic perturbed-softmax draft distribution",
                           "layers": args.layers, "rows_per_step": R, "kv_format": "F16",
                           "l2": "no flush needed: a step streams gigabytes of weights, KV rows and state"},
                "accepted_per_step": accepted_total / args.steps, "emitted_per_step": emitted_total / args.steps,
                "e2e": {"value": tot.emitted / tot.wall_s, "unit": UNIT, "ms_per_step": tot.wall_s / args.steps * 1e3,
                        "h2d_bytes_per_step": R * 20 + B * 4 + R * 8, "d2h_bytes_per_step": B * 4 + 2 * R * 4 + 8},
                "gpu_launches": launches * args.steps, "clocks": clocks,
                "roofline": {"bound": "tensor", "kernel": "gemm_umma_ws_kernel (every quantized GEMM of a step; 512 rows per launch)",
                             "achieved": flops / (ms * 1e-3) / 1e12, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                             "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                             "note": "whole-step time in the denominator: attention, the recurrent scan and acceptance are inside it",
                             "traffic": None},
                "step_bytes": {"weights_once": weight_bytes, "kv": kv_bytes, "recurrent_state": state_bytes, "logits": logit_bytes,
                               "hbm_floor_ms": (weight_bytes + kv_bytes + state_bytes) / peaks["hbm_gbs"] / 1e6},
                "setup": {"prompt_s": round(t_prompt, 1), "prompt_tokens": int(sum(int(lens[sq]) for sq in mine))}}
        print(json.dumps(line), flush=True)
    qb.free()
    sess.close(); model.close(); dev.close()
    finish_dist(dist)


# --------------------------------------------------------------------------- c4: qwen35moe

def run_c4(args, rank: int, local_rank: int, world: int) -> None:
    from yuuka_b200 import cuda, replicas, synth

    dist = init_dist(world, local_rank)
    layers = args.layers if args.layers != 32 else 40
    cfg = synth.moe_config(layers=layers, context=2048)
    t_gen = time.perf_counter()
    tensors = synth.make_model(cfg, "q4_k_m", seed=2)
    t_gen = time.perf_counter() - t_gen
    dev = cuda.Device(local_rank)
    model = cuda.Model(dev, cfg, tensors)
    weight_bytes = model.weight_bytes
    del tensors
    V, B, K = cfg["vocab"], (args.seqs if args.seqs > 0 else 32), 4
    N = K + 1
    total_steps = args.warmup + args.steps
    prompt_len = args.prompt if args.prompt > 0 else 1024
    sess = cuda.Session(model, max_batch=B, max_nodes=N, capacity=prompt_len + (total_steps + 2) * N + 16, kv_format=cuda.KV_F16)
    pend = np.zeros(B, np.int32)
    t_prompt = time.perf_counter()
    for b in range(B):
        prompt = synth.uniform_i32(prompt_len, 0, V, 3000 + rank * 1000 + b)
        pend[b] = int(np.argmax(sess.forward(prompt, seq=b)))
    t_prompt = time.perf_counter() - t_prompt
    ev0, ev1 = dev.event(), dev.event()
    sampler = ClockSampler(local_rank)
    dev_ms, emitted_total, accepted_total, t_e2e = 0.0, 0, 0, 0.0
    # drafts: the previous step's own next tokens are not known ahead; dummy drafts would all be rejected, so a
    # step first asks the model (an uncommitted pass, untimed) for its greedy chain and corrupts it with p = 0.3
    def sync():
        cuda.check(cuda.lib().yuuka_stream_synchronize(sess.stream_handle()))
        if dist is not None:
            dist.barrier()

    rng = np.random.default_rng(5 + rank)
    for step in range(total_steps):
        if step == 0:
            sampler.start()
        if step == args.warmup:
            sync()
            dev_ms, emitted_total, accepted_total = 0.0, 0, 0
            t_e2e = 0.0
        tokens = np.zeros((B, N), np.int32)
        tokens[:, 0] = pend
        for c in range(1, N):           # untimed: the greedy chain behind the pending token, one more row per pass
            lg = sess.verify(tokens[:, :c], mode=cuda.ACCEPT_NONE, want_logits=True).logits
            tokens[:, c] = np.argmax(lg[:, c - 1], axis=-1)
        noise = rng.random((B, K)) < P_CORRUPT
        tokens[:, 1:][noise] = rng.integers(0, V, int(noise.sum()))
        t0 = time.perf_counter()
        sess.stage(tokens)
        sess.record(ev0)
        sess.launch(ev1)
        res = sess.fetch()
        t_e2e += time.perf_counter() - t0
        dev_ms += ev0.elapsed_ms(ev1)
        emitted_total += int(res.accepted.sum()) + B
        accepted_total += int(res.accepted.sum())
        pend = res.emitted[np.arange(B), res.accepted].astype(np.int32)
        launches = sess.last_launch_count
    sync()
    clocks = sampler.stop()
    tot = replicas.reduce_totals(dist, "cuda", dev_ms, t_e2e, float(emitted_total), float(accepted_total))
    if rank == 0:
        peaks = measured_peaks()
        ms = tot.device_ms / args.steps
        line = {"metric": METRIC, "value": tot.emitted / (tot.device_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "expert GEMMs: exact register-fed route; dense GEMMs at 160 rows: tcgen05 with fp16-rounded operands; f32 accumulate",
                "data": "synthetic",
                "config": {"workload": f"configs[4]: qwen35moe shape (hidden 2048, {layers} layers 3 GDN:1 attention, 256 routed experts "
                                       f"top-8 + shared expert, expert FFN 512, vocab 248320), Q4_K experts, {B} sequences per GPU, "
                                       f"{prompt_len}-token prompts, chain k=4, greedy, drafts = greedy chain corrupted with p=0.3",
                           "layers": layers, "rows_per_step": B * N, "kv_format": "F16",
                           "l2": "no flush needed: a step streams the touched experts, ~0.45 GB per layer"},
                "accepted_per_step": accepted_total / args.steps, "emitted_per_step": emitted_total / args.steps,
                "e2e": {"value": tot.emitted / tot.wall_s, "unit": UNIT, "ms_per_step": tot.wall_s / args.steps * 1e3,
                        "h2d_bytes_per_step": B * N * 20 + B * 4, "d2h_bytes_per_step": B * 4 + 2 * B * N * 4 + 8},
                "gpu_launches": launches * args.steps, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": "gemm_tiled_mma_kernel (grouped expert GEMMs) and the dense GEMMs of a step",
                             "achieved": weight_bytes / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": weight_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                             "note": "all weight bytes of the model over the whole step time (about 254 of 256 experts are touched per layer)",
                             "traffic": None},
                "setup": {"weight_gen_s": round(t_gen, 1), "prompt_s": round(t_prompt, 1), "weight_bytes": weight_bytes}}
        print(json.dumps(line), flush=True)
    sess.close(); model.close(); dev.close()
    finish_dist(dist)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seqs", type=int, default=0, help="c3: sequences in all (default 256); c4: sequences per GPU (default 32)")
    ap.add_argument("--prompt", type=int, default=0, help="c4: prompt length (default 1024)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profiler-range", action="store_true",
                    help="cuProfilerStart / Stop around the timed steps (for ncu --profile-from-start off; numbers from such a run are not bench values)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    {"c1": run_c1, "c2": run_c2, "c3": run_c3, "c4": run_c4}[args.config](args, rank, local_rank, world)


if __name__ == "__main__":
    main()
