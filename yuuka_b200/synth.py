"""Seeded synthetic qwen35 / qwen35moe models in packed GGUF tensor layouts.

Tensor names and shapes follow what model/qwen35/load.go:80-215 reads; packed
rows use the block layouts of tensor/dtype.go:102-151. The reference has no
weight quantizer, so the bytes come from this package's own
(csrc/synth_quant.c). The same bytes are handed to the CPU oracle and uploaded
to the GPU.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K = 0, 1, 8, 12, 13, 14
DTYPE_NAMES = {F32: "F32", F16: "F16", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(_build.build_synth())
        vp, i64, i32, f32, u64 = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_uint64
        L.ys_fill_normal_f32.argtypes = [vp, i64, f32, f32, u64]
        L.ys_fill_normal_f32.restype = None
        L.ys_fill_uniform_i32.argtypes = [vp, i64, i32, i32, u64]
        L.ys_fill_uniform_i32.restype = None
        L.ys_fill_uniform_f32.argtypes = [vp, i64, u64]
        L.ys_fill_uniform_f32.restype = None
        L.ys_row_bytes.argtypes = [i32, i64]
        L.ys_row_bytes.restype = i64
        L.ys_quantize.argtypes = [vp, i32, vp, i64, i64]
        L.ys_quantize.restype = i32
        L.ys_fill_normal_quant.argtypes = [vp, i32, i64, i64, f32, u64]
        L.ys_fill_normal_quant.restype = i32
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def row_bytes(dtype: int, cols: int) -> int:
    n = lib().ys_row_bytes(dtype, cols)
    if n < 0:
        raise ValueError(f"row width {cols} does not fit dtype {dtype}")
    return n


def normal_f32(n: int, std: float, seed: int, mean: float = 0.0) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().ys_fill_normal_f32(_p(out), n, mean, std, seed)
    return out


def uniform_i32(n: int, lo: int, hi: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.int32)
    lib().ys_fill_uniform_i32(_p(out), n, lo, hi, seed)
    return out


def uniform_f32(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().ys_fill_uniform_f32(_p(out), n, seed)
    return out


def quantize(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    out = np.empty(rows * row_bytes(dtype, cols), np.uint8)
    if lib().ys_quantize(_p(out), dtype, _p(x), rows, cols) != 0:
        raise ValueError("quantize failed")
    return out


def normal_quant(rows: int, cols: int, dtype: int, std: float, seed: int) -> np.ndarray:
    out = np.empty(rows * row_bytes(dtype, cols), np.uint8)
    if lib().ys_fill_normal_quant(_p(out), dtype, rows, cols, std, seed) != 0:
        raise ValueError("fill_normal_quant failed")
    return out


# --------------------------------------------------------------------------
# configurations

def tiny_config() -> dict:
    """hidden 256, 3 Gated-DeltaNet layers + 1 gated-attention layer, vocab 4096."""
    return dict(block_count=4, context_length=512, hidden=256, ffn=768, heads=4, kv_heads=2,
                head_dim=64, rope_dim=64, rope_freq_base=1.0e6, rms_eps=1e-6, vocab=4096,
                conv_kernel=4, state_size=64, group_count=4, time_step_rank=4, inner_size=256,
                full_attention_interval=4, expert_count=0, expert_used=0, expert_ffn=0,
                shared_ffn=0)


def dense4b_config(layers: int = 32, vocab: int = 248320, context: int = 4096) -> dict:
    """4B-shaped dense qwen35: hidden 2560, 3 GDN : 1 attention, FFN 9216."""
    return dict(block_count=layers, context_length=context, hidden=2560, ffn=9216, heads=16,
                kv_heads=4, head_dim=256, rope_dim=64, rope_freq_base=1.0e7, rms_eps=1e-6,
                vocab=vocab, conv_kernel=4, state_size=128, group_count=16, time_step_rank=32,
                inner_size=4096, full_attention_interval=4, expert_count=0, expert_used=0,
                expert_ffn=0, shared_ffn=0)


def moe_config(layers: int = 40, vocab: int = 248320, experts: int = 256, context: int = 4096) -> dict:
    """qwen35moe shape: hidden 2048, 256 routed experts top-8 + shared, expert FFN 512."""
    return dict(block_count=layers, context_length=context, hidden=2048, ffn=0, heads=16,
                kv_heads=2, head_dim=256, rope_dim=64, rope_freq_base=1.0e7, rms_eps=1e-6,
                vocab=vocab, conv_kernel=4, state_size=128, group_count=16, time_step_rank=32,
                inner_size=4096, full_attention_interval=4, expert_count=experts, expert_used=8,
                expert_ffn=512, shared_ffn=512)


def tiny_moe_config() -> dict:
    cfg = tiny_config()
    cfg.update(ffn=0, expert_count=8, expert_used=2, expert_ffn=256, shared_ffn=256)
    return cfg


def is_recurrent(cfg: dict, layer: int) -> bool:
    return (layer + 1) % cfg["full_attention_interval"] != 0


def quant_plan(scheme: str):
    """dtype per tensor role. 'q4_k_m': attn_v, ffn_down and output in Q6_K, the
    rest Q4_K. A single dtype name applies it everywhere."""
    if scheme == "q4_k_m":
        return lambda role: Q6_K if role in ("attn_v", "ffn_down", "output", "ffn_down_exps",
                                             "ffn_down_shexp") else Q4_K
    single = {"q8_0": Q8_0, "q4_k": Q4_K, "q5_k": Q5_K, "q6_k": Q6_K, "f32": F32, "f16": F16}[scheme]
    return lambda role: single


def make_model(cfg: dict, scheme: str = "q8_0", seed: int = 1234, std: float = 0.02,
               unit_norms: bool = True) -> dict:
    """Returns name -> (dtype, array, rows, cols). Matrices are uint8 packed rows;
    vectors are float32 with rows = 1."""
    pick = quant_plan(scheme)
    t: dict = {}
    counter = [seed * 1000003]

    def nxt():
        counter[0] += 1
        return counter[0]

    def mat(name, role, rows, cols):
        d = pick(role)
        if cols % 256 != 0 and d in (Q4_K, Q5_K, Q6_K):
            d = Q8_0
        t[name] = (d, normal_quant(rows, cols, d, std, nxt()), rows, cols)

    def vec(name, n, kind="norm"):
        s = nxt()
        if kind == "norm":
            v = np.ones(n, np.float32) if unit_norms else (1.0 + normal_f32(n, 0.1, s))
        else:
            v = normal_f32(n, std, s)
        t[name] = (F32, v.astype(np.float32), 1, n)

    H, V = cfg["hidden"], cfg["vocab"]
    S, G, R = cfg["state_size"], cfg["group_count"], cfg["time_step_rank"]
    inner = cfg["inner_size"]
    conv_dim = 2 * G * S + inner
    hd = cfg["head_dim"]
    q_dim, kv_dim, o_dim = cfg["heads"] * hd * 2, cfg["kv_heads"] * hd, cfg["heads"] * hd
    mat("token_embd.weight", "token_embd", V, H)
    mat("output.weight", "output", V, H)
    vec("output_norm.weight", H)
    for i in range(cfg["block_count"]):
        p = f"blk.{i}."
        vec(p + "attn_norm.weight", H)
        vec(p + "post_attention_norm.weight", H)
        if is_recurrent(cfg, i):
            mat(p + "attn_qkv.weight", "attn_qkv", conv_dim, H)
            mat(p + "attn_gate.weight", "attn_gate", inner, H)
            mat(p + "ssm_out.weight", "ssm_out", H, inner)
            mat(p + "ssm_beta.weight", "ssm_beta", R, H)
            mat(p + "ssm_alpha.weight", "ssm_alpha", R, H)
            # conv taps are O(1) so the SiLU input is not vanishing
            t[p + "ssm_conv1d.weight"] = (F32, normal_f32(cfg["conv_kernel"] * conv_dim, 0.5, nxt()),
                                          1, cfg["conv_kernel"] * conv_dim)
            h = np.arange(R, dtype=np.float64)
            # log-decay softplus(alpha+dt)*a lands near -0.3 (decay ~0.75), which
            # exposes state errors that a decay of ~0.997 would hide
            t[p + "ssm_dt.bias"] = (F32, (0.1 * (1 + (h % 3))).astype(np.float32), 1, R)
            t[p + "ssm_a"] = (F32, (-(0.2 + 0.4 * ((h * 0.6180339887) % 1.0))).astype(np.float32), 1, R)
            vec(p + "ssm_norm.weight", S)
        else:
            mat(p + "attn_q.weight", "attn_q", q_dim, H)
            mat(p + "attn_k.weight", "attn_k", kv_dim, H)
            mat(p + "attn_v.weight", "attn_v", kv_dim, H)
            mat(p + "attn_output.weight", "attn_output", H, o_dim)
            vec(p + "attn_q_norm.weight", hd)
            vec(p + "attn_k_norm.weight", hd)
        if cfg["expert_count"] > 0:
            E, F, SF = cfg["expert_count"], cfg["expert_ffn"], cfg["shared_ffn"]
            # router weights are O(1/sqrt(H)) so router logits are ~N(0,1)
            t[p + "ffn_gate_inp.weight"] = (F32, normal_f32(E * H, H ** -0.5, nxt()), E, H)
            vec(p + "ffn_gate_inp_shexp.weight", H, kind="w")
            mat(p + "ffn_gate_shexp.weight", "ffn_gate_shexp", SF, H)
            mat(p + "ffn_up_shexp.weight", "ffn_up_shexp", SF, H)
            mat(p + "ffn_down_shexp.weight", "ffn_down_shexp", H, SF)
            mat(p + "ffn_gate_exps.weight", "ffn_gate_exps", F * E, H)
            mat(p + "ffn_up_exps.weight", "ffn_up_exps", F * E, H)
            mat(p + "ffn_down_exps.weight", "ffn_down_exps", H * E, F)
        else:
            mat(p + "ffn_gate.weight", "ffn_gate", cfg["ffn"], H)
            mat(p + "ffn_up.weight", "ffn_up", cfg["ffn"], H)
            mat(p + "ffn_down.weight", "ffn_down", H, cfg["ffn"])
    return t


def weight_bytes(tensors: dict, skip=("token_embd.weight",)) -> int:
    """Bytes every verify step must stream: all tensors except the embedding
    table, of which only the fed rows are read."""
    return sum(a.nbytes for n, (_, a, _, _) in tensors.items() if n not in skip)


def corrupt_draft(greedy: np.ndarray, vocab: int, p: float, seed: int) -> np.ndarray:
    """Draft = the greedy continuation with each position independently replaced
    by a uniform random id with probability p."""
    u = uniform_f32(greedy.size, seed)
    r = uniform_i32(greedy.size, 0, vocab, seed + 1)
    return np.where(u < p, r, greedy).astype(np.int32)


def tree_16() -> np.ndarray:
    """parent[] of the 1 + 16-node verification tree: node 0 is the pending
    token; drafts 1-4 hang off it; 5,6 off 1; 7,8 off 2; 9-12 are single
    children of 5-8 and 13-16 of 9-12 (4 drafts per depth, depth 4)."""
    return np.array([-1, 0, 0, 0, 0, 1, 1, 2, 2, 5, 6, 7, 8, 9, 10, 11, 12], np.int32)
