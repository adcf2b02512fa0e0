"""ctypes binding of the CPU oracle (oracle/liboracle.so).

Test infrastructure only: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py. The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F32, F16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = 0, 1, 2, 6, 8, 12, 13, 14
KV_F32, KV_F16, KV_Q8_0 = 0, 1, 2


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "yuuka_oracle.c")
    hdr = os.path.join(_HERE, "yuuka_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr)))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


class Config(C.Structure):
    _fields_ = [
        ("block_count", C.c_int32), ("context_length", C.c_int32), ("hidden", C.c_int32),
        ("ffn", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("rope_dim", C.c_int32), ("rope_freq_base", C.c_double),
        ("rms_eps", C.c_float), ("vocab", C.c_int32), ("conv_kernel", C.c_int32),
        ("state_size", C.c_int32), ("group_count", C.c_int32), ("time_step_rank", C.c_int32),
        ("inner_size", C.c_int32), ("full_attention_interval", C.c_int32),
        ("expert_count", C.c_int32), ("expert_used", C.c_int32), ("expert_ffn", C.c_int32),
        ("shared_ffn", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_LIB_PATH)
    vp, i32, i64, f32, u8p = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_void_p
    sig = {
        "yo_f32_to_f16": (C.c_uint16, [f32]),
        "yo_f16_to_f32": (f32, [C.c_uint16]),
        "yo_row_bytes": (i64, [i32, i64]),
        "yo_dequantize_row": (i32, [vp, i64, i32, u8p, i64]),
        "yo_matmul": (i32, [vp, vp, i32, u8p, i32, i64, i64]),
        "yo_set_threads": (None, [i32]),
        "yo_get_threads": (i32, []),
        "yo_kv_row_bytes": (i64, [i32, i32]),
        "yo_kv_encode_row": (i32, [u8p, i32, vp, i32]),
        "yo_kv_decode_row": (i32, [vp, i32, u8p, i32]),
        "yo_table_map": (i32, [vp, i32, i32, i32, vp, vp]),
        "yo_config_validate": (i32, [vp, C.c_char_p, C.c_size_t]),
        "yo_is_recurrent": (i32, [vp, i32]),
        "yo_rms_norm": (None, [vp, vp, vp, i32, f32]),
        "yo_l2_norm_head": (None, [vp, i32, f32, f32]),
        "yo_apply_rope": (None, [vp, i32, i32, i32, i32, i32, C.c_double]),
        "yo_softmax_inplace": (None, [vp, i32]),
        "yo_gdn_per_token_scan": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
        "yo_gdn_chunked_scan": (None, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
        "yo_gdn_norm_gate": (None, [vp, vp, vp, i32, i32, i32, f32]),
        "yo_select_experts": (None, [vp, i32, vp, vp, i32]),
        "yo_sigmoid": (f32, [f32]), "yo_silu": (f32, [f32]), "yo_softplus": (f32, [f32]),
        "yo_model_create": (vp, [vp]),
        "yo_model_destroy": (None, [vp]),
        "yo_model_set_tensor": (i32, [vp, C.c_char_p, i32, vp, i64, i64]),
        "yo_model_check": (i32, [vp, C.c_char_p, C.c_size_t]),
        "yo_state_create": (vp, [vp, i32, i32, i32, i32, vp, i32]),
        "yo_state_destroy": (None, [vp]),
        "yo_state_reset": (None, [vp]),
        "yo_state_pos": (i32, [vp]),
        "yo_state_set_pos": (i32, [vp, i32]),
        "yo_state_snapshot_bytes": (i64, [vp]),
        "yo_state_snapshot": (i32, [vp, u8p, i64]),
        "yo_state_restore": (i32, [vp, u8p, i64]),
        "yo_state_kv": (vp, [vp, i32, i32, vp]),
        "yo_state_conv": (vp, [vp, i32, vp]),
        "yo_state_s": (vp, [vp, i32, vp]),
        "yo_state_last_hidden": (vp, [vp]),
        "yo_forward_one": (i32, [vp, vp, i32, i32]),
        "yo_logits": (vp, [vp]),
        "yo_forward": (i32, [vp, vp, vp, i32, vp]),
        "yo_prefill_logits": (i32, [vp, vp, vp, i32, vp]),
        "yo_argmax": (i32, [vp, i32]),
        "yo_lookup_draft": (i32, [vp, i32, i32, i32, vp]),
        "yo_spec_verify_reference": (i32, [vp, vp, vp, vp, i32, vp, vp, vp]),
        "yo_verify_chain": (i32, [vp, vp, i32, vp, i32, vp, vp, vp]),
        "yo_verify_tree_greedy": (i32, [vp, vp, vp, vp, i32, vp, vp, vp, vp]),
        "yo_accept_greedy_tree": (i32, [vp, i32, vp, vp, i32, vp, vp, vp]),
        "yo_exp_det": (f32, [f32]),
        "yo_accept_rejection_tree": (i32, [vp, vp, i32, vp, vp, i32, f32, vp, vp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def row_bytes(dtype: int, cols: int) -> int:
    return lib().yo_row_bytes(dtype, cols)


def dequantize_row(dtype: int, src) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.uint8)
    elems = {F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34),
             Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}[dtype]
    n = src.size // elems[1] * elems[0]
    dst = np.empty(n, np.float32)
    rc = lib().yo_dequantize_row(_p(dst), n, dtype, _p(src), src.size)
    if rc != 0:
        raise ValueError(f"dequantize_row failed: {rc}")
    return dst


def matmul(w, dtype: int, rows: int, cols: int, x) -> np.ndarray:
    """dst[b, r] = sum_i x[b, i] * W[r, i] (tensor/quant.go:326-339)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x).reshape(-1, cols)
    dst = np.empty((x.shape[0], rows), np.float32)
    rc = lib().yo_matmul(_p(dst), _p(x), x.shape[0], _p(w), dtype, rows, cols)
    if rc != 0:
        raise ValueError("matmul failed")
    return dst


def kv_encode_row(fmt: int, row) -> np.ndarray:
    row = _f32(row)
    dst = np.zeros(lib().yo_kv_row_bytes(fmt, row.size), np.uint8)
    lib().yo_kv_encode_row(_p(dst), fmt, _p(row), row.size)
    return dst


def kv_decode_row(fmt: int, src, n: int) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.uint8)
    dst = np.empty(n, np.float32)
    lib().yo_kv_decode_row(_p(dst), fmt, _p(src), n)
    return dst


def table_map(blocks, block_size: int, pos: int):
    blocks = _i32(blocks)
    b, o = C.c_int32(), C.c_int32()
    rc = lib().yo_table_map(_p(blocks), blocks.size, block_size, pos, C.byref(b), C.byref(o))
    if rc != 0:
        raise IndexError(f"position {pos} is not mapped")
    return b.value, o.value


def argmax(logits) -> int:
    logits = _f32(logits)
    return lib().yo_argmax(_p(logits), logits.size)


def lookup_draft(history, max_draft: int, min_match: int):
    history = _i32(history)
    out = np.zeros(max(max_draft, 1), np.int32)
    n = lib().yo_lookup_draft(_p(history), history.size, max_draft, min_match, _p(out))
    return out[:n].tolist()


def select_experts(logits, k: int):
    logits = _f32(logits)
    ids = np.zeros(k, np.int32)
    w = np.zeros(k, np.float32)
    lib().yo_select_experts(_p(logits), logits.size, _p(ids), _p(w), k)
    return ids, w


def gdn_per_token_scan(state, conv, alpha, beta, rows, groups, rank, S):
    """Updates state in place; returns out[rows, rank, S]."""
    conv = _f32(conv)
    conv_dim = conv.size // rows
    out = np.zeros((rows, rank, S), np.float32)
    alpha, beta = _f32(alpha), _f32(beta)
    assert state.dtype == np.float32 and state.flags.c_contiguous
    lib().yo_gdn_per_token_scan(_p(state), _p(conv), _p(alpha), _p(beta), _p(out), rows, groups,
                                rank, S, conv_dim)
    return out


def gdn_chunked_scan(state, conv, alpha, beta, rows, groups, rank, S):
    """The chunkwise WY form of the same recurrence. Updates state in place; returns out[rows, rank, S]."""
    conv = _f32(conv)
    conv_dim = conv.size // rows
    out = np.zeros((rows, rank, S), np.float32)
    alpha, beta = _f32(alpha), _f32(beta)
    assert state.dtype == np.float32 and state.flags.c_contiguous
    lib().yo_gdn_chunked_scan(_p(state), _p(conv), _p(alpha), _p(beta), _p(out), rows, groups, rank, S, conv_dim)
    return out


def accept_greedy_tree(logits, tokens, parent):
    logits = _f32(logits)
    tokens, parent = _i32(tokens), _i32(parent)
    n, V = tokens.size, logits.shape[-1]
    acc = C.c_int32()
    path = np.full(n, -1, np.int32)
    emitted = np.full(n, -1, np.int32)
    lib().yo_accept_greedy_tree(_p(logits), V, _p(tokens), _p(parent), n, C.byref(acc), _p(path),
                                _p(emitted))
    a = acc.value
    return a, path[:a].copy(), emitted[:a + 1].copy()


def accept_rejection_tree(logits, draft_probs, tokens, parent, temperature, uniforms):
    logits, draft_probs, uniforms = _f32(logits), _f32(draft_probs), _f32(uniforms)
    tokens, parent = _i32(tokens), _i32(parent)
    n, V = tokens.size, logits.shape[-1]
    acc = C.c_int32()
    path = np.full(n, -1, np.int32)
    emitted = np.full(n, -1, np.int32)
    lib().yo_accept_rejection_tree(_p(logits), _p(draft_probs), V, _p(tokens), _p(parent), n,
                                   temperature, _p(uniforms), C.byref(acc), _p(path), _p(emitted))
    a = acc.value
    return a, path[:a].copy(), emitted[:a + 1].copy()


class Model:
    """Oracle model over a dict name -> (dtype, uint8/float32 array, rows, cols)."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = Config(**cfg)
        self.cfg_dict = dict(cfg)
        self._keep = []
        self.h = lib().yo_model_create(C.byref(self.cfg))
        if not self.h:
            msg = C.create_string_buffer(256)
            lib().yo_config_validate(C.byref(self.cfg), msg, 256)
            raise ValueError("invalid config: " + msg.value.decode())
        for name, (dtype, data, rows, cols) in tensors.items():
            data = np.ascontiguousarray(data)
            self._keep.append(data)
            rc = lib().yo_model_set_tensor(self.h, name.encode(), dtype, _p(data), rows, cols)
            if rc != 0:
                raise ValueError(f"set_tensor {name}: {rc}")
        msg = C.create_string_buffer(256)
        if lib().yo_model_check(self.h, msg, 256) != 0:
            raise ValueError(msg.value.decode())

    @property
    def vocab(self):
        return self.cfg.vocab

    def close(self):
        if self.h:
            lib().yo_model_destroy(self.h)
            self.h = None


class State:
    def __init__(self, model: Model, capacity: int, kv_format: int = KV_F16, pool_blocks: int = 0,
                 block_size: int = 0, table=None):
        self.model = model
        t = _i32(table) if table is not None else None
        self.h = lib().yo_state_create(model.h, capacity, kv_format, pool_blocks, block_size,
                                       _p(t), 0 if t is None else t.size)
        if not self.h:
            raise ValueError("state_create failed")

    @property
    def pos(self):
        return lib().yo_state_pos(self.h)

    def set_pos(self, pos):
        if lib().yo_state_set_pos(self.h, pos) != 0:
            raise ValueError("bad position")

    def reset(self):
        lib().yo_state_reset(self.h)

    def snapshot(self) -> np.ndarray:
        n = lib().yo_state_snapshot_bytes(self.h)
        out = np.empty(n, np.uint8)
        lib().yo_state_snapshot(self.h, _p(out), n)
        return out

    def restore(self, data):
        data = np.ascontiguousarray(data, dtype=np.uint8)
        if lib().yo_state_restore(self.h, _p(data), data.size) != 0:
            raise ValueError("snapshot size mismatch")

    def kv(self, layer, which) -> np.ndarray:
        n = C.c_int64()
        ptr = lib().yo_state_kv(self.h, layer, which, C.byref(n))
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(n.value,))

    def rec_s(self, layer) -> np.ndarray:
        n = C.c_int64()
        ptr = lib().yo_state_s(self.h, layer, C.byref(n))
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(n.value,))

    def rec_conv(self, layer) -> np.ndarray:
        n = C.c_int64()
        ptr = lib().yo_state_conv(self.h, layer, C.byref(n))
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(n.value,))

    def forward(self, tokens) -> np.ndarray:
        tokens = _i32(tokens)
        out = np.empty(self.model.vocab, np.float32)
        rc = lib().yo_forward(self.model.h, self.h, _p(tokens), tokens.size, _p(out))
        if rc != 0:
            raise RuntimeError(f"forward failed: {rc}")
        return out

    def step(self, token) -> np.ndarray:
        return self.forward([token])

    def prefill_logits(self, tokens) -> np.ndarray:
        tokens = _i32(tokens)
        out = np.empty((tokens.size, self.model.vocab), np.float32)
        rc = lib().yo_prefill_logits(self.model.h, self.h, _p(tokens), tokens.size, _p(out))
        if rc != 0:
            raise RuntimeError(f"prefill_logits failed: {rc}")
        return out

    def spec_verify_reference(self, logits, draft):
        """engine/speculative.go:181-239. Returns (accepted, emitted, next_logits)."""
        logits = _f32(logits).copy()
        draft = _i32(draft)
        acc, n_em = C.c_int32(), C.c_int32()
        emitted = np.zeros(draft.size + 1, np.int32)
        rc = lib().yo_spec_verify_reference(self.model.h, self.h, _p(logits), _p(draft), draft.size,
                                            C.byref(acc), _p(emitted), C.byref(n_em))
        if rc != 0:
            raise RuntimeError(f"verify failed: {rc}")
        return acc.value, emitted[:n_em.value].copy(), logits

    def verify_chain(self, pending, draft, want_logits=False):
        draft = _i32(draft)
        acc = C.c_int32()
        emitted = np.zeros(draft.size + 1, np.int32)
        allv = np.empty((draft.size + 1, self.model.vocab), np.float32) if want_logits else None
        rc = lib().yo_verify_chain(self.model.h, self.h, int(pending), _p(draft), draft.size,
                                   C.byref(acc), _p(emitted), _p(allv))
        if rc != 0:
            raise RuntimeError(f"verify_chain failed: {rc}")
        return acc.value, emitted[:acc.value + 1].copy(), allv

    def verify_tree_greedy(self, tokens, parent, want_logits=False):
        tokens, parent = _i32(tokens), _i32(parent)
        n = tokens.size
        acc = C.c_int32()
        path = np.full(n, -1, np.int32)
        emitted = np.zeros(n, np.int32)
        allv = np.empty((n, self.model.vocab), np.float32) if want_logits else None
        rc = lib().yo_verify_tree_greedy(self.model.h, self.h, _p(tokens), _p(parent), n,
                                         C.byref(acc), _p(path), _p(emitted), _p(allv))
        if rc != 0:
            raise RuntimeError(f"verify_tree failed: {rc}")
        a = acc.value
        return a, path[:a].copy(), emitted[:a + 1].copy(), allv

    def close(self):
        if self.h:
            lib().yo_state_destroy(self.h)
            self.h = None
