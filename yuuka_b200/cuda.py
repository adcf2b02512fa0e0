"""ctypes mirror of include/yuuka_cuda.h: what the cgo binding does in Go
(backend/hip/hip.go in the reference), for Python tests and the benchmark.

Every call goes through libyuuka_cuda.so. There is no fallback: if the library
is missing or no device answers, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_DEVICE, ERR_ALLOCATION, ERR_INTERNAL = range(6)
F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30
KV_F32, KV_F16, KV_Q8_0 = 0, 1, 2
PATH_AUTO, PATH_FP32, PATH_MMA = 0, 1, 2
GEMM_ACCUMULATE = 1
GEMM_TILED = 2
ACCEPT_GREEDY, ACCEPT_REJECTION, ACCEPT_NONE = 0, 1, 2
SESSION_EXACT_WIDE = 1
SESSION_WIDE_FROM_33 = 2
SESSION_TEST_DROP_COPIES = 0x80000000
GEMM_TEST_DROP_COPIES = 0x80000000
OP_NAMES = {16: "gemm", 18: "rmsnorm", 20: "attn_prep", 24: "embedding", 29: "attention", 37: "lm_head", 9: "silu_mul",
            100: "gdn_scan", 102: "accept", 103: "commit", 104: "moe_route", 105: "moe_experts",
            106: "moe_combine"}
ABI_VERSION = 1


class YuukaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class UnsupportedError(YuukaError):
    """YUUKA_ERR_UNSUPPORTED, the counterpart of hip.ErrUnsupported."""


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("arch", C.c_char * 64), ("cuda_version", C.c_char * 64),
                ("total_memory", C.c_uint64), ("multiprocessors", C.c_uint32), ("clock_mhz", C.c_uint32),
                ("l2_bytes", C.c_uint32), ("smem_per_block_optin", C.c_uint32), ("pci_domain", C.c_int32),
                ("pci_bus", C.c_int32), ("pci_device", C.c_int32)]


class ModelConfig(C.Structure):
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


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("rank", C.c_uint32), ("dims", C.c_uint64 * 8),
                ("bytes", C.c_uint64), ("data", C.c_void_p)]


class SessionConfig(C.Structure):
    _fields_ = [("max_batch", C.c_int32), ("max_nodes", C.c_int32), ("capacity", C.c_int32),
                ("block_size", C.c_int32), ("pool_blocks", C.c_int32), ("kv_format", C.c_int32),
                ("want_logits", C.c_int32), ("flags", C.c_uint32)]


class SessionInfo(C.Structure):
    _fields_ = [("max_batch", C.c_int32), ("max_nodes", C.c_int32), ("capacity", C.c_int32), ("block_size", C.c_int32),
                ("pool_blocks", C.c_int32), ("kv_format", C.c_int32), ("vocab", C.c_int32)]


class SpecOptions(C.Structure):
    _fields_ = [("max_draft", C.c_int32), ("min_match", C.c_int32)]


class SpecRequest(C.Structure):
    _fields_ = [("max_tokens", C.c_int32), ("options", SpecOptions), ("stop_tokens", C.c_void_p), ("n_stop", C.c_int32)]


class SpecResult(C.Structure):
    _fields_ = [("prompt_tokens", C.c_int32), ("output_tokens", C.c_int32), ("finish_reason", C.c_int32),
                ("steps", C.c_int32), ("draft_tokens", C.c_int32), ("accepted_draft", C.c_int32)]


class VerifyBatch(C.Structure):
    _fields_ = [("batch", C.c_int32), ("nodes", C.c_int32), ("tokens", C.c_void_p),
                ("parent", C.c_void_p), ("mode", C.c_uint32), ("temperature", C.c_float),
                ("draft_probs", C.c_void_p), ("uniforms", C.c_void_p), ("accepted", C.c_void_p),
                ("emitted", C.c_void_p), ("path", C.c_void_p), ("logits", C.c_void_p), ("seq_ids", C.c_void_p)]


# name -> (restype, argtypes); the exported symbol list the ABI test checks
_vp, _i32, _u32, _u64, _f32 = C.c_void_p, C.c_int32, C.c_uint32, C.c_uint64, C.c_float
SIGNATURES = {
    "yuuka_abi_version": (_u32, []),
    "yuuka_last_error": (C.c_char_p, []),
    "yuuka_device_open": (_i32, [_i32, _vp]),
    "yuuka_device_close": (None, [_vp]),
    "yuuka_device_info_get": (_i32, [_vp, _vp]),
    "yuuka_device_memory_get": (_i32, [_vp, _vp, _vp]),
    "yuuka_buffer_alloc": (_i32, [_vp, _u64, _vp]),
    "yuuka_buffer_free": (None, [_vp]),
    "yuuka_buffer_size": (_u64, [_vp]),
    "yuuka_buffer_ptr": (_vp, [_vp]),
    "yuuka_stream_create": (_i32, [_vp, _vp]),
    "yuuka_stream_destroy": (None, [_vp]),
    "yuuka_stream_synchronize": (_i32, [_vp]),
    "yuuka_event_create": (_i32, [_vp, _vp]),
    "yuuka_event_destroy": (None, [_vp]),
    "yuuka_event_record": (_i32, [_vp, _vp]),
    "yuuka_event_wait": (_i32, [_vp]),
    "yuuka_event_elapsed_ms": (_i32, [_vp, _vp, _vp]),
    "yuuka_memcpy_h2d": (_i32, [_vp, _vp, _u64]),
    "yuuka_memcpy_h2d_at": (_i32, [_vp, _u64, _vp, _u64]),
    "yuuka_memcpy_d2h": (_i32, [_vp, _vp, _u64]),
    "yuuka_memcpy_d2h_at": (_i32, [_vp, _vp, _u64, _u64]),
    "yuuka_memset": (_i32, [_vp, _vp, _i32, _u64]),
    "yuuka_buffer_copy": (_i32, [_vp, _vp, _u64, _vp, _u64, _u64, _vp]),
    "yuuka_gemm_quant": (_i32, [_vp, _vp, _u64, _vp, _u64, _u32, _vp, _u64, _u32, _u64, _u64, _u64,
                                _u32, _u32, _vp]),
    "yuuka_gemm_quant_static": (_i32, [_vp, _vp, _u64, _vp, _u64, _u32, _vp, _u64, _u32, _u64, _u64, _u64,
                                _u32, _u32, _vp]),
    "yuuka_allocator_create": (_i32, [_i32, _i32, _vp]),
    "yuuka_allocator_destroy": (None, [_vp]),
    "yuuka_allocator_acquire": (_i32, [_vp, _vp]),
    "yuuka_allocator_retain": (_i32, [_vp, _i32]),
    "yuuka_allocator_release": (_i32, [_vp, _i32]),
    "yuuka_allocator_refs": (_i32, [_vp, _i32]),
    "yuuka_allocator_stats_get": (_i32, [_vp, _vp]),
    "yuuka_table_cover": (_i32, [_vp, _vp, _vp, _i32, _i32]),
    "yuuka_table_map": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "yuuka_session_info_get": (_i32, [_vp, _vp]),
    "yuuka_spec_options_normalize": (None, [_vp]),
    "yuuka_spec_lookup_draft": (_i32, [_vp, _i32, _i32, _i32, _vp]),
    "yuuka_spec_generate": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _vp]),
    "yuuka_spec_generate_device": (_i32, [_vp, _i32, _vp, _i32, _vp, _i32, _vp, _vp]),
    "yuuka_spec_lookup_draft_device": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "yuuka_weights_tiled_bytes": (_u64, [_u32, _u64, _u64]),
    "yuuka_weights_tile": (_i32, [_vp, _vp, _u64, _vp, _u64, _u32, _u64, _u64, _vp]),
    "yuuka_model_create": (_i32, [_vp, _vp, _vp]),
    "yuuka_model_destroy": (None, [_vp]),
    "yuuka_model_set_tensor": (_i32, [_vp, C.c_char_p, _u32, _vp, _u64, _u64]),
    "yuuka_model_finalize": (_i32, [_vp]),
    "yuuka_model_weight_bytes": (_u64, [_vp]),
    "yuuka_gguf_open": (_i32, [C.c_char_p, _vp]),
    "yuuka_gguf_close": (None, [_vp]),
    "yuuka_gguf_version": (_u32, [_vp]),
    "yuuka_gguf_alignment": (_u64, [_vp]),
    "yuuka_gguf_tensor_count": (_u64, [_vp]),
    "yuuka_gguf_metadata_count": (_u64, [_vp]),
    "yuuka_gguf_tensor_at": (_i32, [_vp, _u64, _vp]),
    "yuuka_gguf_tensor_find": (_i32, [_vp, C.c_char_p, _vp]),
    "yuuka_gguf_meta_int": (_i32, [_vp, C.c_char_p, _vp]),
    "yuuka_gguf_meta_float": (_i32, [_vp, C.c_char_p, _vp]),
    "yuuka_gguf_meta_string": (_i32, [_vp, C.c_char_p, _vp, _vp]),
    "yuuka_gguf_meta_array_len": (_i32, [_vp, C.c_char_p, _vp]),
    "yuuka_gguf_model_config": (_i32, [_vp, _vp]),
    "yuuka_model_load_gguf": (_i32, [_vp, C.c_char_p, _vp]),
    "yuuka_session_create": (_i32, [_vp, _vp, _vp]),
    "yuuka_session_destroy": (None, [_vp]),
    "yuuka_session_set_block_table": (_i32, [_vp, _i32, _vp, _i32]),
    "yuuka_session_copy_block": (_i32, [_vp, _i32, _i32]),
    "yuuka_session_set_flags": (_i32, [_vp, _u32]),
    "yuuka_session_reset": (_i32, [_vp, _i32]),
    "yuuka_session_set_position": (_i32, [_vp, _i32, _i32]),
    "yuuka_session_position": (_i32, [_vp, _i32, _vp]),
    "yuuka_session_snapshot_bytes": (_u64, [_vp]),
    "yuuka_session_snapshot": (_i32, [_vp, _i32, _vp, _u64]),
    "yuuka_session_restore": (_i32, [_vp, _i32, _vp, _u64]),
    "yuuka_session_prefill_logits": (_i32, [_vp, _i32, _vp, _i32, _vp]),
    "yuuka_session_forward": (_i32, [_vp, _i32, _vp, _i32, _vp]),
    "yuuka_verify_step": (_i32, [_vp, _vp]),
    "yuuka_accept_tree": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _u32, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "yuuka_verify_stage": (_i32, [_vp, _vp]),
    "yuuka_verify_launch": (_i32, [_vp, _vp]),
    "yuuka_verify_fetch": (_i32, [_vp, _vp]),
    "yuuka_verify_launch_profiled": (_i32, [_vp, _vp, _vp, _u64, _vp]),
    "yuuka_session_stream": (_vp, [_vp]),
    "yuuka_session_last_launch_count": (_u32, [_vp]),
}

_lib = None


def lib_path() -> str:
    return _build.CUDA_LIB


def lib():
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            path = _build.build_cuda()
        L = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        if L.yuuka_abi_version() != ABI_VERSION:
            raise RuntimeError(f"libyuuka_cuda ABI {L.yuuka_abi_version()} != binding ABI {ABI_VERSION}")
        _lib = L
    return _lib


def check(status: int) -> None:
    if status == OK:
        return
    msg = lib().yuuka_last_error().decode(errors="replace")
    if status == ERR_UNSUPPORTED:
        raise UnsupportedError(status, msg)
    raise YuukaError(status, msg)


class Device:
    def __init__(self, index: int = 0):
        self.h = C.c_void_p()
        check(lib().yuuka_device_open(index, C.byref(self.h)))
        self.index = index

    def info(self) -> DeviceInfo:
        info = DeviceInfo()
        check(lib().yuuka_device_info_get(self.h, C.byref(info)))
        return info

    def memory(self) -> tuple[int, int]:
        """(free, total) bytes of device memory right now."""
        free, total = C.c_uint64(), C.c_uint64()
        check(lib().yuuka_device_memory_get(self.h, C.byref(free), C.byref(total)))
        return free.value, total.value

    def alloc(self, nbytes: int) -> "Buffer":
        return Buffer(self, nbytes)

    def upload(self, array) -> "Buffer":
        a = np.ascontiguousarray(array)
        buf = Buffer(self, max(a.nbytes, 16))
        buf.write(a)
        return buf

    def stream(self) -> "Stream":
        return Stream(self)

    def event(self) -> "Event":
        return Event(self)

    def close(self):
        if self.h:
            lib().yuuka_device_close(self.h)
            self.h = C.c_void_p()


class Buffer:
    def __init__(self, dev: Device, nbytes: int):
        self.dev = dev
        self.h = C.c_void_p()
        check(lib().yuuka_buffer_alloc(dev.h, nbytes, C.byref(self.h)))
        self.nbytes = nbytes

    def write(self, array, offset: int = 0):
        a = np.ascontiguousarray(array)
        check(lib().yuuka_memcpy_h2d_at(self.h, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def read(self, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype)
        check(lib().yuuka_memcpy_d2h_at(out.ctypes.data_as(C.c_void_p), self.h, offset, out.nbytes))
        return out

    def read_into(self, out: np.ndarray, offset: int = 0):
        check(lib().yuuka_memcpy_d2h_at(out.ctypes.data_as(C.c_void_p), self.h, offset, out.nbytes))

    def free(self):
        if self.h:
            lib().yuuka_buffer_free(self.h)
            self.h = C.c_void_p()


class Stream:
    def __init__(self, dev: Device):
        self.dev = dev
        self.h = C.c_void_p()
        check(lib().yuuka_stream_create(dev.h, C.byref(self.h)))

    def synchronize(self):
        check(lib().yuuka_stream_synchronize(self.h))

    def record(self, event: "Event"):
        check(lib().yuuka_event_record(self.h, event.h))

    def destroy(self):
        if self.h:
            lib().yuuka_stream_destroy(self.h)
            self.h = C.c_void_p()


class Event:
    def __init__(self, dev: Device):
        self.h = C.c_void_p()
        check(lib().yuuka_event_create(dev.h, C.byref(self.h)))

    def wait(self):
        check(lib().yuuka_event_wait(self.h))

    def elapsed_ms(self, end: "Event") -> float:
        ms = C.c_float()
        check(lib().yuuka_event_elapsed_ms(self.h, end.h, C.byref(ms)))
        return ms.value

    def destroy(self):
        if self.h:
            lib().yuuka_event_destroy(self.h)
            self.h = C.c_void_p()


def to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bits (round to nearest even), as uint16."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def from_bf16(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def tiled_bytes(dtype: int, n_out: int, n_in: int) -> int:
    return lib().yuuka_weights_tiled_bytes(dtype, n_out, n_in)


def tile_weights(stream: Stream, dst: Buffer, src: Buffer, dtype: int, n_out: int, n_in: int,
                 dst_offset: int = 0, src_offset: int = 0):
    check(lib().yuuka_weights_tile(stream.h, dst.h, dst_offset, src.h, src_offset, dtype, n_out, n_in, None))


def gemm_quant(stream: Stream, out: Buffer, x: Buffer, w: Buffer, n_in: int, n_out: int, rows: int,
               w_dtype: int, x_dtype: int = F32, path: int = PATH_AUTO, flags: int = 0,
               out_offset: int = 0, x_offset: int = 0, w_offset: int = 0, completion: Event | None = None):
    check(lib().yuuka_gemm_quant(stream.h, out.h, out_offset, x.h, x_offset, x_dtype, w.h, w_offset, w_dtype,
                                 n_in, n_out, rows, path, flags, completion.h if completion else None))


class AllocatorStats(C.Structure):
    _fields_ = [("block_size", C.c_int32), ("total", C.c_int32), ("used", C.c_int32), ("free", C.c_int32),
                ("shared", C.c_int32), ("allocated", C.c_uint64), ("released", C.c_uint64)]


class Allocator:
    """memory.Allocator (memory/memory.go:34-179) behind the C ABI."""

    def __init__(self, blocks: int, block_size: int):
        self.h = C.c_void_p()
        check(lib().yuuka_allocator_create(blocks, block_size, C.byref(self.h)))
        self.block_size = block_size

    def acquire(self) -> int:
        i = C.c_int32()
        check(lib().yuuka_allocator_acquire(self.h, C.byref(i)))
        return i.value

    def retain(self, block: int):
        check(lib().yuuka_allocator_retain(self.h, block))

    def release(self, block: int):
        check(lib().yuuka_allocator_release(self.h, block))

    def refs(self, block: int) -> int:
        return lib().yuuka_allocator_refs(self.h, block)

    def stats(self) -> AllocatorStats:
        st = AllocatorStats()
        check(lib().yuuka_allocator_stats_get(self.h, C.byref(st)))
        return st

    def close(self):
        if self.h:
            lib().yuuka_allocator_destroy(self.h)
            self.h = C.c_void_p()


class Table:
    """memory.Table Cover / Map / Blocks (memory/memory.go:181-266) over an Allocator."""

    def __init__(self, alloc: Allocator, capacity_blocks: int):
        self.alloc = alloc
        self._blocks = np.zeros(max(capacity_blocks, 1), np.int32)
        self._count = C.c_int32(0)

    def cover(self, positions: int):
        check(lib().yuuka_table_cover(self.alloc.h, self._blocks.ctypes.data, C.byref(self._count), self._blocks.size, positions))

    def blocks(self) -> np.ndarray:
        return self._blocks[:self._count.value].copy()

    def map(self, pos: int) -> tuple[int, int]:
        b, o = C.c_int32(), C.c_int32()
        check(lib().yuuka_table_map(self._blocks.ctypes.data, self._count.value, self.alloc.block_size, pos, C.byref(b), C.byref(o)))
        return b.value, o.value


FINISH_LENGTH, FINISH_STOP = 0, 1


def spec_options_normalize(max_draft: int, min_match: int) -> tuple[int, int]:
    """SpeculativeOptions.normalize (engine/speculative.go:21-34)."""
    o = SpecOptions(max_draft, min_match)
    lib().yuuka_spec_options_normalize(C.byref(o))
    return o.max_draft, o.min_match


def spec_lookup_draft(history, max_draft: int, min_match: int) -> list[int]:
    """lookupDraft (engine/speculative.go:39-66)."""
    h = np.ascontiguousarray(history, np.int32)
    out = np.zeros(max(max_draft, 1), np.int32)
    n = lib().yuuka_spec_lookup_draft(h.ctypes.data, h.size, max_draft, min_match, out.ctypes.data)
    return out[:n].tolist()


def spec_generate(sess: "Session", prompt, max_tokens: int, max_draft: int = 0, min_match: int = 0, stop_tokens=(),
                  seq: int = 0):
    """generateSpeculative (engine/speculative.go:68-251) on sequence seq of sess; returns (tokens, SpecResult)."""
    p = np.ascontiguousarray(prompt, np.int32)
    stops = np.ascontiguousarray(list(stop_tokens), np.int32)
    req = SpecRequest(max_tokens, SpecOptions(max_draft, min_match), stops.ctypes.data if stops.size else None, stops.size)
    out = np.zeros(max(max_tokens, 1), np.int32)
    res = SpecResult()
    check(lib().yuuka_spec_generate(sess.h, seq, p.ctypes.data, p.size, C.byref(req), out.ctypes.data, C.byref(res)))
    return out[:res.output_tokens].tolist(), res


def accept_tree(stream: "Stream", logits: "Buffer", tokens, vocab: int, parent=None, mode: int = ACCEPT_GREEDY,
                temperature: float = 1.0, draft_probs: "Buffer | None" = None, uniforms=None, begin: "Event | None" = None,
                end: "Event | None" = None):
    """yuuka_accept_tree: tokens [batch, nodes]; returns (accepted [batch], emitted [batch, nodes], path [batch, nodes])."""
    tokens = np.ascontiguousarray(tokens, np.int32)
    B, N = tokens.shape
    par = None if parent is None else np.ascontiguousarray(np.broadcast_to(np.asarray(parent, np.int32), (B, N)))
    uni = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)
    acc, em, path = np.zeros(B, np.int32), np.full((B, N), -1, np.int32), np.full((B, N), -1, np.int32)
    check(lib().yuuka_accept_tree(stream.h, logits.h, B, N, vocab, tokens.ctypes.data, par.ctypes.data if par is not None else None,
                                  mode, temperature, draft_probs.h if draft_probs is not None else None,
                                  uni.ctypes.data if uni is not None else None, acc.ctypes.data, em.ctypes.data, path.ctypes.data,
                                  begin.h if begin else None, end.h if end else None))
    return acc, em, path


def spec_generate_device(sess: "Session", prompt, max_tokens: int, max_draft: int = 0, min_match: int = 0, stop_tokens=(),
                         seq: int = 0, burst: int = 4):
    """yuuka_spec_generate_device: drafting on the device, `burst` steps per host synchronization."""
    p = np.ascontiguousarray(prompt, np.int32)
    stops = np.ascontiguousarray(list(stop_tokens), np.int32)
    req = SpecRequest(max_tokens, SpecOptions(max_draft, min_match), stops.ctypes.data if stops.size else None, stops.size)
    out = np.zeros(max(max_tokens, 1), np.int32)
    res = SpecResult()
    check(lib().yuuka_spec_generate_device(sess.h, seq, p.ctypes.data, p.size, C.byref(req), burst, out.ctypes.data,
                                           C.byref(res)))
    return out[:res.output_tokens].tolist(), res


def spec_lookup_draft_device(dev: "Device", history, max_draft: int, min_match: int) -> list[int]:
    h = np.ascontiguousarray(history, np.int32)
    hb = dev.upload(h if h.size else np.zeros(1, np.int32))
    ob = dev.alloc(4 * (1 + max(max_draft, 0)))
    st = dev.stream()
    check(lib().yuuka_spec_lookup_draft_device(st.h, hb.h, h.size, max_draft, min_match, ob.h))
    out = ob.read(np.int32, 1 + max(max_draft, 0))
    for b in (hb, ob):
        b.free()
    st.destroy()
    return out[1:1 + int(out[0])].tolist()


STATIC_SCRATCH_BYTES = 8 << 20


def gemm_quant_static(stream: Stream, out: Buffer, x: Buffer, w: Buffer, n_in: int, n_out: int, rows: int,
                      w_dtype: int, x_dtype: int = F32, path: int = PATH_AUTO, flags: int = GEMM_TILED,
                      out_offset: int = 0, x_offset: int = 0, w_offset: int = 0, completion: Event | None = None):
    """yuuka_gemm_quant with its scratch in a fixed device array (allocates nothing)."""
    check(lib().yuuka_gemm_quant_static(stream.h, out.h, out_offset, x.h, x_offset, x_dtype, w.h, w_offset, w_dtype,
                                        n_in, n_out, rows, path, flags, completion.h if completion else None))


class Gguf:
    """Validated read-only view of a GGUF model file (gguf/reader.go). Host only."""

    def __init__(self, path: str):
        self.h = C.c_void_p()
        check(lib().yuuka_gguf_open(os.fsencode(path), C.byref(self.h)))

    @property
    def version(self) -> int:
        return lib().yuuka_gguf_version(self.h)

    @property
    def alignment(self) -> int:
        return lib().yuuka_gguf_alignment(self.h)

    def __len__(self) -> int:
        return lib().yuuka_gguf_tensor_count(self.h)

    @property
    def metadata_count(self) -> int:
        return lib().yuuka_gguf_metadata_count(self.h)

    @staticmethod
    def _view(t: GgufTensor) -> dict:
        data = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(t.bytes,)) if t.bytes else np.zeros(0, np.uint8)
        return dict(name=t.name.decode(), dtype=t.dtype, dims=[int(t.dims[i]) for i in range(t.rank)], bytes=int(t.bytes),
                    data=data)

    def tensor_at(self, index: int) -> dict:
        t = GgufTensor()
        check(lib().yuuka_gguf_tensor_at(self.h, index, C.byref(t)))
        return self._view(t)

    def tensor(self, name: str) -> dict:
        t = GgufTensor()
        check(lib().yuuka_gguf_tensor_find(self.h, name.encode(), C.byref(t)))
        return self._view(t)

    def meta_int(self, key: str) -> int:
        v = C.c_int64()
        check(lib().yuuka_gguf_meta_int(self.h, key.encode(), C.byref(v)))
        return v.value

    def meta_float(self, key: str) -> float:
        v = C.c_double()
        check(lib().yuuka_gguf_meta_float(self.h, key.encode(), C.byref(v)))
        return v.value

    def meta_string(self, key: str) -> str:
        p, n = C.c_void_p(), C.c_uint64()
        check(lib().yuuka_gguf_meta_string(self.h, key.encode(), C.byref(p), C.byref(n)))
        return C.string_at(p, n.value).decode()

    def meta_array_len(self, key: str) -> int:
        v = C.c_uint64()
        check(lib().yuuka_gguf_meta_array_len(self.h, key.encode(), C.byref(v)))
        return v.value

    def model_config(self) -> dict:
        c = ModelConfig()
        check(lib().yuuka_gguf_model_config(self.h, C.byref(c)))
        return {name: getattr(c, name) for name, _ in ModelConfig._fields_}

    def close(self):
        if self.h:
            lib().yuuka_gguf_close(self.h)
            self.h = C.c_void_p()


class Model:
    """Device model: GGUF tensors uploaded verbatim (engine/gpu/model.go:288-301)."""

    def __init__(self, dev: Device, cfg: dict, tensors: dict | None = None):
        self.dev = dev
        self.cfg = dict(cfg)
        self.h = C.c_void_p()
        c = ModelConfig(**cfg)
        check(lib().yuuka_model_create(dev.h, C.byref(c), C.byref(self.h)))
        if tensors is not None:
            for name, (dtype, data, rows, cols) in tensors.items():
                self.set_tensor(name, dtype, data, rows, cols)
            self.finalize()

    @classmethod
    def from_gguf(cls, dev: Device, path: str) -> "Model":
        """yuuka_model_load_gguf: config from the file's metadata, every tensor uploaded, finalized."""
        g = Gguf(path)
        try:
            cfg = g.model_config()
        finally:
            g.close()
        self = cls.__new__(cls)
        self.dev = dev
        self.cfg = cfg
        self.h = C.c_void_p()
        check(lib().yuuka_model_load_gguf(dev.h, os.fsencode(path), C.byref(self.h)))
        return self

    def set_tensor(self, name: str, dtype: int, data, rows: int, cols: int):
        a = np.ascontiguousarray(data)
        check(lib().yuuka_model_set_tensor(self.h, name.encode(), dtype, a.ctypes.data_as(C.c_void_p), rows, cols))

    def finalize(self):
        check(lib().yuuka_model_finalize(self.h))

    @property
    def weight_bytes(self) -> int:
        return lib().yuuka_model_weight_bytes(self.h)

    @property
    def vocab(self) -> int:
        return self.cfg["vocab"]

    def close(self):
        if self.h:
            lib().yuuka_model_destroy(self.h)
            self.h = C.c_void_p()


class VerifyResult:
    def __init__(self, accepted, emitted, path, logits):
        self.accepted, self.emitted, self.path, self.logits = accepted, emitted, path, logits


class Session:
    """Paged KV pool, block tables, recurrent state and step buffers for up to
    max_batch sequences (engine/gpu/session.go holds one sequence)."""

    def __init__(self, model: Model, max_batch: int = 1, max_nodes: int = 16, capacity: int = 512,
                 kv_format: int = KV_F16, block_size: int = 0, pool_blocks: int = 0, want_logits: bool = True,
                 flags: int = 0):
        self.model = model
        self.max_batch, self.max_nodes, self.capacity = max_batch, max_nodes, capacity
        cfg = SessionConfig(max_batch, max_nodes, capacity, block_size, pool_blocks, kv_format, int(want_logits), flags)
        self.h = C.c_void_p()
        check(lib().yuuka_session_create(model.h, C.byref(cfg), C.byref(self.h)))
        self._staged = None

    def set_block_table(self, seq: int, blocks):
        b = np.ascontiguousarray(blocks, np.int32)
        check(lib().yuuka_session_set_block_table(self.h, seq, b.ctypes.data_as(C.c_void_p), b.size))

    def reset(self, seq: int = 0):
        check(lib().yuuka_session_reset(self.h, seq))

    def set_position(self, seq: int, pos: int):
        check(lib().yuuka_session_set_position(self.h, seq, pos))

    def position(self, seq: int = 0) -> int:
        v = C.c_int32()
        check(lib().yuuka_session_position(self.h, seq, C.byref(v)))
        return v.value

    def snapshot(self, seq: int = 0) -> np.ndarray:
        n = lib().yuuka_session_snapshot_bytes(self.h)
        out = np.empty(n, np.uint8)
        check(lib().yuuka_session_snapshot(self.h, seq, out.ctypes.data_as(C.c_void_p), n))
        return out

    def restore(self, data, seq: int = 0):
        d = np.ascontiguousarray(data, np.uint8)
        check(lib().yuuka_session_restore(self.h, seq, d.ctypes.data_as(C.c_void_p), d.size))

    def prefill_logits(self, tokens, seq: int = 0) -> np.ndarray:
        t = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((t.size, self.model.vocab), np.float32)
        check(lib().yuuka_session_prefill_logits(self.h, seq, t.ctypes.data_as(C.c_void_p), t.size,
                                                 out.ctypes.data_as(C.c_void_p)))
        return out

    def forward(self, tokens, seq: int = 0, want_logits: bool = True):
        t = np.ascontiguousarray(tokens, np.int32)
        out = np.empty(self.model.vocab, np.float32) if want_logits else None
        check(lib().yuuka_session_forward(self.h, seq, t.ctypes.data_as(C.c_void_p), t.size,
                                          out.ctypes.data_as(C.c_void_p) if want_logits else None))
        return out

    def set_flags(self, flags: int):
        check(lib().yuuka_session_set_flags(self.h, flags))

    def copy_block(self, dst_block: int, src_block: int):
        check(lib().yuuka_session_copy_block(self.h, dst_block, src_block))

    def _batch(self, tokens, parent, mode, want_logits, temperature=1.0, draft_probs=None, uniforms=None, seq_ids=None):
        tokens = np.ascontiguousarray(tokens, np.int32)
        if tokens.ndim == 1:
            tokens = tokens[None, :]
        B, N = tokens.shape
        par = None
        if parent is not None:
            par = np.ascontiguousarray(np.broadcast_to(np.asarray(parent, np.int32), (B, N)))
        keep = dict(tokens=tokens, parent=par, accepted=np.zeros(B, np.int32), emitted=np.full((B, N), -1, np.int32),
                    path=np.full((B, N), -1, np.int32),
                    logits=np.empty((B, N, self.model.vocab), np.float32) if want_logits else None)
        vb = VerifyBatch()
        vb.batch, vb.nodes = B, N
        vb.tokens = tokens.ctypes.data
        vb.parent = par.ctypes.data if par is not None else None
        vb.mode, vb.temperature = mode, temperature
        if draft_probs is not None:
            vb.draft_probs = draft_probs.h  # Buffer: f32 [batch, nodes, vocab] on the device
        if uniforms is not None:
            keep["uniforms"] = np.ascontiguousarray(uniforms, np.float32)
            assert keep["uniforms"].size == B * N * 2
            vb.uniforms = keep["uniforms"].ctypes.data
        vb.accepted = keep["accepted"].ctypes.data
        vb.emitted = keep["emitted"].ctypes.data
        vb.path = keep["path"].ctypes.data
        vb.logits = keep["logits"].ctypes.data if want_logits else None
        if seq_ids is not None:
            keep["seq_ids"] = np.ascontiguousarray(seq_ids, np.int32)
            assert keep["seq_ids"].size == B
            vb.seq_ids = keep["seq_ids"].ctypes.data
        return vb, keep

    @staticmethod
    def _result(keep) -> VerifyResult:
        return VerifyResult(keep["accepted"], keep["emitted"], keep["path"], keep["logits"])

    def verify(self, tokens, parent=None, mode: int = ACCEPT_GREEDY, want_logits: bool = False,
               temperature: float = 1.0, draft_probs: "Buffer | None" = None, uniforms=None, seq_ids=None) -> VerifyResult:
        """One verify step; tokens [batch, nodes] with the pending token in column 0.

        mode ACCEPT_REJECTION needs temperature, draft_probs (device Buffer, f32 [batch, nodes, vocab])
        and uniforms (f32 [batch, nodes, 2] in [0, 1)).
        """
        vb, keep = self._batch(tokens, parent, mode, want_logits, temperature, draft_probs, uniforms, seq_ids)
        check(lib().yuuka_verify_step(self.h, C.byref(vb)))
        return self._result(keep)

    def stage(self, tokens, parent=None, mode: int = ACCEPT_GREEDY, want_logits: bool = False, seq_ids=None,
              temperature: float = 1.0, draft_probs: "Buffer | None" = None, uniforms=None):
        vb, keep = self._batch(tokens, parent, mode, want_logits, temperature, draft_probs, uniforms, seq_ids)
        check(lib().yuuka_verify_stage(self.h, C.byref(vb)))
        self._staged = (vb, keep)

    def launch(self, completion: Event | None = None):
        check(lib().yuuka_verify_launch(self.h, completion.h if completion else None))

    def launch_profiled(self, capacity: int = 4096):
        """Runs the staged step with per-op events; returns [(op_code, nanoseconds)]."""
        codes = np.zeros(capacity, np.uint32)
        times = np.zeros(capacity, np.uint64)
        n = C.c_uint64()
        check(lib().yuuka_verify_launch_profiled(self.h, codes.ctypes.data_as(C.c_void_p),
                                                 times.ctypes.data_as(C.c_void_p), capacity, C.byref(n)))
        return list(zip(codes[:n.value].tolist(), times[:n.value].tolist()))

    def fetch(self) -> VerifyResult:
        vb, keep = self._staged
        check(lib().yuuka_verify_fetch(self.h, C.byref(vb)))
        return self._result(keep)

    def stream_handle(self):
        return lib().yuuka_session_stream(self.h)

    def record(self, event: Event):
        check(lib().yuuka_event_record(self.stream_handle(), event.h))

    @property
    def last_launch_count(self) -> int:
        return lib().yuuka_session_last_launch_count(self.h)

    def close(self):
        if self.h:
            lib().yuuka_session_destroy(self.h)
            self.h = C.c_void_p()
