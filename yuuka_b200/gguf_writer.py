"""Writes a model as a GGUF file (format versions 2 and 3), for synthetic models and for tests of
the reader in csrc/gguf.cu. Layout as gguf/reader.go parses it: magic, version, counts, metadata
key/value pairs, tensor directory (name, rank, dims in GGML order, type id, offset), padding to
general.alignment, tensor data at aligned offsets.
"""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _str(s) -> bytes:
    b = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(b)) + b


def value(typ: int, v) -> bytes:
    """One metadata value without its type tag. Arrays are (elem_type, [items])."""
    if typ == STR:
        return _str(v)
    if typ == ARR:
        elem, items = v
        out = struct.pack("<IQ", elem, len(items))
        for it in items:
            if elem == ARR:
                out += struct.pack("<I", ARR)
            out += value(elem, it)
        return out
    return struct.pack(_FMT[typ], v)


def config_metadata(cfg: dict, arch: str | None = None, tokens: bool = False) -> list:
    """(key, type, value) triples for a model config (the keys model/qwen35/config.go:48-174 reads)."""
    moe = cfg.get("expert_count", 0) > 0
    arch = arch or ("qwen35moe" if moe else "qwen35")
    k = lambda name: f"{arch}.{name}"
    md = [("general.architecture", STR, arch),
          (k("block_count"), U32, cfg["block_count"]), (k("context_length"), U32, cfg["context_length"]),
          (k("embedding_length"), U32, cfg["hidden"]),
          (k("attention.head_count"), U32, cfg["heads"]), (k("attention.head_count_kv"), U32, cfg["kv_heads"]),
          (k("attention.key_length"), U32, cfg["head_dim"]), (k("attention.value_length"), U32, cfg["head_dim"]),
          (k("rope.dimension_count"), U32, cfg["rope_dim"]), (k("rope.freq_base"), F32, cfg["rope_freq_base"]),
          (k("attention.layer_norm_rms_epsilon"), F32, cfg["rms_eps"]),
          (k("ssm.conv_kernel"), U32, cfg["conv_kernel"]), (k("ssm.state_size"), U32, cfg["state_size"]),
          (k("ssm.group_count"), U32, cfg["group_count"]), (k("ssm.time_step_rank"), U32, cfg["time_step_rank"]),
          (k("ssm.inner_size"), U32, cfg["inner_size"]), (k("full_attention_interval"), U32, cfg["full_attention_interval"]),
          (k("rope.dimension_sections"), ARR, (I32, [cfg["rope_dim"] // 4, cfg["rope_dim"] // 4, 0, 0]))]
    if moe:
        md += [(k("expert_count"), U32, cfg["expert_count"]), (k("expert_used_count"), U32, cfg["expert_used"]),
               (k("expert_feed_forward_length"), U32, cfg["expert_ffn"]),
               (k("expert_shared_feed_forward_length"), U32, cfg["shared_ffn"])]
    else:
        md.append((k("feed_forward_length"), U32, cfg["ffn"]))
    if tokens:
        md.append(("tokenizer.ggml.tokens", ARR, (STR, [f"t{i}" for i in range(cfg["vocab"])])))
    else:
        md.append((k("vocab_size"), U32, cfg["vocab"]))
    return md


def tensor_dims(name: str, rows: int, cols: int, cfg: dict | None = None) -> list[int]:
    """GGML dims of a tensor given as rows x cols: [cols] for vectors, [cols, rows] for matrices,
    [kernel, channels] for ssm_conv1d and [cols, rows / experts, experts] for stacked expert tensors."""
    if name.endswith("ssm_conv1d.weight") and cfg:
        k = cfg["conv_kernel"]
        return [k, rows * cols // k]
    if "_exps." in name and cfg and cfg.get("expert_count", 0) > 0:
        return [cols, rows // cfg["expert_count"], cfg["expert_count"]]
    return [cols] if rows == 1 else [cols, rows]


def write(path: str, metadata: list, tensors: dict, cfg: dict | None = None, version: int = 3, alignment: int = 32,
          offsets: dict | None = None) -> None:
    """tensors: name -> (dtype id, array, rows, cols). offsets overrides the data offset of named tensors
    (to build malformed files)."""
    md = list(metadata)
    if alignment != 32:
        md.append(("general.alignment", U32, alignment))
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(md))
    for key, typ, v in md:
        head += _str(key) + struct.pack("<I", typ) + value(typ, v)
    directory, blobs, off = b"", [], 0
    for name, (dtype, data, rows, cols) in tensors.items():
        raw = np.ascontiguousarray(data).view(np.uint8).ravel()
        dims = tensor_dims(name, rows, cols, cfg)
        at = offsets[name] if offsets and name in offsets else off
        directory += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        directory += struct.pack("<IQ", dtype, at)
        blobs.append((off, raw))
        off = (off + raw.size + alignment - 1) // alignment * alignment
    start = (len(head) + len(directory) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + directory)
        f.write(b"\0" * (start - len(head) - len(directory)))
        pos = 0
        for at, raw in blobs:
            f.write(b"\0" * (at - pos))
            f.write(raw.tobytes())
            pos = at + raw.size
        f.write(b"\0" * (off - pos))
