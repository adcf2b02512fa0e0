"""GGUF reader (csrc/gguf.cu) against files written by yuuka_b200/gguf_writer.py: the accept and
reject cases gguf/reader_test.go covers (valid file, nested arrays, malformed headers, metadata,
tensor directory, alignment, ranges, overlaps, split shards) and the config rules of
model/qwen35/config.go:48-174. Host code only: no GPU."""
import struct

import numpy as np
import pytest

from yuuka_b200 import cuda, gguf_writer as gw, synth

F32_T, Q8_0_T = 0, 8


def vec(n, seed=0):
    return (F32_T, np.arange(n, dtype=np.float32) + seed, 1, n)


def reject(path, status=cuda.ERR_INVALID_ARGUMENT, text=None):
    with pytest.raises(cuda.YuukaError) as e:
        cuda.Gguf(str(path))
    assert e.value.status == status, str(e.value)
    if text:
        assert text in str(e.value), str(e.value)


def test_valid_file_metadata_and_tensor_views(tmp_path):
    p = tmp_path / "m.gguf"
    a = np.arange(6, dtype=np.float32)
    q = np.arange(2 * 34, dtype=np.uint8)
    md = [("general.architecture", gw.STR, "llama"), ("n.u8", gw.U8, 7), ("n.i16", gw.I16, -3), ("n.u64", gw.U64, 1 << 40),
          ("x.f32", gw.F32, 0.5), ("x.f64", gw.F64, 1e-6), ("flag", gw.BOOL, 1),
          ("arr", gw.ARR, (gw.I32, [1, 2, 3])), ("names", gw.ARR, (gw.STR, ["a", "bc"]))]
    gw.write(str(p), md, {"w": (F32_T, a, 2, 3), "q": (Q8_0_T, q, 2, 32), "v": vec(5)})
    g = cuda.Gguf(str(p))
    assert g.version == 3 and g.alignment == 32 and len(g) == 3 and g.metadata_count == len(md)
    assert g.meta_string("general.architecture") == "llama"
    assert g.meta_int("n.u8") == 7 and g.meta_int("n.i16") == -3 and g.meta_int("n.u64") == 1 << 40
    assert g.meta_float("x.f32") == 0.5 and g.meta_float("x.f64") == 1e-6
    assert g.meta_array_len("arr") == 3 and g.meta_array_len("names") == 2
    for bad in (lambda: g.meta_int("x.f32"), lambda: g.meta_float("n.u8"), lambda: g.meta_string("arr"),
                lambda: g.meta_int("missing"), lambda: g.meta_array_len("flag")):
        with pytest.raises(cuda.YuukaError):
            bad()
    w = g.tensor("w")
    assert w["dims"] == [3, 2] and w["dtype"] == F32_T and w["bytes"] == 24
    assert np.array_equal(w["data"].view(np.float32), a)
    t1 = g.tensor_at(1)
    assert t1["name"] == "q" and t1["dims"] == [32, 2] and t1["bytes"] == 68 and np.array_equal(t1["data"], q)
    assert g.tensor_at(2)["dims"] == [5]
    with pytest.raises(cuda.YuukaError):
        g.tensor("absent")
    with pytest.raises(cuda.YuukaError):
        g.tensor_at(3)
    g.close()
    g.close()  # idempotent


def test_version_2_alignment_key_and_nested_arrays(tmp_path):
    p = tmp_path / "m.gguf"
    nested = (gw.ARR, [(gw.U8, [1, 2]), (gw.U8, [3])])
    gw.write(str(p), [("nest", gw.ARR, nested)], {"a": vec(3), "b": vec(70, 1)}, version=2, alignment=64)
    g = cuda.Gguf(str(p))
    assert g.version == 2 and g.alignment == 64 and g.meta_array_len("nest") == 2
    assert np.array_equal(g.tensor("b")["data"].view(np.float32), np.arange(70, dtype=np.float32) + 1)
    g.close()
    # a file without tensors may end right after the directory
    gw.write(str(p), [("k", gw.U32, 1)], {})
    g = cuda.Gguf(str(p))
    assert len(g) == 0
    g.close()


def _header(version=3, tensors=0, metadata=0, magic=b"GGUF"):
    return magic + struct.pack("<IQQ", version, tensors, metadata)


def _tensor_entry(name, dims, dtype, offset):
    return gw._str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", dtype, offset)


def test_rejects_malformed_headers_and_metadata(tmp_path):
    p = tmp_path / "bad.gguf"
    cases = [
        (_header(magic=b"GGML"), cuda.ERR_INVALID_ARGUMENT, "bad magic"),
        (b"GGUF\x03\x00", cuda.ERR_INVALID_ARGUMENT, "truncated"),
        (_header(version=1), cuda.ERR_UNSUPPORTED, "version 1"),
        (_header(version=4), cuda.ERR_UNSUPPORTED, "version 4"),
        (_header(tensors=(1 << 24) + 1), cuda.ERR_INVALID_ARGUMENT, "tensor count"),
        (_header(metadata=(1 << 20) + 1), cuda.ERR_INVALID_ARGUMENT, "metadata count"),
        (_header(metadata=1) + gw._str("a") + struct.pack("<I", 99), cuda.ERR_INVALID_ARGUMENT, "unknown metadata type"),
        (_header(metadata=1) + gw._str("") + struct.pack("<II", gw.U32, 1), cuda.ERR_INVALID_ARGUMENT, "empty metadata key"),
        (_header(metadata=2) + (gw._str("a") + struct.pack("<II", gw.U32, 1)) * 2, cuda.ERR_INVALID_ARGUMENT, "duplicate metadata"),
        (_header(metadata=1) + gw._str("b") + struct.pack("<IB", gw.BOOL, 2), cuda.ERR_INVALID_ARGUMENT, "invalid bool"),
        (_header(metadata=1) + gw._str("s") + struct.pack("<IQ", gw.STR, 1 << 31), cuda.ERR_INVALID_ARGUMENT, "string length"),
        (_header(metadata=1) + gw._str("a") + struct.pack("<IIQ", gw.ARR, gw.U32, 1 << 20), cuda.ERR_INVALID_ARGUMENT, "exceeds remaining"),
        (_header(metadata=1) + gw._str("a") + struct.pack("<IIQ", gw.ARR, 77, 1), cuda.ERR_INVALID_ARGUMENT, "array element type"),
        (_header(metadata=1) + gw._str("general.alignment") + struct.pack("<II", gw.U32, 48), cuda.ERR_INVALID_ARGUMENT, "power of two"),
        (_header(metadata=1) + gw._str("general.alignment") + struct.pack("<If", gw.F32, 32.0), cuda.ERR_INVALID_ARGUMENT, "alignment"),
    ]
    for blob, status, text in cases:
        p.write_bytes(blob)
        reject(p, status, text)
    p.write_bytes(b"")
    reject(p, cuda.ERR_INVALID_ARGUMENT, "empty file")
    reject(tmp_path / "absent.gguf", cuda.ERR_INVALID_ARGUMENT, "open")
    # arrays nested deeper than the limit
    deep = struct.pack("<I", gw.ARR)
    for _ in range(6):
        deep += struct.pack("<IQ", gw.ARR, 1) + struct.pack("<I", gw.ARR)
    p.write_bytes(_header(metadata=1) + gw._str("d") + deep + struct.pack("<IQ", gw.U8, 0))
    reject(p, cuda.ERR_INVALID_ARGUMENT, "nesting")


def test_rejects_malformed_tensor_directories(tmp_path):
    p = tmp_path / "bad.gguf"
    pad = b"\0" * 256
    cases = [
        ([("w", [1] * 9, F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "invalid rank"),
        ([("w", [], F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "invalid rank"),
        ([("w", [2], F32_T, 0), ("w", [2], F32_T, 32)], cuda.ERR_INVALID_ARGUMENT, "duplicate tensor"),
        ([("", [2], F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "empty tensor name"),
        ([("w", [0], F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "zero dimension"),
        ([("w", [1 << 40, 1 << 40], F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "overflows"),
        ([("w", [31, 2], Q8_0_T, 0)], cuda.ERR_INVALID_ARGUMENT, "not a multiple of 32"),
        ([("w", [2], 99, 0)], cuda.ERR_UNSUPPORTED, "dtype 99"),
        ([("w", [2], F32_T, 1 << 20)], cuda.ERR_INVALID_ARGUMENT, "exceeds shard size"),
        ([("w", [2], F32_T, 8)], cuda.ERR_INVALID_ARGUMENT, "not aligned"),
        ([("a", [4], F32_T, 0), ("b", [4], F32_T, 0)], cuda.ERR_INVALID_ARGUMENT, "overlap"),
    ]
    for tensors, status, text in cases:
        blob = _header(tensors=len(tensors)) + b"".join(_tensor_entry(*t) for t in tensors)
        blob += b"\0" * (-len(blob) % 32) + pad
        p.write_bytes(blob)
        reject(p, status, text)
    # directory present but the data section would start past the end of the file
    blob = _header(tensors=1, metadata=1) + gw._str("general.alignment") + struct.pack("<II", gw.U32, 4096)
    blob += _tensor_entry("w", [2], F32_T, 0)
    p.write_bytes(blob)
    reject(p, cuda.ERR_INVALID_ARGUMENT, "beyond end of file")


def _shard(path, no, count, tensors, extra=()):
    gw.write(str(path), [("split.no", gw.U16, no), ("split.count", gw.U16, count), *extra], tensors)


def test_split_shards(tmp_path):
    a, b = tmp_path / "m-00001-of-00002.gguf", tmp_path / "m-00002-of-00002.gguf"
    _shard(a, 0, 2, {"x": vec(4)}, extra=[("general.architecture", gw.STR, "qwen35")])
    _shard(b, 1, 2, {"y": vec(6, 10)})
    g = cuda.Gguf(str(a))
    assert len(g) == 2 and g.tensor_at(0)["name"] == "x" and g.tensor_at(1)["name"] == "y"
    assert np.array_equal(g.tensor("y")["data"].view(np.float32), np.arange(6, dtype=np.float32) + 10)
    g.close()
    b.unlink()
    reject(a, cuda.ERR_INVALID_ARGUMENT, "open")                      # missing shard
    _shard(b, 1, 2, {"x": vec(4)})
    reject(a, cuda.ERR_INVALID_ARGUMENT, "more than one shard")       # same tensor twice
    _shard(b, 0, 2, {"y": vec(4)})
    reject(a, cuda.ERR_INVALID_ARGUMENT, "split.no")
    _shard(b, 1, 3, {"y": vec(4)})
    reject(a, cuda.ERR_INVALID_ARGUMENT, "split.count")
    gw.write(str(b), [("split.no", gw.U16, 1), ("split.count", gw.U16, 2)], {"y": vec(4)}, alignment=64)
    reject(a, cuda.ERR_INVALID_ARGUMENT, "differs from shard 0")
    c = tmp_path / "m-00001-of-00003.gguf"
    _shard(c, 0, 2, {"x": vec(4)})
    reject(c, cuda.ERR_INVALID_ARGUMENT, "does not match file name")
    d = tmp_path / "plain.gguf"
    _shard(d, 0, 2, {"x": vec(4)})
    reject(d, cuda.ERR_INVALID_ARGUMENT, "NNNNN-of-NNNNN")


def test_model_config_from_metadata(tmp_path):
    p = tmp_path / "m.gguf"
    cfg = synth.tiny_config()
    gw.write(str(p), gw.config_metadata(cfg), {"v": vec(2)})
    g = cuda.Gguf(str(p))
    got = g.model_config()
    assert got["rms_eps"] == np.float32(cfg["rms_eps"]) and got["rope_freq_base"] == np.float32(cfg["rope_freq_base"])
    for k, v in cfg.items():
        if k not in ("rms_eps", "rope_freq_base"):
            assert got[k] == v, k
    g.close()
    # vocabulary from the tokenizer's token list; MoE keys; shared width defaults to the expert width
    moe = synth.tiny_moe_config()
    md = [m for m in gw.config_metadata(moe, tokens=True) if not m[0].endswith("expert_shared_feed_forward_length")]
    md = [(k, gw.ARR, (gw.U32, [moe["expert_ffn"]] * moe["block_count"])) if k.endswith("expert_feed_forward_length") else (k, t, v)
          for k, t, v in md]
    gw.write(str(p), md, {"v": vec(2)})
    g = cuda.Gguf(str(p))
    got = g.model_config()
    assert got["vocab"] == moe["vocab"] and got["expert_count"] == 8 and got["expert_ffn"] == 256 and got["shared_ffn"] == 256
    assert got["ffn"] == 0
    g.close()

    def config_error(metadata, text, status=cuda.ERR_INVALID_ARGUMENT):
        gw.write(str(p), metadata, {"v": vec(2)})
        g = cuda.Gguf(str(p))
        with pytest.raises(cuda.YuukaError) as e:
            g.model_config()
        g.close()
        assert e.value.status == status and text in str(e.value), str(e.value)

    base = gw.config_metadata(cfg)
    config_error([m for m in base if m[0] != "qwen35.block_count"], "missing required metadata qwen35.block_count")
    config_error([("general.architecture", gw.STR, "llama")] + base[1:], "not \"qwen35\"", cuda.ERR_UNSUPPORTED)
    config_error([(k, t, 0) if k == "qwen35.ssm.state_size" else (k, t, v) for k, t, v in base], "invalid value 0")
    config_error([(k, gw.F32, 4.0) if k == "qwen35.attention.head_count" else (k, t, v) for k, t, v in base], "not an integer")
    config_error([(k, gw.U32, 1) if k == "qwen35.rope.freq_base" else (k, t, v) for k, t, v in base], "not a float")
    config_error([m for m in base if m[0] != "qwen35.vocab_size"], "vocabulary size is unavailable")
    config_error(base + [("qwen35.rope.scaling.type", gw.STR, "yarn")], "rope.scaling", cuda.ERR_UNSUPPORTED)
    config_error([(k, t, (gw.I32, [1, 2, 3])) if k.endswith("dimension_sections") else (k, t, v) for k, t, v in base], "4 entries")
    varied = [(k, gw.ARR, (gw.U32, [256, 512])) if k.endswith("expert_feed_forward_length") else (k, t, v)
              for k, t, v in gw.config_metadata(moe)]
    config_error(varied, "varies at layer 1", cuda.ERR_UNSUPPORTED)


def test_rope_scaling_names_that_mean_unscaled(tmp_path):
    p = tmp_path / "m.gguf"
    base = gw.config_metadata(synth.tiny_config())
    for text in ("", "none", " None ", "DEFAULT"):
        gw.write(str(p), base + [("qwen35.rope.scaling.type", gw.STR, text)], {"v": vec(2)})
        g = cuda.Gguf(str(p))
        assert g.model_config()["hidden"] == 256
        g.close()
