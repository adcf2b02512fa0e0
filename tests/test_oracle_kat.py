"""The oracle's primitives against the reference's own known-answer vectors.

Each case restates the inputs and expected values of one reference unit test
(cited per test); nothing of the reference is read at run time.
"""
import math
import struct

import numpy as np
import pytest

from oracle import pyoracle as yo


def put_half(buf, off, v):
    h = yo.lib().yo_f32_to_f16(v)
    buf[off] = h & 0xFF
    buf[off + 1] = h >> 8


def test_float16_round_trip():
    # tensor/quant_test.go:14-35
    L = yo.lib()
    for v in [0.0, 1.0, -1.0, 0.5, 65504.0, 6.103515625e-05, 5.960464477539063e-08]:
        got = L.yo_f16_to_f32(L.yo_f32_to_f16(v))
        if v == 0:
            assert got == 0 and math.copysign(1, got) == math.copysign(1, v)
        else:
            assert abs(got - v) <= abs(v) * 0.001
    assert math.isinf(L.yo_f16_to_f32(L.yo_f32_to_f16(float("inf"))))
    assert L.yo_f16_to_f32(L.yo_f32_to_f16(float("-inf"))) == float("-inf")


def test_float16_rounds_half_up():
    # tensor/half.go:59 adds 0x1000 before truncating: ties round away from zero
    L = yo.lib()
    tie = struct.unpack("<f", struct.pack("<I", 0x3F801000))[0]   # 1 + 2^-11
    assert L.yo_f32_to_f16(tie) == 0x3C01


def test_dequantize_q4_0():
    # tensor/quant_test.go:37-55
    src = np.zeros(18, np.uint8)
    put_half(src, 0, 0.5)
    for i in range(16):
        src[2 + i] = (i & 0x0F) | ((15 - i) << 4)
    dst = yo.dequantize_row(yo.Q4_0, src)
    for i in range(16):
        assert dst[i] == 0.5 * (i - 8)
        assert dst[i + 16] == 0.5 * (15 - i - 8)


def test_dequantize_q5_0():
    # tensor/quant_test.go:57-81
    src = np.zeros(22, np.uint8)
    put_half(src, 0, 1.0)
    src[2] = 0x03
    for i in range(16):
        src[6 + i] = i & 0x0F
    dst = yo.dequantize_row(yo.Q5_0, src)
    assert dst[0] == 0 and dst[1] == 1 and dst[2] == -14 and dst[16] == -16


def test_dequantize_q8_0():
    # tensor/quant_test.go:83-99
    src = np.zeros(34, np.uint8)
    put_half(src, 0, 0.5)
    for i in range(32):
        src[2 + i] = (i - 16) & 0xFF
    dst = yo.dequantize_row(yo.Q8_0, src)
    assert np.array_equal(dst, 0.5 * (np.arange(32, dtype=np.float32) - 16))


def test_dequantize_q4_k():
    # tensor/quant_test.go:101-127: scales 1, mins 0, every byte 0x01
    src = np.zeros(144, np.uint8)
    put_half(src, 0, 1.0)
    put_half(src, 2, 0.0)
    src[4:8] = 1
    src[12:16] = 1
    src[16:144] = 0x01
    dst = yo.dequantize_row(yo.Q4_K, src)
    want = np.array([1.0 if i % 64 < 32 else 0.0 for i in range(256)], np.float32)
    assert np.array_equal(dst, want)


def test_dequantize_q5_k():
    # tensor/quant_test.go:129-153
    src = np.zeros(176, np.uint8)
    put_half(src, 0, 1.0)
    put_half(src, 2, 0.0)
    src[4:8] = 1
    src[12:16] = 1
    src[16] = 0x55
    dst = yo.dequantize_row(yo.Q5_K, src)
    for i in (0, 64, 128, 192):
        assert dst[i] == 16
    assert dst[1] == 0


def test_dequantize_q6_k():
    # tensor/quant_test.go:155-172
    src = np.zeros(210, np.uint8)
    src[0] = 0x0F
    src[128] = 0x02
    src[192] = 1
    put_half(src, 208, 1.0)
    dst = yo.dequantize_row(yo.Q6_K, src)
    assert dst[0] == 15 and dst[1] == -32


@pytest.mark.parametrize("dtype", [yo.F32, yo.F16, yo.Q4_0, yo.Q5_0, yo.Q8_0, yo.Q4_K, yo.Q5_K, yo.Q6_K])
def test_matmul_matches_dequantized_dot(dtype):
    # tensor/quant_test.go:252-342: byte pattern (r*37 + i*11) % 255, x = i%9 - 4
    rows, cols = 3, 256
    rb = yo.row_bytes(dtype, cols)
    data = np.zeros(rows * rb, np.uint8)
    for r in range(rows):
        row = data[r * rb:(r + 1) * rb]
        row[:] = (r * 37 + np.arange(rb) * 11) % 255
        if dtype == yo.F32:
            row[:] = np.frombuffer(((np.arange(cols) % 7) - 3).astype("<f4").tobytes(), np.uint8)
        elif dtype == yo.F16:
            for i in range(cols):
                put_half(row, i * 2, float(i % 5) - 2)
        elif dtype in (yo.Q4_0, yo.Q5_0, yo.Q8_0):
            bb = {yo.Q4_0: 18, yo.Q5_0: 22, yo.Q8_0: 34}[dtype]
            for i in range(cols // 32):
                put_half(row, i * bb, 0.03125)
        elif dtype in (yo.Q4_K, yo.Q5_K):
            bb = 144 if dtype == yo.Q4_K else 176
            for i in range(0, rb, bb):
                put_half(row, i, 0.25)
                put_half(row, i + 2, 0.125)
        elif dtype == yo.Q6_K:
            for i in range(0, rb, 210):
                put_half(row, i + 208, 0.25)
    x = ((np.arange(cols) % 9) - 4).astype(np.float32)
    got = yo.matmul(data, dtype, rows, cols, x)[0]
    for r in range(rows):
        dec = yo.dequantize_row(dtype, data[r * rb:(r + 1) * rb])
        s = np.float32(0)
        for i in range(cols):
            s = np.float32(s + np.float32(dec[i] * x[i]))
        assert abs(float(got[r]) - float(s)) <= 1e-5


def test_matmul_thread_count_does_not_change_results():
    rng = np.random.default_rng(0)
    rows, cols = 700, 512
    w = rng.integers(0, 255, rows * yo.row_bytes(yo.Q8_0, cols), dtype=np.uint8)
    for b in range(0, w.size, 34):
        put_half(w, b, 0.01)
    x = rng.standard_normal((3, cols)).astype(np.float32)
    yo.lib().yo_set_threads(1)
    a = yo.matmul(w, yo.Q8_0, rows, cols, x)
    yo.lib().yo_set_threads(0)
    b = yo.matmul(w, yo.Q8_0, rows, cols, x)
    assert np.array_equal(a, b)


def test_kv_format_round_trip():
    # model/qwen35/kv_format_test.go:13-48
    values = (np.sin(np.arange(64) * 0.37) * 3).astype(np.float32)
    values[0] = 0
    for fmt, tol in ((yo.KV_F32, 0), (yo.KV_F16, 1e-3), (yo.KV_Q8_0, 2e-2)):
        dec = yo.kv_decode_row(fmt, yo.kv_encode_row(fmt, values), 64)
        assert np.max(np.abs(dec - values)) <= tol


def test_kv_q8_0_pads_partial_block():
    # model/qwen35/kv_format_test.go:71-79
    assert yo.lib().yo_kv_row_bytes(yo.KV_Q8_0, 40) == 68


def test_table_map():
    # memory/memory.go:253-266
    blocks = [7, 3, 9]
    assert yo.table_map(blocks, 16, 0) == (7, 0)
    assert yo.table_map(blocks, 16, 17) == (3, 1)
    assert yo.table_map(blocks, 16, 47) == (9, 15)
    with pytest.raises(IndexError):
        yo.table_map(blocks, 16, 48)
    with pytest.raises(IndexError):
        yo.table_map(blocks, 16, -1)


def test_lookup_draft():
    # engine/speculative_test.go:139-151
    assert yo.lookup_draft([1, 2, 3, 4, 1, 2, 3], 4, 2) == [4, 1, 2, 3]
    assert yo.lookup_draft([1, 2, 3], 4, 2) == []
    assert yo.lookup_draft([5, 5, 5, 5], 3, 2) == [5]


def test_argmax_first_maximum_wins():
    # engine/speculative.go:263-271
    assert yo.argmax([0, 3, 3, 1]) == 1
    assert yo.argmax([2, 2, 2]) == 0


def test_select_experts():
    # model/qwen35/moe_test.go:129-143
    ids, w = yo.select_experts([0.1, 0.9, 0.5, 0.3], 2)
    assert ids.tolist() == [1, 2]
    assert abs(float(w[0] + w[1]) - 1) <= 1e-6
    assert w[0] > w[1]
    ids, _ = yo.select_experts([0.5, 0.5, 0.5], 2)      # forward.go:408: lowest index wins ties
    assert ids.tolist() == [0, 1]


def test_config_validation_rules():
    # model/qwen35/config.go:231-276
    from yuuka_b200 import synth
    cfg = synth.tiny_config()
    import ctypes as C
    msg = C.create_string_buffer(256)
    ok = yo.Config(**cfg)
    assert yo.lib().yo_config_validate(C.byref(ok), msg, 256) == 0
    for key, bad in (("kv_heads", 3), ("rope_dim", 63), ("rope_dim", 128), ("inner_size", 100),
                     ("conv_kernel", 1), ("full_attention_interval", 0), ("vocab", 0)):
        c = yo.Config(**{**cfg, key: bad})
        assert yo.lib().yo_config_validate(C.byref(c), msg, 256) != 0, key
    # layer i is full attention iff (i+1) % interval == 0 (config.go:280-282)
    assert [yo.lib().yo_is_recurrent(C.byref(ok), i) for i in range(4)] == [1, 1, 1, 0]
