"""Quantized GEMM kernels against the CPU oracle (tensor/quant.go matvec), through the C ABI."""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = cuda.Device(0)
    yield d
    d.close()


def run_gemm(dev, w_packed, w_dtype, n_out, n_in, x, path, x_dtype=cuda.F32, accumulate=None, tiled=True):
    stream = dev.stream()
    raw = dev.alloc(w_packed.nbytes + 256)
    raw.write(w_packed)
    if tiled:
        wb = dev.alloc(cuda.tiled_bytes(w_dtype, n_out, n_in) + 256)
        cuda.tile_weights(stream, wb, raw, w_dtype, n_out, n_in)
        stream.synchronize()
        raw.free()
    else:
        wb = raw
    xb = dev.upload(cuda.to_bf16(x) if x_dtype == cuda.BF16 else x.astype(np.float32))
    rows = x.shape[0]
    ob = dev.alloc(rows * n_out * 4)
    flags = cuda.GEMM_TILED if tiled else 0
    if accumulate is not None:
        ob.write(accumulate.astype(np.float32))
        flags |= cuda.GEMM_ACCUMULATE
    cuda.gemm_quant(stream, ob, xb, wb, n_in, n_out, rows, w_dtype, x_dtype, path, flags)
    stream.synchronize()
    out = ob.read(np.float32, rows * n_out).reshape(rows, n_out)
    for b in (wb, xb, ob):
        b.free()
    stream.destroy()
    return out


def stats(got, want):
    err = np.abs(got - want)
    cos = float(np.dot(got.ravel(), want.ravel()) / (np.linalg.norm(got) * np.linalg.norm(want)))
    return float(err.max()), cos


CASES = [(dt, m) for dt in (synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q5_K) for m in (1, 2, 4, 9, 16, 33)]


@pytest.mark.parametrize("dtype,rows", CASES)
def test_fp32_route_matches_oracle(dev, dtype, rows):
    n_out, n_in = 520, 2560
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, 100 + dtype)
    x = synth.normal_f32(rows * n_in, 1.0, 7 + rows).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_FP32)
    # same fp32 decode, different summation order
    assert np.max(np.abs(got - want)) <= 2e-5 * (1 + np.max(np.abs(want)))


@pytest.mark.parametrize("dtype,rows", CASES)
def test_mma_route_matches_oracle(dev, dtype, rows):
    n_out, n_in = 520, 2560
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, 200 + dtype)
    x = synth.normal_f32(rows * n_in, 1.0, 17 + rows).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    err, cos = stats(got, want)
    # outputs have std ~1. Up to 47 rows: exact integer weights and two-half activations, fp32 accumulate (measured
    # 1e-5); from 48 rows: the tensor-memory route with fp16-rounded operands
    assert err <= (2e-4 if rows < 48 else 4e-3) and cos >= 0.999999, (err, cos)


@pytest.mark.parametrize("n_out,n_in,dtype", [
    (9216, 2560, synth.Q4_K), (2560, 2560, synth.Q4_K), (2560, 9216, synth.Q6_K), (2560, 4096, synth.Q4_K),
    (32, 2560, synth.Q4_K), (12352, 2560, synth.Q4_K), (1000, 768, synth.Q8_0), (4096, 256, synth.Q8_0),
])
def test_mma_route_model_shapes(dev, n_out, n_in, dtype):
    rows = 9
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, n_out + n_in)
    x = synth.normal_f32(rows * n_in, 1.0, 3).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    err, cos = stats(got, want)
    assert err <= 4e-4 and cos >= 0.999999, (err, cos)
    # run-twice bitwise determinism (split-K partials are reduced in a fixed order)
    again = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    assert np.array_equal(got, again)


def test_bf16_activations_microbench_shape(dev):
    # kernel microbench shape: K=2560, N=9216 Q4_K, bf16 activations N(0,1)
    n_out, n_in, rows = 9216, 2560, 16
    w = synth.normal_quant(n_out, n_in, synth.Q4_K, 0.02, 5)
    x = synth.normal_f32(rows * n_in, 1.0, 9).reshape(rows, n_in)
    xb = cuda.from_bf16(cuda.to_bf16(x)).reshape(rows, n_in)
    want = yo.matmul(w, synth.Q4_K, n_out, n_in, xb)
    for path in (cuda.PATH_MMA, cuda.PATH_FP32):
        got = run_gemm(dev, w, synth.Q4_K, n_out, n_in, x, path, x_dtype=cuda.BF16)
        err, cos = stats(got, want)
        assert err <= 8e-3 and cos >= 0.999999, (path, err, cos)


def test_lm_head_shape_q6_k(dev):
    n_out, n_in, rows = 248320, 2560, 9
    w = synth.normal_quant(n_out, n_in, synth.Q6_K, 0.02, 77)
    x = synth.normal_f32(rows * n_in, 1.0, 78).reshape(rows, n_in)
    want = yo.matmul(w, synth.Q6_K, n_out, n_in, x)
    got = run_gemm(dev, w, synth.Q6_K, n_out, n_in, x, cuda.PATH_AUTO)
    err, cos = stats(got, want)
    assert err <= 4e-4 and cos >= 0.999999, (err, cos)
    assert np.array_equal(np.argmax(got, -1), np.argmax(want, -1)) or err < 1e-4


@pytest.mark.parametrize("dtype", [synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q5_K])
def test_gguf_layout_route_matches_oracle(dev, dtype):
    # weights left in GGUF row-major order take the generic fp32 kernel
    n_out, n_in, rows = 300, 1280 if dtype != synth.Q8_0 else 96, 5
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, 300 + dtype)
    x = synth.normal_f32(rows * n_in, 1.0, 31).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_AUTO, tiled=False)
    assert np.max(np.abs(got - want)) <= 2e-5 * (1 + np.max(np.abs(want)))
    with pytest.raises(cuda.UnsupportedError):
        run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA, tiled=False)


def test_tiling_is_a_permutation(dev):
    # every GGUF byte appears exactly once in the tiled copy (rows padded with zeros)
    for dtype, n_out, n_in in ((synth.Q4_K, 40, 512), (synth.Q6_K, 16, 256), (synth.Q8_0, 33, 256), (synth.Q5_K, 16, 512)):
        rb = synth.row_bytes(dtype, n_in)
        raw_h = np.random.default_rng(dtype).integers(1, 256, n_out * rb, dtype=np.uint8)
        stream = dev.stream()
        raw = dev.upload(raw_h)
        nbytes = cuda.tiled_bytes(dtype, n_out, n_in)
        assert nbytes == -(-n_out // 16) * 16 * rb
        tb = dev.alloc(nbytes)
        cuda.tile_weights(stream, tb, raw, dtype, n_out, n_in)
        stream.synchronize()
        t = tb.read(np.uint8, nbytes)
        assert np.array_equal(np.sort(t[t != 0]), np.sort(raw_h))
        assert int((t == 0).sum()) == nbytes - raw_h.size
        raw.free(); tb.free(); stream.destroy()


def test_accumulate_flag_adds_to_output(dev):
    n_out, n_in, rows = 2560, 4096, 9
    w = synth.normal_quant(n_out, n_in, synth.Q4_K, 0.02, 1)
    x = synth.normal_f32(rows * n_in, 1.0, 2).reshape(rows, n_in)
    res = synth.normal_f32(rows * n_out, 1.0, 3).reshape(rows, n_out)
    want = yo.matmul(w, synth.Q4_K, n_out, n_in, x) + res
    for path in (cuda.PATH_MMA, cuda.PATH_FP32):
        got = run_gemm(dev, w, synth.Q4_K, n_out, n_in, x, path, accumulate=res)
        assert np.max(np.abs(got - want)) <= 8e-3


def test_rejections(dev):
    stream = dev.stream()
    b = dev.alloc(1 << 16)
    with pytest.raises(cuda.UnsupportedError):      # row width not a multiple of the block
        cuda.gemm_quant(stream, b, b, b, 100, 8, 1, cuda.Q4_K)
    with pytest.raises(cuda.UnsupportedError):      # no tiled form for F32 weights
        cuda.gemm_quant(stream, b, b, b, 256, 8, 1, cuda.F32, flags=cuda.GEMM_TILED)
    assert cuda.tiled_bytes(cuda.F32, 8, 256) == 0
    with pytest.raises(cuda.YuukaError) as e:       # weight range exceeds the buffer
        cuda.gemm_quant(stream, b, b, b, 2560, 4096, 1, cuda.Q4_K)
    assert e.value.status == cuda.ERR_INVALID_ARGUMENT
    with pytest.raises(cuda.UnsupportedError):      # unknown dtype
        cuda.gemm_quant(stream, b, b, b, 256, 8, 1, 99)
    b.free()
    stream.destroy()
