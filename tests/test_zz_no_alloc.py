"""yuuka_gemm_quant_static (scratch in a fixed device array) against yuuka_gemm_quant, through the C ABI.

Collected last on purpose: it has to pass alone and after every other GPU test
has used the device.
"""
import numpy as np
import pytest

from yuuka_b200 import cuda, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = cuda.Device(0)
    yield d
    d.close()


def tiled_weights(dev, stream, dtype, n_out, n_in, seed):
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, seed)
    raw = dev.alloc(w.nbytes + 256)
    raw.write(w)
    wb = dev.alloc(cuda.tiled_bytes(dtype, n_out, n_in) + 256)
    cuda.tile_weights(stream, wb, raw, dtype, n_out, n_in)
    stream.synchronize()
    raw.free()
    return wb


# (dtype, n_out, n_in, rows, path): split-K across CTAs, no split, fp32 route, rows > 32, and from 48 rows on
# the tensor-memory route: 2560 outputs split K seven ways with the parts summed by a second kernel, 9216
# outputs split it two ways with the sum inside the kernel; both keep their partial sums in the fixed array
SHAPES = [
    (synth.Q6_K, 2560, 9216, 9, cuda.PATH_MMA),
    (synth.Q4_K, 2560, 2560, 9, cuda.PATH_MMA),
    (synth.Q4_K, 9216, 2560, 17, cuda.PATH_AUTO),
    (synth.Q8_0, 528, 2560, 2, cuda.PATH_AUTO),
    (synth.Q5_K, 520, 4096, 40, cuda.PATH_MMA),
    (synth.Q4_K, 2560, 2560, 64, cuda.PATH_MMA),
    (synth.Q6_K, 9216, 2560, 64, cuda.PATH_MMA),
]


@pytest.mark.parametrize("dtype,n_out,n_in,rows,path", SHAPES)
def test_static_scratch_matches_allocating_entry_point(dev, dtype, n_out, n_in, rows, path):
    stream = dev.stream()
    wb = tiled_weights(dev, stream, dtype, n_out, n_in, 300 + dtype)
    results = []
    for call in range(2):  # two calls in a row: the second finds the counters as the first left them
        x = synth.normal_f32(rows * n_in, 1.0, 50 + call).reshape(rows, n_in)
        xb = dev.upload(x)
        want_b = dev.alloc(rows * n_out * 4)
        got_b = dev.alloc(rows * n_out * 4)
        cuda.gemm_quant(stream, want_b, xb, wb, n_in, n_out, rows, dtype, cuda.F32, path, cuda.GEMM_TILED)
        cuda.gemm_quant_static(stream, got_b, xb, wb, n_in, n_out, rows, dtype, cuda.F32, path, cuda.GEMM_TILED)
        stream.synchronize()
        want = want_b.read(np.float32, rows * n_out)
        got = got_b.read(np.float32, rows * n_out)
        assert np.isfinite(want).all() and np.abs(want).max() > 0
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call {call}: results differ"
        results.append(got)
        for b in (xb, want_b, got_b):
            b.free()
    assert not np.array_equal(results[0], results[1])  # the two calls really had different inputs
    wb.free()
    stream.destroy()


def test_calls_after_the_first_leave_free_device_memory_unchanged(dev):
    """What the entry point is for: once the first call on the device has done its set-up, calls allocate
    nothing, whatever shape, type or route arrives next. Every buffer of the test exists before the first
    reading of free memory; the shapes then grow and change kernels (fp32 route, the three register-fed
    tile widths, the tensor-memory route with both kinds of K split), which would make yuuka_gemm_quant grow
    its scratch and, with lazy module loading, make the driver load new kernels."""
    stream = dev.stream()
    cases = [(synth.Q8_0, 528, 2560, 2), (synth.Q4_K, 2560, 2560, 9), (synth.Q6_K, 2560, 9216, 9),
             (synth.Q5_K, 520, 4096, 17), (synth.Q4_K, 9216, 2560, 40), (synth.Q4_K, 2560, 2560, 64),
             (synth.Q6_K, 9216, 2560, 64)]
    bufs = []
    for i, (dtype, n_out, n_in, rows) in enumerate(cases):
        wb = tiled_weights(dev, stream, dtype, n_out, n_in, 500 + i)
        xb = dev.upload(synth.normal_f32(rows * n_in, 1.0, 600 + i))
        ob = dev.alloc(rows * n_out * 4)
        bufs.append((wb, xb, ob))
    # the first call does the set-up
    dtype, n_out, n_in, rows = cases[0]
    cuda.gemm_quant_static(stream, bufs[0][2], bufs[0][1], bufs[0][0], n_in, n_out, rows, dtype, cuda.F32, cuda.PATH_AUTO,
                           cuda.GEMM_TILED)
    stream.synchronize()
    free0, _ = dev.memory()
    for (dtype, n_out, n_in, rows), (wb, xb, ob) in zip(cases, bufs):
        cuda.gemm_quant_static(stream, ob, xb, wb, n_in, n_out, rows, dtype, cuda.F32, cuda.PATH_AUTO, cuda.GEMM_TILED)
        stream.synchronize()
        free, _ = dev.memory()
        assert free == free0, f"{rows} rows x {n_out} x {n_in}: free memory moved by {free0 - free} bytes"
        assert np.isfinite(ob.read(np.float32, rows * n_out)).all()
    for wb, xb, ob in bufs:
        wb.free(); xb.free(); ob.free()
    stream.destroy()


def test_static_scratch_accumulate_and_bf16(dev):
    dtype, n_out, n_in, rows = synth.Q4_K, 2560, 9216, 9
    stream = dev.stream()
    wb = tiled_weights(dev, stream, dtype, n_out, n_in, 77)
    x = synth.normal_f32(rows * n_in, 1.0, 5).reshape(rows, n_in)
    xb = dev.upload(cuda.to_bf16(x))
    base = synth.normal_f32(rows * n_out, 1.0, 6)
    want_b, got_b = dev.upload(base), dev.upload(base)
    flags = cuda.GEMM_TILED | cuda.GEMM_ACCUMULATE
    cuda.gemm_quant(stream, want_b, xb, wb, n_in, n_out, rows, dtype, cuda.BF16, cuda.PATH_MMA, flags)
    cuda.gemm_quant_static(stream, got_b, xb, wb, n_in, n_out, rows, dtype, cuda.BF16, cuda.PATH_MMA, flags)
    stream.synchronize()
    want, got = want_b.read(np.float32, rows * n_out), got_b.read(np.float32, rows * n_out)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert not np.array_equal(got, base)
    for b in (wb, xb, want_b, got_b):
        b.free()
    stream.destroy()


def test_static_scratch_rejects_what_does_not_fit(dev):
    # 576 rows x 9216 columns of prepared activations alone are 11.9 MB > the 8 MiB array
    dtype, n_out, n_in, rows = synth.Q4_K, 32, 9216, 576
    stream = dev.stream()
    wb = dev.alloc(cuda.tiled_bytes(dtype, n_out, n_in) + 256)
    xb = dev.alloc(rows * n_in * 4)
    ob = dev.alloc(rows * n_out * 4)
    with pytest.raises(cuda.YuukaError) as e:
        cuda.gemm_quant_static(stream, ob, xb, wb, n_in, n_out, rows, dtype, cuda.F32, cuda.PATH_MMA, cuda.GEMM_TILED)
    assert e.value.status == 2 and "bytes of scratch" in str(e.value)
    # GGUF-layout weights are not accepted either
    with pytest.raises(cuda.YuukaError) as e:
        cuda.gemm_quant_static(stream, ob, xb, wb, n_in, n_out, 4, dtype, cuda.F32, cuda.PATH_AUTO, 0)
    assert e.value.status == 1
    for b in (wb, xb, ob):
        b.free()
    stream.destroy()
