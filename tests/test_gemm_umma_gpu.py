"""Large-M route of the quantized GEMM (tcgen05 tensor cores, accumulator in tensor memory) against
the CPU oracle (tensor/quant.go matmul), through the C ABI. It takes over from 48 rows."""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda, synth

from .test_gemm_gpu import run_gemm, stats

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = cuda.Device(0)
    yield d
    d.close()


@pytest.mark.parametrize("dtype", [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.Q5_K])
@pytest.mark.parametrize("rows", [48, 64, 100, 256, 272, 300, 512, 600])
def test_umma_route_matches_oracle(dev, dtype, rows):
    n_out, n_in = 520, 512   # five blocks of 128 weight rows, the last one partial; two superblocks
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, 300 + dtype)
    x = synth.normal_f32(rows * n_in, 1.0, 40 + rows).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    err, cos = stats(got, want)
    # fp16 operands, fp32 accumulate; outputs have std ~0.45 at 512 columns
    assert err <= 4e-3 and cos >= 0.999999, (err, cos)


@pytest.mark.parametrize("n_out,n_in,dtype,rows", [
    (9216, 2560, synth.Q4_K, 160), (2560, 9216, synth.Q6_K, 160), (18432, 2560, synth.Q4_K, 512), (4096, 256, synth.Q8_0, 64),
])
def test_umma_route_model_shapes_and_determinism(dev, n_out, n_in, dtype, rows):
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, n_out + n_in)
    x = synth.normal_f32(rows * n_in, 1.0, 4).reshape(rows, n_in)
    want = yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    err, cos = stats(got, want)
    assert err <= 1e-2 and cos >= 0.999999, (err, cos)
    again = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA)
    assert np.array_equal(got, again)


def test_umma_route_accumulates(dev):
    n_out, n_in, rows, dtype = 640, 768, 80, synth.Q4_K
    w = synth.normal_quant(n_out, n_in, dtype, 0.02, 9)
    x = synth.normal_f32(rows * n_in, 1.0, 10).reshape(rows, n_in)
    base = synth.normal_f32(rows * n_out, 1.0, 11).reshape(rows, n_out)
    want = base + yo.matmul(w, dtype, n_out, n_in, x)
    got = run_gemm(dev, w, dtype, n_out, n_in, x, cuda.PATH_MMA, accumulate=base)
    err, cos = stats(got, want)
    assert err <= 4e-3 and cos >= 0.999999, (err, cos)
