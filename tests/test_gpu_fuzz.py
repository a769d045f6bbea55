"""Seeded shape fuzz of the two products whose kernels divide their work in ways that depend on the shape: the
streamed one-row product (every warp takes an equal share of the CTA's (tile, K stage) units, tiles that are cut
are summed by the last arriver) and the tensor-core product (128 x 192 tiles clipped by the tensor maps at both
matrix edges, results leaving through TMA stores). Same contract as the fixed-shape tests: the one-row product
within 1e-5 of exact (float64) arithmetic over the dequantised weights with the reference's metric
|g - w| / max(|w|, 1) (ferrum_wgpu/src/ops/quant/tests.rs:L133-L176 holds 1e-5 against the oracle), the tensor-core
product within the 2e-2 per-value bound of that path; a second run of every case must reproduce the first bit for bit."""
import numpy as np
import pytest

from ferrum_gpu_b200 import Mode, QKind, linear_q, upload_quantised
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _cases(seed, count, ks, n_max, m_max):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        out.append((int(rng.integers(1, m_max + 1)), int(rng.choice(ks)), int(rng.integers(1, n_max + 1)),
                    [QKind.Q8_0, QKind.Q4_0][int(rng.integers(0, 2))], int(rng.integers(0, 1 << 30))))
    return out


@pytest.mark.parametrize("m,k,n,kind,seed", _cases(11, 24, [256, 512, 768, 1024, 2048, 4096], 5000, 1))
def test_one_row_product_on_random_shapes(dev, m, k, n, kind, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    x = rng.standard_normal(k, dtype=np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, 1)
    want = x.astype(np.float64) @ orc.snap_matrix(int(kind), w, k, n).astype(np.float64).reshape(k, n)
    err = np.abs(got.reshape(-1) - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() < 1e-5, (k, n, kind, err.max())
    assert np.array_equal(got, linear_q(dev, x, qw, 1)), "the same launch twice gives the same bits"
    qw.close()


@pytest.mark.parametrize("m,k,n,kind,seed", _cases(12, 16, [64, 192, 320, 768, 1024, 2048], 1500, 900))
def test_tensor_product_on_random_shapes(dev, m, k, n, kind, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal(m * k, dtype=np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, m, Mode.TENSOR_F16)
    want = orc.matmul(x, orc.snap_matrix(int(kind), w, k, n), m, k, n, threads=8).reshape(m, n)
    err = np.abs(got - want).max()
    assert err < 2e-2 and err < 0.02 * max(np.abs(want).max(), 1.0), (m, k, n, kind, err)
    assert np.array_equal(got, linear_q(dev, x, qw, m, Mode.TENSOR_F16))
    qw.close()


@pytest.mark.parametrize("kind", [QKind.Q8_0, QKind.Q4_0])
@pytest.mark.parametrize("m,k,n", [(9, 512, 9600), (12, 1024, 16000), (17, 768, 12000), (33, 4096, 11008), (64, 1024, 20000),
                                   (64, 2048, 9473), (64, 1024, 5632), (40, 4096, 4800)])
def test_long_output_products_of_a_few_rows_keep_f32_accuracy(dev, kind, m, k, n):
    """Outputs long enough to fill the device take the tcgen05 form of the batched-decode product (weights and x both
    as two fp16 terms, products exact in the f32 accumulator, 256 k at a time): same 1e-5 bound as every exact-path
    product, and the same distance from exact arithmetic whatever the size of a row's scales (a row is normalised by
    a power of two); bit-reproducible."""
    rng = np.random.default_rng(m * 1000 + k + n)
    w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    w.reshape(k, n)[:, : n // 3] *= np.float32(1e-4)   # a third of the rows with tiny scales
    w.reshape(k, n)[:, -7:] *= np.float32(300.0)       # and a few large ones
    x = rng.standard_normal(m * k, dtype=np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, m)
    wd = orc.snap_matrix(int(kind), w, k, n).astype(np.float64).reshape(k, n)
    want = x.astype(np.float64).reshape(m, k) @ wd
    mag = np.abs(x.astype(np.float64).reshape(m, k)) @ np.abs(wd)
    e_abs = np.abs(got.reshape(m, n) - want)
    # every row, whatever its scales: a few f32 roundings of the sum of magnitudes (the mma.sync product of the same
    # rows measures 4e-8 .. 8e-8 here); the rows of ordinary size: the reference's own metric
    assert (e_abs / (mag + 1e-300)).max() < 3e-7, (m, k, n, kind, (e_abs / (mag + 1e-300)).max())
    mid = slice(n // 3, n - 7)
    assert (e_abs[:, mid] / np.maximum(np.abs(want[:, mid]), 1.0)).max() < 1e-5, (m, k, n, kind)
    assert np.array_equal(got, linear_q(dev, x, qw, m))
    qw.close()
