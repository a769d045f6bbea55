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
