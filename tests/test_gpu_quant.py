"""Parity of the device codec and the quantised products against the CPU oracle, through the C ABI.
Mirrors ferrum_wgpu/src/ops/quant/tests.rs."""
import numpy as np
import pytest

from ferrum_gpu_b200 import CudaError, Mode, QKind, linear_q, upload_quantised, upload_qweight
from ferrum_gpu_b200 import _ffi
from oracle import oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu

KINDS = [QKind.Q8_0, QKind.Q4_0]
FP8 = [QKind.FP8_E4M3, QKind.FP8_E5M2]  # one-byte floats in Q8_0's block (ops/quant.rs:L38-L41)
MX = [QKind.MXFP4]  # E2M1 nibbles with a power-of-two scale byte (ops/quant.rs:L36-L37)
STORED = KINDS + [QKind.F16] + FP8 + MX  # F16: plain f16 values, no scale (ops/quant.rs:L33-L36)
# device bytes per 32 elements (MXFP4: 17 in a file, 18 on the device, where the scale takes a 16-bit slot)
BLOCK_BYTES = {QKind.Q8_0: 34, QKind.Q4_0: 18, QKind.F16: 64, QKind.FP8_E4M3: 34, QKind.FP8_E5M2: 34, QKind.MXFP4: 18}
REDUCING = 1e-5  # ferrum_wgpu/src/tolerance.rs:L7


@pytest.mark.parametrize("kind", STORED)
@pytest.mark.parametrize("k,n", [(32, 1), (32, 5), (64, 3), (96, 65), (128, 64), (768, 130)])
def test_device_encoder_is_bit_identical_to_the_cpu_encoder(dev, kind, k, n):
    for w in (helpers.nasty(k * n), orc.rand_vec(k * n, 4) * np.float32(0.02)):
        qw = upload_quantised(dev, kind, w, k, n)
        assert np.array_equal(qw.blocks(), orc.quantise_matrix(int(kind), w, k, n)), (kind, k, n)
        assert (qw.kind(), qw.k(), qw.n()) == (kind, k, n)
        assert qw.device_bytes() == k * n * BLOCK_BYTES[kind] // 32
        qw.close()


@pytest.mark.parametrize("kind", STORED)
@pytest.mark.parametrize("k,n", [(32, 1), (32, 5), (64, 3), (96, 65), (128, 64)])
def test_dequantised_values_are_bit_identical_to_the_cpu_decode(dev, kind, k, n):
    """ops/quant/tests.rs:L106-L131, both by the decode kernel and by the identity-matrix read-back."""
    raw = orc.quantise_matrix(int(kind), helpers.nasty(k * n), k, n)
    rows = orc.decode(int(kind), raw, k * n).reshape(n, k)
    qw = upload_qweight(dev, kind, raw, k, n)
    assert np.array_equal(qw.blocks(), raw)
    assert np.array_equal(qw.dequantised().view(np.uint32), rows.view(np.uint32))
    eye = np.eye(k, dtype=np.float32)
    got = linear_q(dev, eye, qw, k)  # y[r, col] = W[col, r]
    assert np.array_equal(got, rows.T), (kind, k, n)
    qw.close()


@pytest.mark.parametrize("kind", STORED + [QKind.F32])
@pytest.mark.parametrize("rows,k,n", [(1, 32, 1), (1, 256, 100), (7, 96, 13), (33, 64, 65), (2, 512, 3),
                                      (8, 2048, 37), (5, 2816, 70), (64, 1024, 200), (130, 768, 257)])
def test_linear_matches_the_cpu_matmul_on_the_dequantised_weights(dev, kind, rows, k, n):
    """ops/quant/tests.rs:L133-L157 and L271-L304 (every kernel x precision x awkward shapes). The
    reference's shapes (k <= 512) use its unscaled uniform weights; the wider ones added here scale the
    weights by 1/sqrt(k) so the outputs stay O(1): with O(15) outputs the serial f32 sum of the oracle is
    itself 3e-5 off, which measures the oracle, not the kernel."""
    w = orc.rand_vec(k * n, 4)
    if k > 512:
        w = w * np.float32(1.0 / np.sqrt(k))
    want_w = orc.snap_matrix(int(kind), w, k, n)
    x = orc.rand_vec(rows * k, 5)
    want = orc.matmul(x, want_w, rows, k, n)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, rows)
    e = orc.max_rel_err(got, want)
    assert e < REDUCING, (kind, rows, k, n, e)
    again = linear_q(dev, x, qw, rows)
    assert np.array_equal(got, again), "a repeated run is bit-identical"
    qw.close()


def test_f32_weight_with_a_width_that_is_not_whole_blocks(dev):
    """An ineligible width stays f32 (ferrum_wgpu/src/models/llama/lin.rs:L54-L61)."""
    for rows, k, n in [(1, 24, 9), (3, 24, 40), (20, 50, 7)]:
        w, x = orc.rand_vec(k * n, 6), orc.rand_vec(rows * k, 7)
        qw = upload_quantised(dev, QKind.F32, w, k, n)
        assert orc.max_rel_err(linear_q(dev, x, qw, rows), orc.matmul(x, w, rows, k, n)) < REDUCING
        qw.close()


def test_pack_and_quantise_refuse_bad_shapes(dev):
    """ops/quant/tests.rs:L73-L87, L200-L215"""
    for kind in KINDS:
        with pytest.raises(CudaError) as e:
            upload_qweight(dev, kind, np.zeros(100, dtype=np.uint8), 33, 1)
        assert "whole" in str(e.value) and e.value.code == _ffi.FC_ERR_SHAPE
        with pytest.raises(CudaError) as e:
            upload_qweight(dev, kind, np.zeros(3, dtype=np.uint8), 32, 1)
        assert "needs" in str(e.value)
        with pytest.raises(CudaError):
            upload_quantised(dev, kind, np.zeros(33, dtype=np.float32), 33, 1)
        with pytest.raises(CudaError):
            upload_quantised(dev, kind, np.zeros(63, dtype=np.float32), 32, 2)
    qw = upload_quantised(dev, QKind.Q8_0, orc.rand_vec(64 * 4, 1), 64, 4)
    with pytest.raises(CudaError):
        linear_q(dev, np.zeros(65, dtype=np.float32), qw, 1)
    qw.close()


@pytest.mark.parametrize("kind", KINDS)
def test_sweep_shapes_of_the_isolated_matmul_config(dev, kind):
    """The decode-side rows of the isolated sweep (M in {1, 8, 64}) on its K, N corners, against
    the oracle at 1e-5 with N(0,1) activations and N(0,0.02) weights."""
    rng = np.random.default_rng(11)
    for k, n in [(768, 768), (2048, 2816), (4096, 768)]:
        w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        want_w = orc.snap_matrix(int(kind), w, k, n)
        qw = upload_quantised(dev, kind, w, k, n)
        for m in (1, 8, 64):
            x = rng.standard_normal(m * k, dtype=np.float32)
            e = orc.max_rel_err(linear_q(dev, x, qw, m), orc.matmul(x, want_w, m, k, n, threads=8))
            assert e < REDUCING, (kind, m, k, n, e)
        qw.close()


@pytest.mark.parametrize("kind", KINDS + FP8 + MX + [QKind.F16])
@pytest.mark.parametrize("rows,k,n", [(9, 128, 8), (16, 256, 70), (33, 1024, 200), (64, 2816, 130), (40, 384, 1536)])
def test_batched_decode_tensor_product_keeps_f32_accuracy(dev, kind, rows, k, n):
    """9..64 rows (concurrent decode streams) run on mma.sync with x split into two fp16 terms and the
    block scale applied in f32: the result must stay within the f32 bound of the oracle, be exact on
    the identity (bit-identical dequantisation), and repeat bit for bit (split-K without atomics)."""
    w = orc.rand_vec(k * n, 4) * np.float32(1.0 / np.sqrt(k))
    want_w = orc.snap_matrix(int(kind), w, k, n)
    x = orc.rand_vec(rows * k, 5)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, rows)
    assert orc.max_rel_err(got, orc.matmul(x, want_w, rows, k, n)) < REDUCING, (kind, rows, k, n)
    assert np.array_equal(got, linear_q(dev, x, qw, rows))
    if rows * 2 <= k:  # one-hot rows read weight columns back exactly
        eye = np.zeros((rows, k), dtype=np.float32)
        eye[np.arange(rows), np.arange(rows) * 2] = 1.0
        cols = linear_q(dev, eye, qw, rows)
        assert np.array_equal(cols, want_w.reshape(k, n)[np.arange(rows) * 2])
    qw.close()


# ---- Q2_K: super-blocks of 256 with 4-bit sub-block scales and mins (ops/quant.rs:L42-L43) -------------

def _q2k_inputs(k, n):
    i = np.arange(k * n)
    wave = (np.sin(i.astype(np.float32) * np.float32(0.37), dtype=np.float32) * np.float32(0.8)
            + ((i * 7 % 13).astype(np.float32) - np.float32(6.0)) * np.float32(0.02)).astype(np.float32)
    return [helpers.nasty(k * n), orc.rand_vec(k * n, 4) * np.float32(0.02), wave,
            np.abs(orc.rand_vec(k * n, 6)), -np.abs(orc.rand_vec(k * n, 7))]


@pytest.mark.parametrize("k,n", [(256, 1), (256, 5), (512, 3), (768, 130), (1024, 64)])
def test_q2k_device_encoder_and_decoder_are_bit_identical_to_the_cpu_codec(dev, k, n):
    """The 16-candidate scale search of `fit` (ferrum_gguf/src/codec/q2k.rs:L25-L88) decides on exact ties of
    an f32 error sum, so the device encoder repeats the reference's operations one rounding at a time."""
    for w in _q2k_inputs(k, n):
        raw = orc.quantise_matrix(int(QKind.Q2_K), w, k, n)
        qw = upload_quantised(dev, QKind.Q2_K, w, k, n)
        assert (qw.kind(), qw.k(), qw.n()) == (QKind.Q2_K, k, n)
        assert qw.device_bytes() == k * n * 84 // 256
        assert np.array_equal(qw.blocks(), raw), (k, n)
        rows = orc.decode(int(QKind.Q2_K), raw, k * n).reshape(n, k)
        assert np.array_equal(qw.dequantised().view(np.uint32), rows.view(np.uint32))
        qw.close()
        qb = upload_qweight(dev, QKind.Q2_K, raw, k, n)  # the file-block upload and its inverse
        assert np.array_equal(qb.blocks(), raw)
        assert np.array_equal(qb.dequantised().view(np.uint32), rows.view(np.uint32))
        if k == 256:
            got = linear_q(dev, np.eye(k, dtype=np.float32), qb, k)  # y[r, col] = W[col, r]
            assert np.array_equal(got, rows.T)
        qb.close()


def test_q2k_on_a_width_of_whole_32s_only_is_stored_as_q4_0(dev):
    """`effective` (ops/quant.rs:L134-L144)."""
    k, n = 96, 7
    w = orc.rand_vec(k * n, 4)
    qw = upload_quantised(dev, QKind.Q2_K, w, k, n)
    assert qw.kind() == QKind.Q4_0
    assert np.array_equal(qw.blocks(), orc.quantise_matrix(int(QKind.Q4_0), w, k, n))
    qw.close()
    with pytest.raises(CudaError):
        upload_qweight(dev, QKind.Q2_K, np.zeros(84, np.uint8), 96, 1)


@pytest.mark.parametrize("rows,k,n", [(1, 256, 100), (7, 512, 13), (8, 2816, 70), (33, 1024, 200), (64, 768, 130),
                                      (130, 768, 257)])
def test_q2k_linear_matches_the_cpu_matmul_on_the_dequantised_weights(dev, rows, k, n):
    w = orc.rand_vec(k * n, 4) * np.float32(1.0 / np.sqrt(k))
    want_w = orc.snap_matrix(int(QKind.Q2_K), w, k, n)
    x = orc.rand_vec(rows * k, 5)
    want = orc.matmul(x, want_w, rows, k, n)
    qw = upload_quantised(dev, QKind.Q2_K, w, k, n)
    got = linear_q(dev, x, qw, rows)
    assert orc.max_rel_err(got, want) < REDUCING, (rows, k, n)
    assert np.array_equal(got, linear_q(dev, x, qw, rows))
    qw.close()


@pytest.mark.parametrize("kind", STORED + [QKind.Q2_K])
def test_device_encoder_matches_the_cpu_encoder_on_special_values(dev, kind):
    """NaN, infinities, signed zeros, subnormals and values past the f16 range inside otherwise ordinary
    blocks: the device encoder takes the same branches as the CPU one (`f32::max` ignores NaN, `as i8` sends
    NaN to 0, an infinite scale makes every code NaN, ...)."""
    k, n = 512, 6
    w = (orc.rand_vec(k * n, 12) * np.float32(0.5)).reshape(k, n)
    if kind != QKind.Q2_K:
        # (Q2_K's `nearest_int` reads the low bits of `x + 12582912.0`: for a NaN that is the payload, which an x86
        # host and the GPU choose differently - the reference's own answer depends on the machine there)
        w[3, 0] = np.nan
        w[40, 1] = np.inf
        w[77, 2] = -np.inf
        w[288:320, 0] = np.nan          # an all-NaN block
        w[300, 5] = np.float32(3.0e38)  # (Q2_K: a super-block scale past the f16 range is infinite, and inf * 0 a NaN)
    w[100, 3] = -0.0
    w[130:140, 4] = np.float32(1e-41)   # subnormal f32
    w[301, 5] = np.float32(-7.0e4)      # past the f16 range
    w[256:288, 0] = 0.0                 # an all-zero block
    w = w.reshape(-1)
    raw = orc.quantise_matrix(int(kind), w, k, n)
    qw = upload_quantised(dev, kind, w, k, n)
    assert np.array_equal(qw.blocks(), raw), kind
    want = orc.decode(int(kind), raw, k * n)
    got = qw.dequantised().reshape(-1)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32)), kind
    qw.close()


def test_a_given_up_wait_is_reported_by_the_next_synchronisation(dev):
    """The device-pointer products return before their kernels run; a kernel that gives up a bounded wait raises
    a status word, and fc_device_sync is where the caller learns of it. The word is raised from the host here: no
    kernel has to time out."""
    lib = _ffi.load()
    assert lib.fc_device_sync(dev.handle) == _ffi.FC_OK
    dev.check(lib.fc_debug_raise_status(dev.handle, 3))
    assert lib.fc_device_sync(dev.handle) == _ffi.FC_ERR_TIMEOUT
    assert b"bounded wait" in lib.fc_last_error(dev.handle)
    assert lib.fc_device_sync(dev.handle) == _ffi.FC_OK, "the status is cleared once reported"
