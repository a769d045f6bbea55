"""The scoring path's fused causal attention against a float64 restatement of what the reference
computes with three dispatches (scores, row softmax, probabilities x V:
ferrum_wgpu/src/ops/llama.rs:L119-L146; CPU semantics ferrum_ref/src/kernels/attention.rs). Every
kernel variant must agree: mma.sync with one or two row tiles per warp, and the tcgen05 kernel with
tensor-memory accumulators. Inputs are fp16 by contract, so the restatement starts from the same
rounded values; what remains is the fp16 rounding of the probabilities and of the result.
Tolerance: 4e-3 absolute on outputs of magnitude <= ~1 (fp16 has 11 significant bits)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ATOL = 4e-3


def _reference(qkv, n_seqs, t, heads, kv_heads):
    x = qkv.astype(np.float64).reshape(n_seqs, t, heads + 2 * kv_heads, 64)
    q, k, v = x[:, :, :heads], x[:, :, heads:heads + kv_heads], x[:, :, heads + kv_heads:]
    out = np.empty((n_seqs, t, heads, 64))
    mask = np.triu(np.ones((t, t), dtype=bool), 1)
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = np.einsum("bid,bjd->bij", q[:, :, h], k[:, :, g]) / 8.0
        s[:, mask] = -np.inf
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, :, h] = np.einsum("bij,bjd->bid", p, v[:, :, g])
    return out.reshape(n_seqs * t, heads * 64)


def _problem(seed, n_seqs, t, heads, kv_heads, scale=1.0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n_seqs * t, (heads + 2 * kv_heads) * 64)) * scale).astype(np.float16)


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("t", [1, 17, 64, 65, 128, 129, 200, 256, 257, 383, 640, 1024])
def test_variants_match_the_float64_restatement(dev, variant, t):
    n_seqs, heads, kv_heads = 3, 4, 2
    qkv = _problem(t, n_seqs, t, heads, kv_heads)
    want = _reference(qkv, n_seqs, t, heads, kv_heads)
    got, _ = dev.attention_f16(qkv, n_seqs, t, heads, kv_heads, variant=variant)
    err = np.abs(got.astype(np.float64) - want).max()
    assert err < ATOL, (variant, t, err)


@pytest.mark.parametrize("heads,kv_heads", [(1, 1), (3, 1), (2, 2), (12, 4), (16, 2)])
def test_head_groupings(dev, heads, kv_heads):
    n_seqs, t = 2, 300
    qkv = _problem(7, n_seqs, t, heads, kv_heads)
    want = _reference(qkv, n_seqs, t, heads, kv_heads)
    for variant in (1, 3):
        got, _ = dev.attention_f16(qkv, n_seqs, t, heads, kv_heads, variant=variant)
        err = np.abs(got.astype(np.float64) - want).max()
        assert err < ATOL, (variant, heads, kv_heads, err)


def test_sharp_softmax_and_the_default_choice(dev):
    # large scores: the row maximum moves between key tiles, so the running rescale is exercised
    n_seqs, t, heads, kv_heads = 2, 520, 2, 1
    qkv = _problem(11, n_seqs, t, heads, kv_heads, scale=3.0)
    want = _reference(qkv, n_seqs, t, heads, kv_heads)
    for variant in (0, 1, 3):
        got, _ = dev.attention_f16(qkv, n_seqs, t, heads, kv_heads, variant=variant)
        err = np.abs(got.astype(np.float64) - want).max()
        assert err < 3 * ATOL, (variant, err)  # |v| up to ~12 here


def test_first_row_copies_v_and_rows_do_not_leak_across_sequences(dev):
    n_seqs, t, heads, kv_heads = 4, 130, 2, 1
    qkv = _problem(13, n_seqs, t, heads, kv_heads)
    got, _ = dev.attention_f16(qkv, n_seqs, t, heads, kv_heads, variant=3)
    x = qkv.reshape(n_seqs, t, heads + 2 * kv_heads, 64)
    for s in range(n_seqs):
        for h in range(heads):
            # position 0 attends to itself only: the result is exactly its v row
            np.testing.assert_array_equal(got.reshape(n_seqs, t, heads, 64)[s, 0, h], x[s, 0, heads + kv_heads])
