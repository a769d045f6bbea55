"""Pins the CPU oracle against every known-answer test the reference holds for the hot path.

Each test names the reference test it restates (file:line). CPU only.
"""
import math

import numpy as np
import pytest

from ferrum_gpu_b200._ffi import FC_Q4_0, FC_Q8_0, FC_ROPE_NEOX, FC_ROPE_NORM
from oracle import oracle as orc
from tests import helpers

KINDS = [FC_Q8_0, FC_Q4_0]


def data(n):
    """ferrum_gguf/src/codec/quant.rs:L185-L189"""
    return np.array([np.float32(np.float32(i * 37 % 101) - np.float32(50.0)) / np.float32(13.0)
                     for i in range(n)], dtype=np.float32)


# ---- f16 (ferrum_gguf/src/codec/f16.rs:L59-L95) ---------------------------------------------

def test_f16_known_values():
    assert orc.f16_to_f32(0x3C00) == 1.0
    assert orc.f16_to_f32(0xC000) == -2.0
    assert orc.f16_to_f32(0x0000) == 0.0
    assert orc.f16_to_f32(0x7BFF) == 65504.0
    assert orc.f16_to_f32(0x0001) == 2.0 ** -24
    assert math.isinf(orc.f16_to_f32(0x7C00))
    assert math.isnan(orc.f16_to_f32(0x7E00))
    assert orc.f32_to_f16(1.0) == 0x3C00
    assert orc.f32_to_f16(-2.0) == 0xC000
    assert orc.f32_to_f16(65504.0) == 0x7BFF
    assert orc.f32_to_f16(1e9) == 0x7C00
    assert orc.f32_to_f16(1e-30) == 0
    assert math.isnan(orc.f16_to_f32(orc.f32_to_f16(float("nan"))))


def test_every_half_round_trips_exactly_and_matches_numpy():
    allh = np.arange(65536, dtype=np.uint16)
    want = allh.view(np.float16).astype(np.float32)
    for h in range(65536):
        x = orc.f16_to_f32(h)
        if math.isnan(x):
            assert np.isnan(want[h])
            continue
        assert x == want[h]
        assert orc.f32_to_f16(x) == h, hex(h)


def test_f16_rounding_is_to_nearest_even():
    assert orc.f32_to_f16(1.0 + 2.0 ** -11) == 0x3C00
    assert orc.f32_to_f16(1.0 + 3.0 * 2.0 ** -11) == 0x3C02
    assert orc.f32_to_f16(1.0 + 2.0 ** -11 + 2.0 ** -20) == 0x3C01
    # independent check of RNE against numpy on random floats spanning normal/subnormal halves
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(4000) * 10.0 ** rng.uniform(-9, 5, 4000)).astype(np.float32)
    for x in xs:
        assert orc.f32_to_f16(float(x)) == int(np.float32(x).astype(np.float16).view(np.uint16))


# ---- block codec (ferrum_gguf/src/codec/quant.rs:L193-L287) ----------------------------------

def test_sizes():
    assert orc.block_bytes(FC_Q8_0, 64) == 68
    assert orc.block_bytes(FC_Q4_0, 64) == 36
    assert orc.block_bytes(FC_Q8_0, 33) == 0
    assert orc.block_bytes(FC_Q4_0, 31) == 0
    with pytest.raises(ValueError):
        orc.encode(FC_Q8_0, np.ones(5, dtype=np.float32))


def test_q8_0_error_is_within_half_a_step_of_the_block_scale():
    d = data(96)
    back = orc.decode(FC_Q8_0, orc.encode(FC_Q8_0, d), 96)
    for blk, got in zip(d.reshape(-1, 32), back.reshape(-1, 32)):
        step = np.abs(blk).max() / 127.0
        assert np.all(np.abs(blk - got) <= step * 0.51 + 1e-4)


def test_q8_0_known_block():
    blk = np.zeros(32, dtype=np.float32)
    blk[0], blk[1] = 127.0, -63.5
    b = orc.encode(FC_Q8_0, blk)
    assert orc.f16_to_f32(int(b[0]) | int(b[1]) << 8) == 1.0
    assert np.int8(b[2]) == 127
    assert b[3:4].view(np.int8)[0] == -64  # -63.5 rounds away from zero
    assert orc.decode(FC_Q8_0, b, 32)[0] == 127.0


def test_q4_0_is_coarse_but_bounded_and_idempotent():
    d = data(64)
    once = orc.decode(FC_Q4_0, orc.encode(FC_Q4_0, d), 64)
    for blk, got in zip(d.reshape(-1, 32), once.reshape(-1, 32)):
        amax = np.abs(blk).max()
        assert np.all(np.abs(blk - got) <= amax / 8.0 * 1.01 + 1e-4)
    twice = orc.decode(FC_Q4_0, orc.encode(FC_Q4_0, once), 64)
    assert np.array_equal(once, twice)


def test_q4_0_nibble_order_is_low_half_first():
    blk = np.zeros(32, dtype=np.float32)
    blk[0], blk[16] = -8.0, 7.0
    back = orc.decode(FC_Q4_0, orc.encode(FC_Q4_0, blk), 32)
    assert back[0] == -8.0 and back[16] == 7.0 and back[1] == 0.0


def test_zero_blocks_and_length_mismatches():
    z = np.zeros(32, dtype=np.float32)
    for kind in KINDS:
        assert np.array_equal(orc.decode(kind, orc.encode(kind, z), 32), z)
    with pytest.raises(ValueError):
        orc.decode(FC_Q8_0, np.zeros(7, dtype=np.uint8), 32)


def test_q4_0_ties_keep_the_first_largest_magnitude():
    # +3 before -3: the fold keeps the first, d = 3 / -8 (negative), so +3 -> q = 0
    blk = np.zeros(32, dtype=np.float32)
    blk[2], blk[5] = 3.0, -3.0
    b = orc.encode(FC_Q4_0, blk)
    d = orc.f16_to_f32(int(b[0]) | int(b[1]) << 8)
    assert d == np.float32(3.0) / np.float32(-8.0)
    dec = orc.decode(FC_Q4_0, b, 32)
    assert dec[2] == 3.0 and dec[5] == np.float32(-3.0 / 8.0 * 7.0)


def test_encoders_match_an_independent_numpy_restatement():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(32 * 40).astype(np.float32) * np.float32(0.02),
                        helpers.nasty(32 * 14)])
    blocks = x.reshape(-1, 32)
    # Q8_0
    amax = np.abs(blocks).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, 1), np.float32(0)).astype(np.float32)
    t = (blocks * inv[:, None]).astype(np.float32)
    q = np.clip(np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), -128, 127).astype(np.int8)
    got = orc.encode(FC_Q8_0, x).reshape(-1, 34)
    assert np.array_equal(got[:, :2].copy().view(np.uint16)[:, 0], d.astype(np.float16).view(np.uint16))
    assert np.array_equal(got[:, 2:].view(np.int8), q)
    # Q4_0
    idx = np.abs(blocks).argmax(axis=1)  # first maximum
    mx = blocks[np.arange(len(blocks)), idx]
    d4 = (mx / np.float32(-8.0)).astype(np.float32)
    inv4 = np.where(d4 != 0, np.float32(1.0) / np.where(d4 != 0, d4, 1), np.float32(0)).astype(np.float32)
    t4 = ((blocks * inv4[:, None]).astype(np.float32) + np.float32(8.5)).astype(np.float32)
    q4 = np.clip(np.trunc(t4), 0, 15).astype(np.uint8)
    want = q4[:, :16] | (q4[:, 16:] << 4)
    got4 = orc.encode(FC_Q4_0, x).reshape(-1, 18)
    assert np.array_equal(got4[:, :2].copy().view(np.uint16)[:, 0], d4.astype(np.float16).view(np.uint16))
    assert np.array_equal(got4[:, 2:], want)


# ---- reference device layout + requantise identity (ferrum_wgpu/src/ops/quant/tests.rs) -------

def test_pack_reorders_blocks_column_major_and_widens_the_scale():
    """ops/quant/tests.rs:L44-L71"""
    k, n = 64, 2
    raw = bytearray()
    for blk in range(4):
        h = orc.f32_to_f16(float(blk) + 1.0)
        raw += bytes([h & 0xFF, h >> 8]) + bytes((i + blk * 40) & 0xFF for i in range(32))
    w = orc.pack_reference_layout(FC_Q8_0, np.frombuffer(bytes(raw), dtype=np.uint8), k, n)
    assert w.size == 2 * 2 * 9
    for b, col, file_blk in [(0, 0, 0), (1, 0, 1), (0, 1, 2), (1, 1, 3)]:
        rec = w[(b * n + col) * 9:][:9]
        assert rec[:1].view(np.float32)[0] == float(file_blk) + 1.0
        first = int.from_bytes(bytes((i + file_blk * 40) & 0xFF for i in range(4)), "little")
        assert rec[1] == first
    h = orc.f32_to_f16(0.5)
    q4 = np.frombuffer(bytes([h & 0xFF, h >> 8]) + bytes(range(16)), dtype=np.uint8)
    w = orc.pack_reference_layout(FC_Q4_0, q4, 32, 1)
    assert w.size == 5 and w[:1].view(np.float32)[0] == 0.5
    assert w[4] == int.from_bytes(bytes([12, 13, 14, 15]), "little")


def test_requantising_dequantised_weights_reproduces_the_values():
    """ops/quant/tests.rs:L89-L104"""
    for kind in KINDS:
        for k, n in [(32, 1), (64, 7), (96, 40), (256, 9)]:
            w = helpers.nasty(k * n)
            rows = orc.decode(kind, orc.quantise_matrix(kind, w, k, n), k * n)  # [n, k]
            again = orc.quantise_matrix(kind, orc.transpose(rows, n, k), k, n)
            assert np.array_equal(orc.decode(kind, again, k * n), rows), (kind, k, n)


def test_quantise_refuses_bad_shapes():
    """ops/quant/tests.rs:L73-L87"""
    for kind in KINDS:
        with pytest.raises(ValueError):
            orc.quantise_matrix(kind, np.zeros(33, dtype=np.float32), 33, 1)
        with pytest.raises(ValueError):
            orc.quantise_matrix(kind, np.zeros(63, dtype=np.float32), 32, 2)


# ---- matmul (ferrum_ref/src/kernels/matmul.rs:L113-L179) --------------------------------------

def test_matmul_known_values():
    got = orc.matmul([1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 3, 2)
    assert got.tolist() == [58.0, 64.0, 139.0, 154.0]


def test_matmul_non_square_and_one_row():
    a, b = orc.rand_vec(7, 1), orc.rand_vec(35, 2)
    got = orc.matmul(a, b, 1, 7, 5)
    for j in range(5):
        want = np.float32(0)
        for p in range(7):
            want = np.float32(want + np.float32(a[p] * b[p * 5 + j]))
        assert got[j] == want  # same order, same roundings


def test_matmul_shape_errors_name_the_operand():
    with pytest.raises(ValueError, match="operand a has 1 elements, shape needs 2"):
        orc.matmul([1.0], [1.0, 2.0], 2, 1, 1)
    with pytest.raises(ValueError, match="operand b"):
        orc.matmul([1.0], [1.0, 2.0], 1, 1, 1)


def test_matmul_empty_and_threaded_bit_identical():
    assert orc.matmul([], [], 2, 0, 2).tolist() == [0.0] * 4
    m, k, n = 13, 9, 11
    a, b = orc.rand_vec(m * k, 3), orc.rand_vec(k * n, 4)
    want = orc.matmul(a, b, m, k, n)
    for t in [0, 1, 2, 5, 64]:
        assert np.array_equal(orc.matmul(a, b, m, k, n, threads=t), want)


def test_rand_vec_is_deterministic_and_in_range():
    assert np.array_equal(orc.rand_vec(8, 7), orc.rand_vec(8, 7))
    assert not np.array_equal(orc.rand_vec(8, 7), orc.rand_vec(8, 8))
    v = orc.rand_vec(1000, 9)
    assert np.all((v >= -1.0) & (v < 1.0))
    # xorshift64 by hand for the first value of seed 7
    s = 7
    s ^= (s << 13) & (2 ** 64 - 1)
    s ^= s >> 7
    s ^= (s << 17) & (2 ** 64 - 1)
    assert orc.rand_vec(1, 7)[0] == np.float32(np.float32(s >> 40) / np.float32(1 << 24) * 2 - 1)


def test_rng_xorshift64star():
    """ferrum_ref/src/kernels/rng.rs:L55-L82"""
    a, b = orc.Rng(7), orc.Rng(7)
    for _ in range(100):
        x = a.next_f32()
        assert x == b.next_f32() and 0.0 <= x < 1.0
    assert orc.Rng(7).next_u64() != orc.Rng(8).next_u64()
    assert orc.Rng(0).next_u64() != 0
    r = orc.Rng(3)
    seen = [0] * 5
    for _ in range(2000):
        seen[r.below(5)] += 1
    assert all(c > 300 for c in seen)
    assert orc.Rng(1).below(1) == 0
    # one step by hand
    s = 7
    s ^= s >> 12
    s ^= (s << 25) & (2 ** 64 - 1)
    s ^= s >> 27
    assert orc.Rng(7).next_u64() == (s * 0x2545F4914F6CDD1D) & (2 ** 64 - 1)


# ---- nn (ferrum_ref/src/kernels/nn.rs:L147-L243) ----------------------------------------------

def test_gelu_known_values():
    assert orc.gelu(0.0) == 0.0
    assert abs(orc.gelu(1.0) - 0.841192) < 1e-5
    assert abs(orc.gelu(-1.0) + 0.158808) < 1e-5
    assert orc.gelu(20.0) == 20.0


def test_layernorm_normalises_each_row():
    x = orc.rand_vec(24, 1)
    y = orc.layernorm(x, np.ones(8), np.zeros(8), 3, 8).reshape(3, 8)
    for row in y:
        assert abs(row.mean()) < 1e-5 and abs(row.var() - 1.0) < 1e-3
    y2 = orc.layernorm(x, np.full(8, 2.0), np.ones(8), 3, 8)
    assert abs(y2[0] - (2.0 * y[0, 0] + 1.0)) < 1e-5


def test_attention_is_causal_and_first_token_returns_v():
    batch, t, heads, hd = 2, 5, 2, 3
    n = batch * t * heads * hd
    q, k, v = orc.rand_vec(n, 1), orc.rand_vec(n, 2), orc.rand_vec(n, 3)
    out = orc.attention(q, k, v, batch, t, heads, hd)
    assert abs(out[0] - v[0]) < 1e-6
    # changing a future key/value must not change earlier rows
    k2, v2 = k.copy(), v.copy()
    k2[(t - 1) * heads * hd:t * heads * hd] += 1.0
    v2[(t - 1) * heads * hd:t * heads * hd] += 1.0
    out2 = orc.attention(q, k2, v2, batch, t, heads, hd)
    assert np.array_equal(out[:(t - 1) * heads * hd], out2[:(t - 1) * heads * hd])


def test_score_logprob_and_argmax_flag():
    lp, gr = orc.score([1.0, 3.0, 2.0, 5.0, 5.0, 1.0], [1, 1], 3)
    assert gr[0] and not gr[1]  # ties resolve to the first maximum
    row = np.array([1.0, 3.0, 2.0], dtype=np.float64)
    assert abs(lp[0] - (3.0 - np.log(np.exp(row).sum()))) < 1e-5
    # cross-entropy of 4 zero logits is ln 4 (nn.rs:L212-L220)
    lp, _ = orc.score([0.0, 0.0, 0.0, 0.0], [1], 4)
    assert abs(-lp[0] - math.log(4.0)) < 1e-6
    # the server's f64 variant counts any tied maximum as greedy (serving/decoder.rs:L80)
    lp64, gr64 = orc.logprobs_f64([1.0, 3.0, 2.0, 5.0, 5.0, 1.0], [1, 1], 3)
    assert gr64[0] and gr64[1]
    assert abs(lp64[0] - (3.0 - np.log(np.exp(row).sum()))) < 1e-9


def test_argmax_first_maximum_and_nan_never_wins():
    """ferrum_model/src/sampling.rs:L32-L40"""
    assert orc.argmax([1.0, 5.0, 5.0, 2.0]) == 1
    assert orc.argmax([float("nan"), 1.0, 0.5]) == 1
    assert orc.argmax([float("nan"), float("nan")]) == 0


# ---- Llama ops (ferrum_ref/src/models/llama/ops.rs:L165-L300) ---------------------------------

def test_rmsnorm_matches_the_formula_and_gives_unit_rms():
    y = orc.rmsnorm([3.0, 4.0], [1.0, 2.0], 1, 2, 0.0)
    inv = 1.0 / math.sqrt(12.5)
    assert abs(y[0] - 3.0 * inv) < 1e-6 and abs(y[1] - 8.0 * inv) < 1e-6
    r = orc.rand_vec(24, 1)
    y = orc.rmsnorm(r, np.ones(8), 3, 8, 0.0).reshape(3, 8)
    for row in y:
        assert abs((row * row).mean() - 1.0) < 1e-4


def test_silu_known_values():
    assert orc.silu(0.0) == 0.0
    assert abs(orc.silu(1.0) - 0.7310586) < 1e-6
    assert abs(orc.silu(-20.0)) < 1e-6 and abs(orc.silu(20.0) - 20.0) < 1e-5
    assert orc.silu(-1e6) == 0.0 and orc.silu(1e6) == 1e6  # saturation stays finite


def test_rope_at_position_zero_is_the_identity():
    c, s = orc.rope_tables(0, 1, 4, 10000.0)
    assert c.tolist() == [1.0, 1.0] and s.tolist() == [0.0, 0.0]
    x = orc.rand_vec(8, 2)
    assert np.array_equal(orc.apply_rope(x, 1, 2, 4, 4, c, s, FC_ROPE_NORM), x)


def test_rope_preserves_pair_norms_and_the_two_pairings_differ():
    x0 = orc.rand_vec(8, 3)
    c, s = orc.rope_tables(5, 1, 8, 10000.0)
    n = orc.apply_rope(x0, 1, 1, 8, 8, c, s, FC_ROPE_NORM)
    e = orc.apply_rope(x0, 1, 1, 8, 8, c, s, FC_ROPE_NEOX)
    for i in range(4):
        assert abs((x0[2 * i] ** 2 + x0[2 * i + 1] ** 2) - (n[2 * i] ** 2 + n[2 * i + 1] ** 2)) < 1e-5
        assert abs((x0[i] ** 2 + x0[i + 4] ** 2) - (e[i] ** 2 + e[i + 4] ** 2)) < 1e-5
    assert not np.array_equal(n, e)


def test_rope_only_rotates_the_first_rope_dim_channels():
    x = orc.rand_vec(8, 4)
    c, s = orc.rope_tables(3, 1, 4, 10000.0)
    y = orc.apply_rope(x, 1, 1, 8, 4, c, s, FC_ROPE_NEOX)
    assert np.array_equal(y[4:], x[4:]) and not np.array_equal(y[:4], x[:4])


def test_rope_scaling_divides_frequencies_and_positions_by_hand():
    c, s = orc.rope_tables(8, 1, 4, 100.0, [2.0, 1.0], 4.0)
    f1 = np.float32(100.0) ** np.float32(-0.5)
    want0 = np.float32(8.0 * 1.0 / 2.0 / 4.0)
    want1 = np.float32(np.float32(8.0) * f1 / np.float32(4.0))
    assert abs(c[0] - math.cos(want0)) < 1e-6 and abs(s[0] - math.sin(want0)) < 1e-6
    assert abs(c[1] - math.cos(want1)) < 1e-6 and abs(s[1] - math.sin(want1)) < 1e-6
    a = orc.rope_tables(7, 3, 4, 1e4, [1.0, 1.0], 1.0)
    b = orc.rope_tables(7, 3, 4, 1e4)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_attention_with_one_position_returns_v():
    heads, kv, hd = 4, 2, 3
    q, k, v = orc.rand_vec(heads * hd, 5), orc.rand_vec(kv * hd, 6), orc.rand_vec(kv * hd, 7)
    o = orc.attend_row(q, k, v, 1, heads, kv, hd)
    for h in range(heads):
        g = (h // 2) * hd
        assert np.array_equal(o[h * hd:(h + 1) * hd], v[g:g + hd])


def test_gqa_shares_kv_heads_between_grouped_query_heads():
    hd = 4
    q1 = orc.rand_vec(hd, 8)
    q = np.concatenate([q1, q1])
    k, v = orc.rand_vec(3 * hd, 9), orc.rand_vec(3 * hd, 10)
    o = orc.attend_row(q, k, v, 3, 2, 1, hd)
    assert np.array_equal(o[:hd], o[hd:])
    o2 = orc.attend_row(q, orc.rand_vec(6 * hd, 11), orc.rand_vec(6 * hd, 12), 3, 2, 2, hd)
    assert not np.array_equal(o2[:hd], o2[hd:])


# ---- model properties (ferrum_ref/src/models/llama/tests.rs:L69-L111, gpt2 tests) --------------

def test_tied_head_is_the_transposed_embedding():
    t = helpers.ref_random_llama(helpers.tiny_llama_cfg(), 2, False, True)
    assert np.array_equal(t.head, orc.transpose(t.tok, 13, 8))


@pytest.mark.parametrize("ty,biases,kv", [(FC_ROPE_NORM, False, 2), (FC_ROPE_NEOX, True, 2),
                                          (FC_ROPE_NORM, False, 4), (FC_ROPE_NEOX, True, 1)])
def test_cached_decode_matches_the_full_forward_for_every_variant(ty, biases, kv):
    cfg = helpers.tiny_llama_cfg(rope_type=ty, kv_heads=kv)
    m = orc.OracleLlama(helpers.ref_random_llama(cfg, 3, biases, False))
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    full = m.forward_logits(ids)
    for i, t in enumerate(ids):
        step = m.feed(t)
        assert np.abs(step - full[i]).max() < 1e-4
    assert m.pos() == len(ids)


def test_a_prefix_gives_the_same_logits_as_the_prefix_of_a_longer_run():
    m = orc.OracleLlama(helpers.ref_random_llama(helpers.tiny_llama_cfg(), 4, False, False))
    long, short = m.forward_logits([1, 2, 3, 4, 5]), m.forward_logits([1, 2, 3])
    assert np.abs(long[:3] - short).max() < 1e-5


def test_llama_errors():
    cfg = helpers.tiny_llama_cfg()
    m = orc.OracleLlama(helpers.ref_random_llama(cfg, 4, False, False))
    with pytest.raises(ValueError, match="must be in 1..=12"):
        m.forward_logits(list(range(13)))
    with pytest.raises(IndexError):
        m.feed(13)
    for _ in range(12):
        m.feed(1)
    with pytest.raises(RuntimeError, match="context of 12 tokens is full"):
        m.feed(1)
    m.reset()
    assert m.pos() == 0


def test_gpt2_cached_feed_matches_forward_logits():
    from ferrum_gpu_b200.hostmodel import Gpt2Config
    cfg = Gpt2Config(vocab=11, ctx=10, dim=8, heads=2, layers=2, hidden=16)
    m = orc.OracleGpt2(helpers.ref_random_gpt2(cfg, 1))
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    full = m.forward_logits(ids)
    for i, t in enumerate(ids):
        assert np.abs(m.feed(t) - full[i]).max() < 1e-4
    with pytest.raises(RuntimeError, match="context of 10 tokens is full"):
        m.feed(1); m.feed(1); m.feed(1)


# ---- independent float32 numpy implementation of the Llama forward ------------------------------

_np_llama_forward = helpers.np_llama_forward


@pytest.mark.parametrize("name,cfg,biases,tied", helpers.gpu_llama_variants())
def test_oracle_llama_agrees_with_independent_numpy(name, cfg, biases, tied):
    m = helpers.ref_random_llama(cfg, 7, biases, tied)
    ids = [3, 16, 0, 9, 9, 4, 11, 2, 7, 5][:cfg.ctx]
    got = orc.OracleLlama(m).forward_logits(ids)
    want = _np_llama_forward(m, ids)
    assert orc.max_rel_err(got, want) < 2e-5, name


# ---- sampling (ferrum_model/src/sampling.rs:L102-L200, the reference's own cases) --------------------
_L = [1.0, 3.0, 3.0, 0.5, -2.0]


def test_sample_temperature_zero_is_greedy_whatever_the_rng():
    r = orc.Rng(1)
    assert all(orc.sample(_L, rng=r) == 1 for _ in range(10))


def test_sample_top_k_one_equals_greedy():
    r = orc.Rng(2)
    assert all(orc.sample(_L, temperature=1.5, top_k=1, rng=r) == 1 for _ in range(20))


def test_sample_seeded_draws_are_reproducible_and_cover_the_support():
    def run(seed):
        r = orc.Rng(seed)
        return [orc.sample(_L, temperature=1.0, rng=r) for _ in range(200)]
    draws = run(9)
    assert draws == run(9)
    assert 1 in draws and 2 in draws and all(t < 5 for t in draws)
    assert sum(1 for t in draws if t in (1, 2)) > 120


def test_sample_top_p_cuts_the_tail():
    r = orc.Rng(3)
    assert all(orc.sample(_L, temperature=1.0, top_p=0.5, rng=r) in (1, 2) for _ in range(200))


def test_sample_repetition_penalty_demotes_recent_tokens():
    r = orc.Rng(4)
    assert orc.sample(_L, repetition_penalty=4.0, recent=[1], rng=r) == 2   # 3.0 / 4 < 3.0: the tied twin wins
    assert orc.sample([-1.0, -1.5], repetition_penalty=4.0, recent=[0], rng=r) == 1  # negatives go further down
    assert orc.sample(_L, repetition_penalty=4.0, recent=[99], rng=r) == 1  # out-of-range ids are ignored


def test_sample_degenerate_inputs():
    r = orc.Rng(5)
    assert orc.sample([float("nan"), float("nan")], temperature=1.0, rng=r) == 0
    assert orc.sample([0.0], temperature=1.0, rng=r) == 0


def test_host_rng_and_candidate_draw_mirror_the_oracle():
    """The engine mirror's generator and its draw over pre-sorted candidates against `sample` on the full row."""
    from ferrum_gpu_b200.engine import Rng, SampleParams, sample_candidates
    a, b = Rng(9), orc.Rng(9)
    assert [float(a.next_f32()) for _ in range(50)] == [b.next_f32() for _ in range(50)]
    rng = np.random.default_rng(1)
    row = (rng.standard_normal(500) * 2).astype(np.float32)
    for p in (SampleParams(0.7, 20, 1.0, 1.0), SampleParams(1.2, 50, 0.8, 1.0)):
        order = np.argsort(-row, kind="stable")[:p.top_k]
        ours, theirs = Rng(3), orc.Rng(3)
        for _ in range(200):
            assert sample_candidates(order, row[order], p, ours) == orc.sample(row, p.temperature, p.top_k, p.top_p,
                                                                               rng=theirs)


def test_f16_stored_weights_round_to_nearest_even_without_a_scale():
    """QKind::F16 (ferrum_wgpu/src/ops/quant.rs:L33-L36, codec/quant.rs:L70,L108): two bytes per element, little
    endian; the round trip is exactly IEEE binary16 rounding (numpy's float16 cast is the independent check)."""
    from ferrum_gpu_b200._ffi import FC_F16
    rng = np.random.default_rng(4)
    w = np.concatenate([rng.standard_normal(200).astype(np.float32) * np.float32(3.0), helpers.nasty(56)])
    k, n = 64, 4
    finite = np.nan_to_num(w, nan=0.0)  # NaN payloads are not compared
    snapped = orc.snap_matrix(FC_F16, finite, k, n)
    with np.errstate(over="ignore"):
        want = finite.astype(np.float16).astype(np.float32)
    assert np.array_equal(snapped.view(np.uint32), want.view(np.uint32))
    raw = orc.quantise_matrix(FC_F16, finite, k, n)
    assert raw.size == k * n * 2 == orc.block_bytes(FC_F16, k * n)
    with np.errstate(over="ignore"):
        assert np.array_equal(raw.view(np.float16).reshape(n, k).view(np.uint16),
                              finite.reshape(k, n).T.astype(np.float16).view(np.uint16))


# ---- FP8 stored formats (ferrum_gguf/src/codec/fp8.rs; known answers of fp8/tests.rs) ---------------

def test_fp8_codes_have_the_published_values():
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    # fp8/tests.rs:L4-L13
    assert orc.fp8_decode(E4, 0x00) == 0.0
    assert orc.fp8_decode(E4, 0x01) == 2.0 ** -9   # the smallest subnormal
    assert orc.fp8_decode(E4, 0x08) == 2.0 ** -6   # the smallest normal
    assert orc.fp8_decode(E4, 0x38) == 1.0
    assert orc.fp8_decode(E4, 0x7e) == 448.0       # the largest finite value
    assert math.isnan(orc.fp8_decode(E4, 0x7f)) and math.isnan(orc.fp8_decode(E4, 0xff))
    assert orc.fp8_decode(E4, 0xb8) == -1.0
    # fp8/tests.rs:L16-L25
    assert orc.fp8_decode(E5, 0x01) == 2.0 ** -16
    assert orc.fp8_decode(E5, 0x04) == 2.0 ** -14
    assert orc.fp8_decode(E5, 0x3c) == 1.0
    assert orc.fp8_decode(E5, 0x7b) == 57344.0
    assert orc.fp8_decode(E5, 0x7c) == math.inf and orc.fp8_decode(E5, 0xfc) == -math.inf
    assert math.isnan(orc.fp8_decode(E5, 0x7d))


def test_fp8_decode_agrees_with_the_ieee_style_bit_layouts():
    """E5M2 is the top byte of an IEEE half; E4M3 is a half with the exponent re-biased by 8 - an
    independent statement of the two tables."""
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    for code in range(256):
        want = np.array([code << 8], dtype=np.uint16).view(np.float16)[0]
        got = orc.fp8_decode(E5, code)
        assert (math.isnan(got) and np.isnan(want)) or got == float(want), hex(code)
        if code & 0x7f == 0x7f:
            continue  # E4M3's NaN
        e, m = (code >> 3) & 15, code & 7
        mag = m / 8 * 2.0 ** -6 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        assert orc.fp8_decode(E4, code) == (-mag if code & 0x80 else mag), hex(code)


def test_fp8_every_finite_code_round_trips_through_encode():
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    for kind, limit in ((E4, 0x7e), (E5, 0x7b)):  # fp8/tests.rs:L28-L38
        for code in range(limit + 1):
            v = orc.fp8_decode(kind, code)
            assert orc.fp8_decode(kind, orc.fp8_encode(kind, v)) == v
            assert orc.fp8_decode(kind, orc.fp8_encode(kind, -v)) == -v


def test_fp8_encode_rounds_to_nearest_ties_to_even_and_saturates():
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    # fp8/tests.rs:L41-L58
    assert orc.fp8_encode(E4, 1.0625) == 0x38      # midpoint of 1.0 and 1.125: the even code
    assert orc.fp8_encode(E4, 1.0626) == 0x39
    assert orc.fp8_encode(E4, 1.1875) == 0x3a      # midpoint of 1.125 and 1.25
    assert orc.fp8_encode(E4, 1.0e9) == 0x7e and orc.fp8_encode(E4, -1.0e9) == 0xfe
    assert orc.fp8_encode(E4, math.inf) == 0x7e
    assert orc.fp8_encode(E4, -0.0) == 0x80
    assert orc.fp8_encode(E4, math.nan) == 0x7f
    assert orc.fp8_encode(E5, math.nan) == 0x7e
    assert orc.fp8_encode(E5, 1.0e9) == 0x7b


def test_fp8_blocks_scale_to_the_formats_range():
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    # fp8/tests.rs:L61-L82
    data = np.array([math.sin(i * 0.31) * (1.0 + i % 5) for i in range(64)], dtype=np.float32)
    for kind, tol in ((E4, 0.07), (E5, 0.13)):
        raw = orc.encode(kind, data)
        assert raw.size == 2 * 34 == orc.block_bytes(kind, 64)
        back = orc.decode(kind, raw, 64)
        for b in range(2):
            blk, got = data[32 * b:32 * b + 32], back[32 * b:32 * b + 32]
            assert np.all(np.abs(blk - got) <= tol * np.max(np.abs(blk)))
        # the scale is f16(amax / max) and the largest element lands on (or next to) the top code
        d = np.frombuffer(raw[:2].tobytes(), dtype=np.float16)[0]
        assert d == np.float16(np.max(np.abs(data[:32])) / np.float32(448.0 if kind == E4 else 57344.0))
    assert np.array_equal(orc.decode(E4, orc.encode(E4, np.zeros(32, np.float32)), 32), np.zeros(32, np.float32))


def test_fp8_snapping_is_idempotent():
    """Re-encoding dequantised FP8 weights gives the same values (what lets a GPU run and the oracle share one
    dequantised model)."""
    from ferrum_gpu_b200._ffi import FC_FP8_E4M3 as E4, FC_FP8_E5M2 as E5
    w = orc.rand_vec(64 * 40, 21) * np.float32(0.05)
    for kind in (E4, E5):
        once = orc.snap_matrix(kind, w, 64, 40)
        assert np.max(np.abs(once - w)) <= (0.07 if kind == E4 else 0.13) * np.max(np.abs(w))
        twice = orc.snap_matrix(kind, once, 64, 40)
        assert np.max(np.abs(twice - once)) <= 2.0 ** -10 * np.max(np.abs(w))


# ---- MXFP4 (ferrum_gguf/src/codec/mxfp4.rs; known answers of mxfp4/tests.rs) -------------------------

MXFP4_VALUES = [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]


def test_mxfp4_half_scale_is_two_to_the_e_minus_128_for_every_byte():
    for e in range(255):  # mxfp4/tests.rs:L4-L8
        assert orc.mxfp4_half_scale(e) == float(np.float32(2.0 ** (e - 128))), e


def test_mxfp4_a_block_of_representable_values_round_trips_exactly():
    from ferrum_gpu_b200._ffi import FC_MXFP4
    vals = np.array([MXFP4_VALUES[i % 16] * 0.5 for i in range(32)], dtype=np.float32)  # mxfp4/tests.rs:L11-L23
    raw = orc.encode(FC_MXFP4, vals)
    assert raw.size == 17 == orc.block_bytes(FC_MXFP4, 32)
    assert raw[0] == 127           # amax = 6, floor(log2 6) = 2, e = 2 - 2 + 127
    assert raw[1] & 15 == 0 and raw[2] & 15 == 1  # the low nibble of byte j is element j
    assert np.array_equal(orc.decode(FC_MXFP4, raw, 32), vals)


def test_mxfp4_error_is_at_most_half_a_step_inside_the_range():
    from ferrum_gpu_b200._ffi import FC_MXFP4
    data = np.array([((i * 37 % 101) - 50.0) / 25.0 for i in range(64)], dtype=np.float32)  # mxfp4/tests.rs:L26-L45
    back = orc.decode(FC_MXFP4, orc.encode(FC_MXFP4, data), 64)
    for b in range(2):
        blk, got = data[32 * b:32 * b + 32], back[32 * b:32 * b + 32]
        d = orc.mxfp4_half_scale(orc.mxfp4_scale_byte(float(np.max(np.abs(blk)))))
        for x, y in zip(blk, got):
            limit = 2.0 * d if abs(x) <= 12.0 * d else abs(x) - 12.0 * d
            assert abs(x - y) <= limit + 1e-6, (x, y, d)


def test_mxfp4_zeros_tiny_and_huge_values_keep_a_valid_block():
    from ferrum_gpu_b200._ffi import FC_MXFP4
    zeros = np.zeros(32, dtype=np.float32)  # mxfp4/tests.rs:L48-L61
    assert np.array_equal(orc.encode(FC_MXFP4, zeros), np.zeros(17, dtype=np.uint8))
    assert np.array_equal(orc.decode(FC_MXFP4, orc.encode(FC_MXFP4, zeros), 32), zeros)
    v = np.full(32, 0.5, dtype=np.float32)
    v[3] = np.inf
    assert orc.encode(FC_MXFP4, v)[0] == 0        # a non-finite amax falls back to scale 0
    assert orc.encode(FC_MXFP4, np.full(32, 3.0e38, dtype=np.float32))[0] == 252
    assert np.all(np.isfinite(orc.decode(FC_MXFP4, orc.encode(FC_MXFP4, np.full(32, 1e-38, dtype=np.float32)), 32)))


def test_mxfp4_a_tie_between_two_codes_takes_the_lower_one():
    from ferrum_gpu_b200._ffi import FC_MXFP4
    v = np.zeros(32, dtype=np.float32)  # mxfp4/tests.rs:L64-L74
    v[0], v[1] = 6.0, 2.5
    b = orc.encode(FC_MXFP4, v)
    assert b[1] & 15 == 7 and b[1] >> 4 == 0 and b[2] & 15 == 4


def test_mxfp4_scale_byte_boundaries_agree_with_the_exponent_field():
    """floor(log2(amax)) is the f32 exponent except where the f32 logarithm of a value just below a power
    of two rounds up to the integer; the device encoder takes the logarithm in f64 and rounds it to f32,
    and this pins that the two agree on the floats next to every power of two."""
    for k in range(-126, 128):
        p = np.float32(2.0) ** np.float32(k)
        x = p
        for _ in range(24):
            x = np.nextafter(x, np.float32(0.0), dtype=np.float32)
            via_f64 = int(np.floor(np.float32(np.log2(np.float64(x))))) - 2 + 127
            assert orc.mxfp4_scale_byte(float(x)) == min(max(via_f64, 0), 254), (k, float(x))
        assert orc.mxfp4_scale_byte(float(p)) == min(max(k - 2 + 127, 0), 254)


# ---- Q2_K (ferrum_gguf/src/codec/q2k.rs, decode blocks.rs:L199-L220; known answers of q2k/tests.rs) ----

def _q2k_wave(n):
    i = np.arange(n)
    # q2k/tests.rs:L5-L9, in f32 like the reference
    a = np.sin((i.astype(np.float32) * np.float32(0.37)).astype(np.float32), dtype=np.float32) * np.float32(0.8)
    return (a + ((i * 7 % 13).astype(np.float32) - np.float32(6.0)) * np.float32(0.02)).astype(np.float32)


def test_q2k_nearest_int_rounds_half_to_even():
    for x, want in [(0.5, 0), (1.5, 2), (2.5, 2), (-0.5, 0), (-1.5, -2), (3.7, 4), (-3.7, -4), (0.0, 0)]:
        assert orc.q2k_nearest_int(x) == want, x  # q2k/tests.rs:L16-L30


def test_q2k_block_is_84_bytes_and_decodes_to_256_values():
    from ferrum_gpu_b200._ffi import FC_Q2_K
    raw = orc.encode(FC_Q2_K, _q2k_wave(512))
    assert raw.size == 2 * 84 == orc.block_bytes(FC_Q2_K, 512)
    assert orc.decode(FC_Q2_K, raw, 512).size == 512
    assert orc.block_bytes(FC_Q2_K, 288) == 0  # whole super-blocks only


def test_q2k_error_is_far_below_the_signal_and_every_sub_block_is_close():
    from ferrum_gpu_b200._ffi import FC_Q2_K
    data = _q2k_wave(1024)  # q2k/tests.rs:L41-L63
    back = orc.decode(FC_Q2_K, orc.encode(FC_Q2_K, data), 1024)
    signal = np.sqrt(np.mean(data.astype(np.float64) ** 2))
    assert np.sqrt(np.mean((data - back).astype(np.float64) ** 2)) < 0.30 * signal
    for j in range(64):
        sub, got = data[16 * j:16 * j + 16], back[16 * j:16 * j + 16]
        assert np.all(np.abs(sub - got) <= (sub.max() - sub.min()) / 3.0 + 0.02), j


def test_q2k_constant_zero_and_all_negative_blocks_are_valid():
    from ferrum_gpu_b200._ffi import FC_Q2_K
    z = orc.encode(FC_Q2_K, np.zeros(256, np.float32))  # q2k/tests.rs:L66-L77
    assert not z.any()
    assert not orc.decode(FC_Q2_K, z, 256).any()
    c = orc.decode(FC_Q2_K, orc.encode(FC_Q2_K, np.full(256, 0.5, np.float32)), 256)
    assert np.all(np.abs(c - 0.5) < 0.2)
    n = orc.decode(FC_Q2_K, orc.encode(FC_Q2_K, np.full(256, -0.5, np.float32)), 256)
    assert np.all(np.abs(n + 0.5) < 0.05)


def test_q2k_encoding_is_deterministic_and_each_block_is_independent():
    from ferrum_gpu_b200._ffi import FC_Q2_K
    data = _q2k_wave(512)  # q2k/tests.rs:L80-L86
    a = orc.encode(FC_Q2_K, data)
    assert np.array_equal(a, orc.encode(FC_Q2_K, data))
    assert np.array_equal(a[:84], orc.encode(FC_Q2_K, data[:256]))
    assert np.array_equal(a[84:], orc.encode(FC_Q2_K, data[256:]))


def test_q2k_decode_agrees_with_an_independent_numpy_restatement():
    """blocks.rs:L199-L220 by array indexing instead of the scan: element e of a super-block lives in byte
    32 * (e // 128) + e % 32 at shift 2 * ((e % 128) // 32); sub-block e // 16 holds its scale and min."""
    from ferrum_gpu_b200._ffi import FC_Q2_K
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=3 * 84, dtype=np.uint8)
    for b in range(3):  # finite f16 scales
        raw[84 * b + 80:84 * b + 84] = np.array([0.013, 0.007], dtype=np.float16).view(np.uint8)
    got = orc.decode(FC_Q2_K, raw, 768)
    for b in range(3):
        blk = raw[84 * b:84 * b + 84]
        d, dmin = (np.float32(v) for v in blk[80:84].view(np.float16))
        e = np.arange(256)
        q = (blk[16 + 32 * (e // 128) + e % 32] >> (2 * ((e % 128) // 32))) & 3
        sc = blk[e // 16]
        want = (d * (sc & 15).astype(np.float32)) * q.astype(np.float32) - dmin * (sc >> 4).astype(np.float32)
        assert np.array_equal(got[256 * b:256 * b + 256], want.astype(np.float32))


def test_q2k_falls_back_to_q4_0_on_widths_of_whole_32s_only():
    from ferrum_gpu_b200._ffi import FC_Q2_K
    assert orc.effective_kind(FC_Q2_K, 512) == FC_Q2_K and orc.effective_kind(FC_Q2_K, 96) == FC_Q4_0
    assert orc.effective_kind(FC_Q2_K, 24) == FC_Q2_K and orc.effective_kind(FC_Q8_0, 96) == FC_Q8_0
    w = orc.rand_vec(96 * 5, 2)
    assert np.array_equal(orc.snap_matrix(FC_Q2_K, w, 96, 5), orc.snap_matrix(FC_Q4_0, w, 96, 5))
