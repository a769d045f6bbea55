"""Candidate selection for sampled decoding on the device against the restated `sampling::sample`
(ferrum_model/src/sampling.rs:L42-L100): the top-k set and its order are exact (integer / ordering work),
and a draw over the returned candidates picks the token the oracle picks on the full row."""
import numpy as np
import pytest

from ferrum_gpu_b200 import CudaLlama, QKind
from ferrum_gpu_b200.engine import CudaBackend, GenOpts, Rng, SampleParams, sample_candidates
from oracle import oracle as orc

from tests.helpers import tiny_llama_cfg
from ferrum_gpu_b200.hostmodel import random_llama

pytestmark = pytest.mark.gpu


def _expected_topk(row, k, penalty=1.0, recent=()):
    """numpy restatement of sampling.rs:L44-L66: penalty in order, drop NaN, stable sort by total_cmp descending."""
    l = np.array(row, dtype=np.float32)
    if penalty != 1.0:
        for t in recent:
            if 0 <= t < l.size:
                l[t] = l[t] / np.float32(penalty) if l[t] > 0 else l[t] * np.float32(penalty)
    bits = l.view(np.uint32)
    key = np.where(bits >> 31 != 0, ~bits, bits ^ np.uint32(0x80000000)).astype(np.uint64)
    idx = np.nonzero(~np.isnan(l))[0]
    order = idx[np.argsort(-(key[idx].astype(np.int64)), kind="stable")]
    order = order[:k]
    return order.astype(np.int32), l[order]


@pytest.mark.parametrize("vocab", [5, 256, 1000, 32000, 151936])
@pytest.mark.parametrize("k", [1, 7, 40, 1024])
def test_topk_set_and_order_are_exact(dev, vocab, k):
    rng = np.random.default_rng(vocab + k)
    row = rng.standard_normal(vocab).astype(np.float32)
    want_i, want_v = _expected_topk(row, k)
    got_i, got_v = dev.topk(row, k)
    np.testing.assert_array_equal(got_i, want_i)
    np.testing.assert_array_equal(got_v.view(np.uint32), want_v.view(np.uint32))


def test_ties_signed_zeros_infinities_and_nan(dev):
    row = np.zeros(3000, dtype=np.float32)
    row[::7] = 2.5            # hundreds of tied maxima: the lowest indices win, in index order
    row[5] = np.inf
    row[11] = np.nan          # never a candidate
    row[13] = -0.0            # sorts after +0.0
    row[100:200] = -np.inf
    for k in (1, 3, 50, 429, 431, 1024):
        want_i, want_v = _expected_topk(row, k)
        got_i, got_v = dev.topk(row, k)
        np.testing.assert_array_equal(got_i, want_i)
        np.testing.assert_array_equal(got_v.view(np.uint32), want_v.view(np.uint32))
    few = np.array([np.nan, 1.0, np.nan, -2.0], dtype=np.float32)  # fewer candidates than k
    got_i, got_v = dev.topk(few, 10)
    assert got_i.tolist() == [1, 3] and got_v.tolist() == [1.0, -2.0]
    got_i, _ = dev.topk(np.array([np.nan, np.nan], dtype=np.float32), 4)
    assert got_i.size == 0


def test_repetition_penalty_in_order_with_repeats(dev):
    rng = np.random.default_rng(3)
    row = rng.standard_normal(2000).astype(np.float32) * 3
    recent = [int(np.argmax(row)), 17, int(np.argmax(row)), 1999, 5000, 17]   # repeats and an out-of-range id
    want_i, want_v = _expected_topk(row, 64, 1.3, recent)
    got_i, got_v = dev.topk(row, 64, 1.3, recent)
    np.testing.assert_array_equal(got_i, want_i)
    np.testing.assert_array_equal(got_v.view(np.uint32), want_v.view(np.uint32))


def test_draws_over_the_candidates_match_the_oracle_on_the_full_row(dev):
    rng = np.random.default_rng(5)
    row = (rng.standard_normal(32000) * 2).astype(np.float32)
    for p in (SampleParams(0.8, 40, 1.0, 1.0), SampleParams(1.3, 200, 0.9, 1.0), SampleParams(1.0, 5, 0.5, 1.2)):
        recent = [int(i) for i in np.argsort(-row)[:3]] if p.repetition_penalty != 1.0 else []
        idx, val = dev.topk(row, p.top_k, p.repetition_penalty, recent)
        ours, theirs = Rng(77), orc.Rng(77)
        for _ in range(300):
            want = orc.sample(row, p.temperature, p.top_k, p.top_p, p.repetition_penalty, recent, theirs)
            assert sample_candidates(idx, val, p, ours) == want


def test_sampled_generation_matches_the_oracle_loop(dev):
    """`generate` with sampling: feed, select on the device, draw on the host - the tokens of the oracle's loop
    (feed the f32 oracle, `sample` the full row with the same seed)."""
    cfg = tiny_llama_cfg()
    m = random_llama(cfg, seed=21, std=0.3)
    sp = SampleParams(temperature=0.9, top_k=8, top_p=0.95, repetition_penalty=1.1)
    opts = GenOpts(max_new=7, sampling=sp, seed=5)
    prompt = [1, 4, 2]
    got = CudaBackend(dev, None).generate(m, prompt, opts)
    oracle = orc.OracleLlama(m)
    out, rng = list(prompt), orc.Rng(5)
    logits = None
    for t in out:
        logits = oracle.feed(t)
    for i in range(opts.max_new):
        nxt = orc.sample(logits, sp.temperature, sp.top_k, sp.top_p, sp.repetition_penalty, out, rng)
        out.append(nxt)
        if i + 1 < opts.max_new:
            logits = oracle.feed(nxt)
    assert got == out[len(prompt):]
