"""`generate_with` and `sample` on the host (ferrum_gpu_core/src/engine/mod.rs:L204-L242,
ferrum_model/src/sampling.rs:L32-L100): the stop-at-context rules and the draw, without a GPU."""
import numpy as np
import pytest

from ferrum_gpu_b200.engine import GenOpts, Rng, SampleParams, argmax, generate_with, sample
from oracle import oracle as orc


def table_feed(vocab=11):
    """A decoder whose logits depend only on the last token and on how many tokens it has seen."""
    fed = []

    def feed(t):
        fed.append(t)
        row = np.cos(np.arange(vocab, dtype=np.float32) * (t + 1) + len(fed)).astype(np.float32)
        return row

    return feed, fed


def test_only_the_new_tokens_come_back_and_the_last_one_is_not_fed():
    feed, fed = table_feed()
    out = generate_with(feed, 32, [3, 1, 4], GenOpts(max_new=5))
    assert len(out) == 5
    assert fed == [3, 1, 4] + out[:-1]


def test_generation_stops_when_the_context_is_full():
    """history.len() < ctx guards both the sampling and the feed (L230-L240)."""
    feed, fed = table_feed()
    out = generate_with(feed, 8, [3, 1, 4], GenOpts(max_new=50))
    assert len(out) == 5, "3 prompt tokens + 5 new ones fill a context of 8"
    assert fed == [3, 1, 4] + out[:-1], "the token that fills the context is not fed"
    feed, fed = table_feed()
    assert generate_with(feed, 8, [1, 2, 3, 4, 5, 6, 7], GenOpts(max_new=50)) and len(fed) == 7


def test_a_prompt_that_leaves_no_room_is_an_error():
    feed, _ = table_feed()
    with pytest.raises(ValueError, match="the prompt is empty"):
        generate_with(feed, 8, [], GenOpts(max_new=1))
    with pytest.raises(ValueError, match="the prompt has 8 tokens but the context is 8"):
        generate_with(feed, 8, list(range(8)), GenOpts(max_new=1))


def test_sampled_generation_uses_the_seed_and_the_whole_history():
    sp = SampleParams(temperature=0.9, top_k=4, top_p=0.9, repetition_penalty=1.3)
    feed, _ = table_feed()
    out = generate_with(feed, 64, [3, 1, 4], GenOpts(max_new=12, sampling=sp, seed=9))
    feed2, _ = table_feed()
    rng, hist, logits = orc.Rng(9), [3, 1, 4], None
    for t in hist:
        logits = feed2(t)
    want = []
    for i in range(12):
        nxt = orc.sample(logits, sp.temperature, sp.top_k, sp.top_p, sp.repetition_penalty, hist, rng)
        want.append(nxt)
        hist.append(nxt)
        if i + 1 < 12:
            logits = feed2(nxt)
    assert out == want


def test_sample_matches_the_restated_reference_on_awkward_rows():
    rng = np.random.default_rng(3)
    rows = [rng.standard_normal(50).astype(np.float32) for _ in range(6)]
    rows[1][[3, 7]] = np.nan
    rows[2][5] = rows[2][9] = rows[2].max() + 1  # a tie at the top
    rows[3][:] = np.nan
    rows[4][[1, 2]] = [0.0, -0.0]
    for row in rows:
        for p in (SampleParams(), SampleParams(0.7, 0, 1.0, 1.0), SampleParams(1.2, 5, 0.8, 1.4), SampleParams(0.0, 0, 1.0, 2.0)):
            recent = [int(np.nanargmax(row)) if not np.isnan(row).all() else 0, 4, 4, 99]
            ours, theirs = Rng(31), orc.Rng(31)
            for _ in range(40):
                assert sample(row, p, recent, ours) == orc.sample(row, p.temperature, p.top_k, p.top_p,
                                                                  p.repetition_penalty, recent, theirs)
    assert argmax(np.array([1.0, 3.0, 3.0, 0.5, -2.0], dtype=np.float32)) == 1
