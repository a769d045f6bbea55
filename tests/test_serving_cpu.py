"""The scoring callers on CPU: the sliding-window partition and `pair` / `rolling` of
ferrum_gpu_core/src/serving/score.rs, pinned on the reference's own cases (serving/score/tests.rs), and the
partition rule of the multi-GPU group. The C entry points used here are pure host arithmetic."""
import numpy as np
import pytest

from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.serving import ZERO, Score, pair, rolling, token_logprobs, windows


class Table:
    """serving/score/tests.rs:L4-L54: bytes as tokens, a score that depends only on the target token -
    log-prob -(1 + t % 3), argmax when t is even."""

    def __init__(self, ctx):
        self.ctx, self.calls = ctx, []

    def encode(self, text):
        return list(text.encode())

    def bos(self):
        return 0

    def score(self, ids):
        assert len(ids) <= self.ctx + 1, f"window of {len(ids)} for context {self.ctx}"
        self.calls.append(len(ids))
        return [(-(1.0 + t % 3), t % 2 == 0) for t in ids[1:]]


def lp(t):
    return -(1.0 + t % 3)


def test_pair_scores_only_the_continuation():
    """tests.rs:L60-L68"""
    d = Table(32)
    s = pair(d, "ab", "cd")
    assert s.n_tokens == 2 and s.logprob == lp(99) + lp(100)
    assert not s.greedy, "99 is odd"
    assert pair(d, "ab", "d").greedy, "100 is even"


def test_trailing_context_whitespace_moves_to_the_continuation():
    """tests.rs:L70-L77"""
    d = Table(32)
    moved, same = pair(d, "ab ", "c"), pair(d, "ab", " c")
    assert moved == same and moved.n_tokens == 2


def test_an_empty_context_is_scored_after_bos_and_empty_continuation_is_zero():
    """tests.rs:L79-L86"""
    d = Table(32)
    s = pair(d, "", "ab")
    assert (s.n_tokens, s.logprob) == (2, lp(97) + lp(98))
    assert pair(d, "abc", "") == Score(0.0, 0, True)


def test_rolling_scores_every_token_after_bos():
    """tests.rs:L88-L96"""
    d = Table(32)
    s = rolling(d, "abc")
    assert s.n_tokens == 3 and s.logprob == lp(97) + lp(98) + lp(99)
    assert rolling(d, "") == ZERO


def test_long_texts_are_scored_in_windows_and_every_token_exactly_once():
    """tests.rs:L98-L121"""
    text = "".join(chr(ord("a") + i % 26) for i in range(50))
    small, big = Table(8), Table(100)
    s, whole = rolling(small, text), rolling(big, text)
    assert s.n_tokens == 50 == whole.n_tokens
    assert abs(s.logprob - whole.logprob) < 1e-9 and s.greedy == whole.greedy
    assert len(small.calls) > 1 and all(n <= 9 for n in small.calls)
    assert len(big.calls) == 1


def test_token_logprobs_handles_trivial_inputs():
    """tests.rs:L123-L133"""
    d = Table(8)
    assert token_logprobs(d, [1], 1) == ZERO
    assert token_logprobs(d, [1, 2], 5) == ZERO
    assert token_logprobs(d, [1, 2], 0).n_tokens == 1, "from is clamped to 1"


def test_a_decoder_error_is_passed_up():
    """tests.rs:L135-L172"""
    class Failing:
        ctx = 4

        def encode(self, _):
            raise RuntimeError("no tokenizer")

        def bos(self):
            return 0

        def score(self, _):
            raise RuntimeError("device lost")

    with pytest.raises(RuntimeError, match="no tokenizer"):
        pair(Failing(), "a", "b")
    with pytest.raises(RuntimeError, match="no tokenizer"):
        rolling(Failing(), "a")
    with pytest.raises(RuntimeError, match="device lost"):
        token_logprobs(Failing(), [1, 2, 3], 1)


def reference_windows(n_ids, frm, t):
    """serving/score.rs:L27-L49 line by line."""
    frm = max(frm, 1)
    if frm >= n_ids:
        return []
    half = max(t // 2, 1)
    out, nxt = [], frm
    while nxt < n_ids:
        start = 0 if nxt <= t else nxt - half
        end = min(start + t + 1, n_ids)
        out.append((start, end, nxt))
        nxt = end
    return out


def test_the_window_partition_matches_the_reference_rule_and_scores_every_target_once():
    rng = np.random.default_rng(5)
    cases = [(51, 1, 8), (2049, 1, 1024), (5000, 1, 1024), (5000, 3000, 1024), (10, 1, 1), (10, 1, 2), (3, 1, 100),
             (1025, 1, 1024), (1026, 1, 1024), (1, 1, 8), (0, 0, 8)]
    cases += [(int(rng.integers(1, 4000)), int(rng.integers(0, 50)), int(rng.integers(1, 300))) for _ in range(200)]
    for n, frm, ctx in cases:
        got = windows(n, frm, ctx)
        assert got == reference_windows(n, frm, ctx), (n, frm, ctx)
        targets = [t for s, e, f in got for t in range(f, e)]
        assert targets == list(range(max(frm, 1), n)) if max(frm, 1) < n else targets == []
        for s, e, f in got:
            assert e - s <= ctx + 1 and s < f < e
            assert s == 0 or f - s >= max(ctx // 2, 1), "at least half a window of history"


def test_group_sequences_partition():
    lib = _ffi.load()
    for n, parts in [(256, 1), (256, 2), (256, 8), (7, 4), (3, 8), (0, 2), (512, 4)]:
        seen = []
        for part in range(parts):
            cnt = lib.fc_group_sequences(n, part, parts, None, 0)
            buf = np.empty(cnt, dtype=np.uint32)
            assert lib.fc_group_sequences(n, part, parts, buf.ctypes.data, cnt) == cnt
            assert list(buf) == list(range(part, n, parts))
            seen += list(buf)
        assert sorted(seen) == list(range(n))
