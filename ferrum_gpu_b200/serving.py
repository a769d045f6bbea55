"""Log-likelihoods the way the reference's server computes them: the host-side mirror of
`ferrum_gpu_core::serving::score` (serving/score.rs). Same names, argument meaning and results; the windows of a
long text are scored in one batched pass on the device instead of one `score` call after another.

A *decoder* here is any object with the reference's `Decoder` surface that scoring needs
(serving/decoder.rs): `ctx` (positions of context), `bos()`, `encode(text) -> ids`, and either
`score(ids) -> [(logprob, greedy)]` (one window at a time, like the reference) or `score_many(list of ids)`
(all windows at once). Tokenizers are outside this library: `encode` is the caller's."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _ffi


@dataclass(frozen=True)
class Score:
    """`Score` (serving/score.rs:L9-L17): summed log-probability, tokens scored, every one the argmax."""
    logprob: float
    n_tokens: int
    greedy: bool


ZERO = Score(0.0, 0, True)


def windows(n_ids: int, from_: int, ctx: int):
    """The window partition of `token_logprobs` (serving/score.rs:L27-L49): [(start, end, first target)]."""
    lib = _ffi.load()
    n = lib.fc_score_windows(n_ids, from_, ctx, None, None, None, 0)
    s, e, f = (np.empty(n, dtype=np.uint32) for _ in range(3))
    lib.fc_score_windows(n_ids, from_, ctx, s.ctypes.data, e.ctypes.data, f.ctypes.data, n)
    return [(int(s[i]), int(e[i]), int(f[i])) for i in range(n)]


def token_logprobs(d, ids, from_: int) -> Score:
    """Sum log p(ids[i] | ids[..i]) for i in from..len(ids) over windows of the decoder's context
    (serving/score.rs:L27-L49)."""
    ids = list(ids)
    wins = windows(len(ids), from_, d.ctx)
    if not wins:
        return ZERO
    if hasattr(d, "score_many"):
        per = d.score_many([ids[s:e] for s, e, _ in wins])
    else:
        per = [d.score(ids[s:e]) for s, e, _ in wins]
    lp, n, greedy = 0.0, 0, True
    for (start, end, first), rows in zip(wins, per):
        for target in range(first, end):
            l, g = rows[target - start - 1]
            lp += float(np.float32(l))
            n += 1
            greedy = greedy and bool(g)
    return Score(lp, n, greedy)


def pair(d, context: str, continuation: str) -> Score:
    """log p(continuation | context) (serving/score.rs:L52-L80): trailing whitespace of the context moves to
    the continuation, an empty context is scored after the BOS token."""
    trimmed = context.rstrip()
    if len(trimmed) < len(context):
        context, continuation = trimmed, context[len(trimmed):] + continuation
    if not continuation:
        return ZERO
    ctx_ids = [d.bos()] if not context else list(d.encode(context))
    joint = None if not context else list(d.encode(context + continuation))
    if joint is not None and len(joint) > len(ctx_ids) and joint[:len(ctx_ids)] == ctx_ids:
        ids = joint
    else:
        ids = ctx_ids + list(d.encode(continuation))
    return token_logprobs(d, ids, len(ctx_ids))


def rolling(d, text: str) -> Score:
    """Log-likelihood of all of `text`, the first token conditioned on BOS (serving/score.rs:L83-L86)."""
    return token_logprobs(d, [d.bos()] + list(d.encode(text)), 1)


class ModelDecoder:
    """The scoring half of `ModelDecoder` (serving/decoder.rs:L141-L149) over a resident model: `score` is the
    resident model's, `score_many` sends every window through one ragged batch."""

    def __init__(self, model, encode, bos: int, mode=None):
        from .quant import Mode
        self.model, self.encode, self._bos = model, encode, bos
        self.ctx = model.cfg.ctx
        self.mode = Mode.EXACT_F32 if mode is None else mode

    def bos(self) -> int:
        return self._bos

    def score(self, ids):
        lp, gr = self.model.score(ids, self.mode)
        return list(zip(lp.tolist(), gr.tolist()))

    def score_many(self, seqs):
        lps, grs, _ = self.model.score_ragged(seqs, self.mode)
        return [list(zip(lp.tolist(), gr.tolist())) for lp, gr in zip(lps, grs)]
