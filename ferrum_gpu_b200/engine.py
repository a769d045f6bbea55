"""Engine layer: the mirror of `trait Backend` and `GpuBackend`
(ferrum_gpu_core/src/engine/mod.rs:L204-L312, engine/gpu.rs). `CudaBackend` is what
`Session::new_with` would build for `--device cuda`."""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from .device import Device
from .hostmodel import Gpt2, Llama
from .quant import Mode, QKind
from .resident import CudaGpt2, CudaLlama


@dataclass
class SampleParams:
    """`sampling::Params` (ferrum_model/src/sampling.rs:L8-L30)."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0


@dataclass
class GenOpts:
    """The fields of `GenOpts` this path uses (engine/mod.rs:L189-L202): how many tokens, how to pick them, the
    seed of the draw and how many recent tokens the repetition penalty looks at (0: the whole history, as
    `generate_with` passes it to `sample`). `prefill` (new here) feeds the
    prompt in one batched pass instead of token by token as `generate_with` does: Mode.EXACT_F32 (the same logits
    to 1e-5) or Mode.TENSOR_F16 (the scoring kernels; logits to the scoring tolerance)."""
    max_new: int = 16
    sampling: SampleParams | None = None
    seed: int = 1
    penalty_window: int = 0
    prefill: Mode | None = None


class Rng:
    """`ferrum_ref::rng::Rng` (ferrum_ref/src/kernels/rng.rs:L7-L41): xorshift64*, `next_f32` = top 24 bits."""

    def __init__(self, seed: int):
        self.s = (seed or 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF

    def next_u64(self) -> int:
        s = self.s
        s ^= s >> 12
        s ^= (s << 25) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 27
        self.s = s
        return (s * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF

    def next_f32(self) -> np.float32:
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def sample_candidates(idx, val, p: SampleParams, rng: Rng) -> int:
    """The tail of `sampling::sample` (sampling.rs:L67-L100) over candidates that are already penalised, sorted
    and cut to top_k (what `topk` returns): softmax of (l - max) / temperature with sequential f32 sums, the
    nucleus cut with renormalisation, one draw, the last candidate as the fallback."""
    if len(idx) == 0:
        return 0
    f = np.float32
    t = f(p.temperature)
    probs = [f(math.exp(float((f(v) - f(val[0])) / t))) for v in val]  # expf, correctly rounded
    total = f(0.0)
    for x in probs:
        total = f(total + x)
    probs = [f(x / total) for x in probs]
    idx = list(idx)
    if p.top_p < 1.0:
        acc, keep = f(0.0), len(probs)
        for i, x in enumerate(probs):
            acc = f(acc + x)
            if acc >= f(p.top_p):
                keep = i + 1
                break
        idx, probs = idx[:keep], probs[:keep]
        s2 = f(0.0)
        for x in probs:
            s2 = f(s2 + x)
        probs = [f(x / s2) for x in probs]
    r = rng.next_f32()
    acc = f(0.0)
    for i, x in zip(idx, probs):
        acc = f(acc + x)
        if r < acc:
            return int(i)
    return int(idx[-1])


def argmax(logits) -> int:
    """`sampling::argmax` (ferrum_model/src/sampling.rs:L32-L40): first maximum, NaN never wins."""
    best, bv = 0, -np.inf
    for i, v in enumerate(np.asarray(logits, dtype=np.float32)):
        if v > bv:
            best, bv = i, v
    return best


def sample(logits, p: SampleParams, recent, rng: Rng) -> int:
    """`sampling::sample` (ferrum_model/src/sampling.rs:L44-L100) on a host logits row: repetition penalty over
    `recent` (in order, a repeated token is penalised again), argmax at temperature 0, else the candidates by
    descending logit (ties: lower index first, NaN dropped), top_k, softmax, nucleus cut, one draw."""
    f = np.float32
    l = np.array(logits, dtype=np.float32)
    if p.repetition_penalty != 1.0:
        for t in recent:
            if 0 <= t < l.size:
                l[t] = f(l[t] / f(p.repetition_penalty)) if l[t] > 0.0 else f(l[t] * f(p.repetition_penalty))
    if p.temperature <= 0.0:
        return argmax(l)
    idx = [i for i in range(l.size) if not np.isnan(l[i])]
    if not idx:
        return 0
    # f32::total_cmp descending with a stable sort: -0.0 sorts below +0.0, ties keep the lower index first
    key = l.view(np.int32).astype(np.int64)
    key = np.where(key < 0, -(key & 0x7FFFFFFF) - 1, key)
    idx.sort(key=lambda i: -int(key[i]))
    if p.top_k > 0:
        idx = idx[:p.top_k]
    return sample_candidates(idx, [l[i] for i in idx], p, rng)


def generate_with(feed, ctx: int, prompt, opts: GenOpts):
    """`generate_with` (engine/mod.rs:L204-L242): feed each prompt token, then sample `opts.max_new` tokens,
    stopping when the context is full; the last sampled token is not fed. Returns only the new tokens."""
    if len(prompt) == 0:
        raise ValueError("the prompt is empty")
    if len(prompt) >= ctx:
        raise ValueError(f"the prompt has {len(prompt)} tokens but the context is {ctx}")
    params = opts.sampling or SampleParams()
    rng = Rng(opts.seed)
    logits = None
    for t in prompt:
        logits = feed(int(t))
    history = [int(t) for t in prompt]
    out = []
    while len(out) < opts.max_new and len(history) < ctx:
        nxt = sample(logits, params, history[-opts.penalty_window:] if opts.penalty_window else history, rng)
        out.append(nxt)
        history.append(nxt)
        if len(history) < ctx and len(out) < opts.max_new:
            logits = feed(nxt)
    return out


class CudaBackend:
    """`impl Backend for CudaBackend`: generate / decoders / score on one B200."""

    def __init__(self, dev: Device, weights: QKind | None = None):
        self.dev, self.weights = dev, weights

    @classmethod
    def open(cls, ordinal: int = 0, weights: QKind | None = None) -> "CudaBackend":
        return cls(Device.open(ordinal), weights)

    def with_weights(self, q: QKind | None) -> "CudaBackend":
        """`GpuBackend::with_weights` (engine/gpu.rs:L42-L46)."""
        self.weights = q
        return self

    def kind(self) -> str:
        return "cuda"

    def name(self) -> str:
        return self.dev.name()

    def train(self, *_a, **_k):
        raise RuntimeError("training is not available on the cuda backend")

    def llama_decoder(self, model: Llama):
        """`Backend::llama_decoder` -> `Gpt2Feed` closure (engine/mod.rs:L256, gpu.rs:L78-L82)."""
        m = CudaLlama(self.dev, model, self.weights)
        return lambda token: m.feed(token)

    def gpt2_decoder(self, model: Gpt2):
        m = CudaGpt2(self.dev, model, self.weights)
        return lambda token: m.feed(token)

    def generate(self, model, prompt, opts: GenOpts):
        """`Backend::generate` with `generate_with`'s contract (engine/mod.rs:L204-L242): only the new tokens come
        back, a prompt that does not leave room is an error, and generation stops when the context is full. The
        argmax, or the top-k candidates of a sampled draw, are taken on the device; a logits row is read back only
        for sampling without a top_k in 1..1024."""
        if len(prompt) == 0:
            raise ValueError("the prompt is empty")
        ctx = model.cfg.ctx
        if len(prompt) >= ctx:
            raise ValueError(f"the prompt has {len(prompt)} tokens but the context is {ctx}")
        max_new = min(opts.max_new, ctx - len(prompt))  # history reaches ctx: stop there
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        m = cls(self.dev, model, self.weights)
        try:
            history = [int(t) for t in prompt]
            out = []
            sp = opts.sampling
            if sp is not None and sp.temperature > 0.0:
                rng = Rng(opts.seed)
                on_device = 1 <= sp.top_k <= 1024
                logits = None
                if opts.prefill is None:
                    for t in history:
                        logits = m.feed_greedy(t) if on_device else m.feed(t)
                else:
                    logits = m.prefill(history, mode=opts.prefill)
                while len(out) < max_new:
                    recent = history[-opts.penalty_window:] if opts.penalty_window else history
                    if on_device:
                        idx, val = m.topk(sp.top_k, 0, sp.repetition_penalty,
                                          recent if sp.repetition_penalty != 1.0 else ())
                        nxt = sample_candidates(idx, val, sp, rng)
                    else:
                        nxt = sample(logits, sp, recent, rng)
                    out.append(nxt)
                    history.append(nxt)
                    if len(history) < ctx and len(out) < max_new:
                        logits = m.feed_greedy(nxt) if on_device else m.feed(nxt)
                return out
            if max_new == 0:
                return out
            if sp is not None and sp.repetition_penalty != 1.0:  # greedy with a penalty: the host loop
                return generate_with(lambda t: m.feed(t), ctx, history, opts)
            nxt = None
            if opts.prefill is None:
                for t in history:
                    nxt = m.feed_greedy(t)
            else:
                nxt = argmax(m.prefill(history, mode=opts.prefill))
            out.append(nxt)
            # the remaining picks in one call, chained on the device; the last pick is not fed, so the chain
            # consumes max_new - 1 positions and history ends at len(prompt) + max_new <= ctx
            if max_new > 1:
                out.extend(int(t) for t in m.decode_greedy([nxt], max_new - 1)[:, 0])
            return out
        finally:
            m.close()

    def score(self, model, ids, mode: Mode = Mode.TENSOR_F16):
        """Scoring at the engine layer (the reference routes it to the CPU oracle,
        serving/decoder.rs:L141-L149): (logprob, greedy) per position of one or many sequences."""
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        m = cls(self.dev, model, self.weights)
        try:
            ids = np.asarray(ids, dtype=np.int32)
            if ids.ndim == 1:
                return m.score(ids, mode)
            return m.score_batch(ids, mode)
        finally:
            m.close()
