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
    seed of the draw and how many recent tokens the repetition penalty looks at. `prefill` (new here) feeds the
    prompt in one batched pass instead of token by token as `generate_with` does: Mode.EXACT_F32 (the same logits
    to 1e-5) or Mode.TENSOR_F16 (the scoring kernels; logits to the scoring tolerance)."""
    max_new: int = 16
    sampling: SampleParams | None = None
    seed: int = 1
    penalty_window: int = 64
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


def generate_with(feed, prompt, opts: GenOpts):
    """`generate_with` (engine/mod.rs:L204-L242): feed each prompt token, then sample greedily; the
    last sampled token is not fed."""
    if len(prompt) == 0:
        raise ValueError("the prompt is empty")
    out = list(int(t) for t in prompt)
    logits = None
    for t in out:
        logits = feed(t)
    for i in range(opts.max_new):
        nxt = argmax(logits)
        out.append(nxt)
        if i + 1 < opts.max_new:
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
        """`Backend::generate`: the argmax, or the top-k candidates of a sampled draw, are taken on the device;
        a logits row is read back only for sampling without a top_k (1..1024)."""
        if len(prompt) == 0:
            raise ValueError("the prompt is empty")
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        m = cls(self.dev, model, self.weights)
        try:
            out = [int(t) for t in prompt]
            sp = opts.sampling
            if sp is not None and sp.temperature > 0.0:
                if not 1 <= sp.top_k <= 1024:
                    raise ValueError("sampled decoding on the device needs 1 <= top_k <= 1024")
                rng = Rng(opts.seed)
                if opts.prefill is None:
                    for t in out:
                        m.feed_greedy(t)
                else:
                    m.prefill(out, mode=opts.prefill)
                for i in range(opts.max_new):
                    recent = out[-opts.penalty_window:] if sp.repetition_penalty != 1.0 else ()
                    idx, val = m.topk(sp.top_k, 0, sp.repetition_penalty, recent)
                    nxt = sample_candidates(idx, val, sp, rng)
                    out.append(nxt)
                    if i + 1 < opts.max_new:
                        m.feed_greedy(nxt)
                return out
            nxt = None
            if opts.prefill is None:
                for t in out:
                    nxt = m.feed_greedy(t)
            else:
                nxt = argmax(m.prefill(out, mode=opts.prefill))
            if opts.max_new > 0:
                out.append(nxt)
            if opts.max_new > 1:  # the remaining picks in one call, chained on the device
                out.extend(int(t) for t in m.decode_greedy([nxt], opts.max_new - 1)[:, 0])
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
