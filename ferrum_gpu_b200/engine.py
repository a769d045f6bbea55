"""Engine layer: the mirror of `trait Backend` and `GpuBackend`
(ferrum_gpu_core/src/engine/mod.rs:L204-L312, engine/gpu.rs). `CudaBackend` is what
`Session::new_with` would build for `--device cuda`."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .device import Device
from .hostmodel import Gpt2, Llama
from .quant import Mode, QKind
from .resident import CudaGpt2, CudaLlama


@dataclass
class GenOpts:
    """The fields of `GenOpts` this path uses (engine/mod.rs:L189-L202): greedy decoding."""
    max_new: int = 16


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
        """`Backend::generate`: greedy continuation with the argmax taken on the device."""
        if len(prompt) == 0:
            raise ValueError("the prompt is empty")
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        m = cls(self.dev, model, self.weights)
        try:
            out = [int(t) for t in prompt]
            nxt = None
            for t in out:
                nxt = m.feed_greedy(t)
            for i in range(opts.max_new):
                out.append(nxt)
                if i + 1 < opts.max_new:
                    nxt = m.feed_greedy(nxt)
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
