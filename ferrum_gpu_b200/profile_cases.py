"""Small, self-terminating cases of each hot kernel, sized for an `ncu` capture (inputs above the
126 MB L2 where DRAM figures matter, a few launches, well under a GB on the device).

    python -m ferrum_gpu_b200.profile_cases gemm      # tensor-core product, Q4_0, M=16384 K=768 N=1280
    python -m ferrum_gpu_b200.profile_cases head      # fused head + log-sum-exp, M=8192 K=768 N=32000
    python -m ferrum_gpu_b200.profile_cases matvec    # decode matvec, Q4_0 and Q8_0, K=4096 N=32000, M=1
    python -m ferrum_gpu_b200.profile_cases matvec8   # tensor-core decode product, 8 rows, K=4096 N=32000
    python -m ferrum_gpu_b200.profile_cases decode    # batched decode step: 16 streams at cache length ~1500
    python -m ferrum_gpu_b200.profile_cases score     # 8 sequences x 1024 of the Llama scoring configuration
    python -m ferrum_gpu_b200.profile_cases chunk     # 32 sequences x 1024, one layer: activations above L2
    python -m ferrum_gpu_b200.profile_cases attention # the causal attention kernels alone, 16 x 1024 x 12 heads
"""
from __future__ import annotations

import sys

import numpy as np

from . import CudaLlama, Device, Mode, QKind, linear_q, upload_quantised
from .hostmodel import LlamaConfig, config_c3, random_llama, random_tokens


def _weights(k, n, seed=1):
    return (np.random.default_rng(seed).standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def gemm(dev):
    k, n, m = 768, 1280, 16384
    qw = upload_quantised(dev, QKind.Q4_0, _weights(k, n), k, n)
    x = np.random.default_rng(2).standard_normal(m * k, dtype=np.float32)
    for _ in range(3):
        linear_q(dev, x, qw, m, Mode.TENSOR_F16)
    qw.close()


def matvec(dev):
    k, n = 4096, 32000
    x = np.random.default_rng(2).standard_normal(k, dtype=np.float32)
    for kind in (QKind.Q4_0, QKind.Q8_0):
        qw = upload_quantised(dev, kind, _weights(k, n), k, n)
        for _ in range(3):
            linear_q(dev, x, qw, 1)
        qw.close()


def matvec8(dev):
    """The tensor-core decode product at 8 rows (small-batch decode)."""
    k, n = 4096, 32000
    x = np.random.default_rng(2).standard_normal(8 * k, dtype=np.float32)
    for kind in (QKind.Q4_0, QKind.Q8_0):
        qw = upload_quantised(dev, kind, _weights(k, n), k, n)
        for _ in range(3):
            linear_q(dev, x, qw, 8)
        qw.close()


def _c3_model(dev, layers=None, max_streams=1, ctx=None):
    cfg = config_c3()
    if layers:
        cfg.layers = layers
    if ctx:
        cfg.ctx = ctx
    return cfg, CudaLlama(dev, random_llama(cfg, seed=1), QKind.Q4_0, max_streams=max_streams)


def score(dev):
    cfg, g = _c3_model(dev, layers=2)
    ids = np.stack([random_tokens(10 + i, 1024, cfg.vocab) for i in range(8)])
    for _ in range(2):
        g.score_batch(ids, Mode.TENSOR_F16)
    g.close()


def head(dev):
    score(dev)


def chunk(dev):
    """A quarter of one bench chunk (the bench launches its products on 128 x 1024 rows): per-launch
    DRAM traffic scales with the rows, the weights being a few MB."""
    cfg, g = _c3_model(dev, layers=1)
    ids = np.stack([random_tokens(10 + i, 1024, cfg.vocab) for i in range(32)])
    for _ in range(2):
        g.score_batch(ids, Mode.TENSOR_F16)
    g.close()


def attention(dev):
    n_seqs, t, heads, kv = 16, 1024, 12, 4
    qkv = np.random.default_rng(0).standard_normal((n_seqs * t, (heads + 2 * kv) * 64)).astype(np.float16)
    for variant in (1, 3):
        dev.attention_f16(qkv, n_seqs, t, heads, kv, variant=variant, iters=1)


def decode(dev):
    cfg = LlamaConfig(vocab=32000, ctx=2048, dim=1024, heads=16, kv_heads=2, head_dim=64, layers=2, hidden=2816,
                      rope_dim=64, rope_base=1e6, rope_type=1, eps=1e-6)
    g = CudaLlama(dev, random_llama(cfg, seed=1, biases=True), QKind.Q8_0, max_streams=16)
    for s in range(16):
        g.prefill(random_tokens(s, 1500, cfg.vocab), stream=s)
    toks = random_tokens(99, 16, cfg.vocab)
    for _ in range(3):
        g.feed_batch(toks)
    g.close()


def head64(dev):
    """The vocabulary-head product of the 64-stream decode configuration: 64 rows of x against
    151 936 x 1024 Q8_0 weights on the mma.sync decode kernel."""
    k, n, m = 1024, 151936, 64
    qw = upload_quantised(dev, QKind.Q8_0, _weights(k, n), k, n)
    x = np.random.default_rng(2).standard_normal(m * k, dtype=np.float32)
    for _ in range(3):
        linear_q(dev, x, qw, m)
    qw.close()


def decode64(dev):
    """Four layers and the 151936-row head of the 64-stream decode configuration at 1500 cached positions:
    the per-launch times of one step (the full model repeats the layer launches 24 times)."""
    cfg = LlamaConfig(vocab=151936, ctx=2048, dim=1024, heads=16, kv_heads=2, head_dim=64, layers=4, hidden=2816,
                      rope_dim=64, rope_base=1e6, rope_type=1, eps=1e-6)
    g = CudaLlama(dev, random_llama(cfg, seed=1, biases=True, tied=True), QKind.Q8_0, max_streams=64)
    for s in range(64):
        g.prefill(random_tokens(s, 1500, cfg.vocab), stream=s)
    toks = random_tokens(99, 64, cfg.vocab)
    for _ in range(3):
        g.feed_batch(toks)
    g.close()


CASES = {"gemm": gemm, "head": head, "matvec": matvec, "matvec8": matvec8, "decode": decode, "decode64": decode64, "head64": head64, "score": score, "chunk": chunk,
         "attention": attention}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    d = Device.open(0)
    try:
        CASES[name](d)
        d.sync()
        print("case", name, "done;", d.launch_count(), "launches")
    finally:
        d.close()
