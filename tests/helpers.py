"""Shared test inputs, built the way the reference's own tests build theirs."""
import numpy as np

from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.hostmodel import (Gpt2, Gpt2Block, Gpt2Config, Llama, LlamaBlock, LlamaConfig)
from oracle import oracle as orc


def nasty(n: int) -> np.ndarray:
    """ferrum_wgpu/src/ops/quant/tests.rs:L11-L23: spread magnitudes, all-zero blocks, tiny blocks
    (subnormal f16 scale), large blocks and exact small integers."""
    v = orc.rand_vec(n, 9) * np.float32(3.0)
    for i in range(n):
        m = i // 32 % 7
        if m == 0:
            v[i] = v[i] * np.float32(1e-6)
        elif m == 1:
            v[i] = 0.0
        elif m == 2:
            v[i] = v[i] * np.float32(1e4)
        elif m == 3:
            v[i] = np.float32(i % 9) - np.float32(4.0)
    return v


def ref_random_llama(cfg: LlamaConfig, seed: int, biases: bool, tied: bool) -> Llama:
    """`Llama::random` (ferrum_ref/src/models/llama/params.rs:L38-L93), same draw order."""
    d, h, qd, kvd = cfg.dim, cfg.hidden, cfg.q_dim, cfg.kv_dim
    s = [max(seed, 1) * 1000]

    def mat(n, scale):
        s[0] += 1
        return orc.rand_vec(n, s[0]) * np.float32(scale)

    def gain(n):
        s[0] += 1
        return np.float32(1.0) + np.float32(0.1) * orc.rand_vec(n, s[0])

    qk = np.float32(0.5) * np.sqrt(np.float32(8.0) / np.float32(d))
    bias = (lambda n: mat(n, 0.1)) if biases else (lambda n: None)
    blocks = []
    for _ in range(cfg.layers):
        an = gain(d)
        wq = mat(d * qd, qk); bq = bias(qd)
        wk = mat(d * kvd, qk); bk = bias(kvd)
        wv = mat(d * kvd, 0.5); bv = bias(kvd)
        wo = mat(qd * d, 0.5)
        fn = gain(d)
        gate = mat(d * h, 0.5); up = mat(d * h, 0.5); down = mat(h * d, 0.5)
        blocks.append(LlamaBlock(attn_norm=an, wq=wq, wk=wk, wv=wv, wo=wo, ffn_norm=fn, gate=gate,
                                 up=up, down=down, bq=bq, bk=bk, bv=bv))
    tok = mat(cfg.vocab * d, 1.0)
    head = orc.transpose(tok, cfg.vocab, d) if tied else mat(d * cfg.vocab, 0.5)
    out_norm = gain(d)
    return Llama(cfg, tok, blocks, out_norm, head, tied)


def ref_random_gpt2(cfg: Gpt2Config, seed: int) -> Gpt2:
    """`Gpt2::random` (ferrum_ref/src/models/gpt2/mod.rs:L137-L184), same draw order."""
    d, h = cfg.dim, cfg.hidden
    s = [max(seed, 1) * 1000]

    def mat(n, scale):
        s[0] += 1
        return orc.rand_vec(n, s[0]) * np.float32(scale)

    def gain(n):
        s[0] += 1
        return np.float32(1.0) + np.float32(0.1) * orc.rand_vec(n, s[0])

    blocks = []
    for _ in range(cfg.layers):
        kw = {}
        kw["ln1_g"] = gain(d); kw["ln1_b"] = mat(d, 0.1)
        kw["wq"] = mat(d * d, 0.5); kw["bq"] = mat(d, 0.1)
        kw["wk"] = mat(d * d, 0.5); kw["bk"] = mat(d, 0.1)
        kw["wv"] = mat(d * d, 0.5); kw["bv"] = mat(d, 0.1)
        kw["wo"] = mat(d * d, 0.5); kw["bo"] = mat(d, 0.1)
        kw["ln2_g"] = gain(d); kw["ln2_b"] = mat(d, 0.1)
        kw["w1"] = mat(d * h, 0.5); kw["b1"] = mat(h, 0.1)
        kw["w2"] = mat(h * d, 0.5); kw["b2"] = mat(d, 0.1)
        blocks.append(Gpt2Block(**kw))
    tok = mat(cfg.vocab * d, 1.0)
    pos = mat(cfg.ctx * d, 0.5)
    lnf_g = gain(d); lnf_b = mat(d, 0.1)
    head = mat(d * cfg.vocab, 0.5)
    return Gpt2(cfg, tok, pos, blocks, lnf_g, lnf_b, head)


def tiny_llama_cfg(**kw) -> LlamaConfig:
    """ferrum_ref/src/models/llama/tests.rs:L4-L19."""
    base = dict(vocab=13, ctx=12, dim=8, heads=4, kv_heads=2, head_dim=4, layers=2, hidden=16,
                rope_dim=4, rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
    base.update(kw)
    return LlamaConfig(**base)


def gpu_llama_variants():
    """The four shapes of ferrum_wgpu/src/models/llama/tests.rs:L10-L42 (llama; qwen = NEOX +
    biases + tied; MQA + partial rotary; dim 24 = not whole 32-blocks), widened to dim 32/64 where
    the quantised path needs whole blocks."""
    def mk(**kw):
        base = dict(vocab=17, ctx=10, dim=32, heads=4, kv_heads=2, head_dim=8, layers=2, hidden=64,
                    rope_dim=8, rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
        base.update(kw)
        return LlamaConfig(**base)

    return [
        ("llama", mk(), False, False),
        ("qwen", mk(rope_type=_ffi.FC_ROPE_NEOX), True, True),
        ("mqa-partial", mk(kv_heads=1, rope_dim=4), False, False),
        ("dim24", mk(dim=24, heads=3, kv_heads=3, head_dim=8, rope_dim=8), True, False),
    ]


def np_llama_forward(m, ids, f=np.float32):
    """Independent numpy restatement of the Llama forward pass in precision `f` (float32 to cross-check the
    oracle, float64 as the exact-arithmetic yardstick). RoPE angles are the f32 ones every implementation uses."""
    c = m.cfg
    FC_ROPE_NORM = _ffi.FC_ROPE_NORM
    d, qd, kvd, hd = c.dim, c.q_dim, c.kv_dim, c.head_dim
    x = m.tok.reshape(c.vocab, d)[ids].astype(f)
    n = len(ids)
    half = c.rope_dim // 2
    freq = (np.float64(c.rope_base) ** (-2.0 * np.arange(half) / c.rope_dim)).astype(np.float32)
    theta = (np.arange(n, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32).astype(f)
    cos, sin = np.cos(theta).astype(f), np.sin(theta).astype(f)

    def rms(x, g):
        ms = (x * x).mean(axis=1, keepdims=True, dtype=f)
        return (x * (f(1) / np.sqrt(ms + f(c.eps))) * g).astype(f)

    def rope(t, heads):
        t = t.reshape(n, heads, hd).copy()
        if c.rope_type == FC_ROPE_NORM:
            a, b = t[:, :, 0:2 * half:2].copy(), t[:, :, 1:2 * half:2].copy()
            t[:, :, 0:2 * half:2] = a * cos[:, None, :] - b * sin[:, None, :]
            t[:, :, 1:2 * half:2] = a * sin[:, None, :] + b * cos[:, None, :]
        else:
            a, b = t[:, :, :half].copy(), t[:, :, half:2 * half].copy()
            t[:, :, :half] = a * cos[:, None, :] - b * sin[:, None, :]
            t[:, :, half:2 * half] = a * sin[:, None, :] + b * cos[:, None, :]
        return t

    for b in m.blocks:
        h = rms(x, b.attn_norm)
        q = h @ b.wq.reshape(d, qd)
        k = h @ b.wk.reshape(d, kvd)
        v = h @ b.wv.reshape(d, kvd)
        if b.bq is not None:
            q, k, v = q + b.bq, k + b.bk, v + b.bv
        q, k, v = rope(q, c.heads), rope(k, c.kv_heads), v.reshape(n, c.kv_heads, hd)
        g = c.heads // c.kv_heads
        a = np.zeros((n, c.heads, hd), dtype=f)
        for hh in range(c.heads):
            s = (q[:, hh] @ k[:, hh // g].T) * f(1.0 / np.sqrt(f(hd)))
            s = np.where(np.tril(np.ones((n, n), dtype=bool)), s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p = p / p.sum(axis=1, keepdims=True)
            a[:, hh] = p.astype(f) @ v[:, hh // g]
        x = x + a.reshape(n, qd) @ b.wo.reshape(qd, d)
        h = rms(x, b.ffn_norm)
        gt, up = h @ b.gate.reshape(d, c.hidden), h @ b.up.reshape(d, c.hidden)
        x = x + ((gt / (f(1) + np.exp(-gt))) * up).astype(f) @ b.down.reshape(c.hidden, d)
    return rms(x, m.out_norm) @ m.head.reshape(d, c.vocab)
