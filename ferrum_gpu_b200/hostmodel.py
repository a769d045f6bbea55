"""Host-side model structs: the mirror of `ferrum_ref::llama::Llama` and `ferrum_ref::gpt2::Gpt2`.

Plain f32 numpy arrays, matrices stored `[in, out]` row-major, exactly what the reference hands
a backend (ferrum_ref/src/models/llama/mod.rs:L100-L147, models/gpt2/mod.rs:L62-L114). These
are data containers only: no arithmetic on the hot path happens here.

The seeded generators draw every weight from N(0, 0.02) with norm gains 1 and biases 0 (or
N(0, 0.02) q/k/v biases for the Qwen2 shape), the distribution the benchmark configurations
name. They are synthetic stand-ins for real checkpoints.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _ffi


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    if a is None or a.size == 0:
        return C.cast(None, _ffi.f32p)
    return a.ctypes.data_as(_ffi.f32p)


@dataclass
class LlamaConfig:
    """`ferrum_ref::llama::Config` + `RopeScaling` (models/llama/mod.rs:L24-L52, ops.rs:L17-L35)."""
    vocab: int
    ctx: int
    dim: int
    heads: int
    kv_heads: int
    head_dim: int
    layers: int
    hidden: int
    rope_dim: int
    rope_base: float = 10000.0
    rope_type: int = _ffi.FC_ROPE_NORM
    eps: float = 1e-5
    rope_linear_factor: float = 1.0
    freq_factors: np.ndarray | None = None

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def validate(self) -> None:
        """`Config::validate` (models/llama/mod.rs:L65-L97); raises ValueError with its messages."""
        dims = [self.vocab, self.ctx, self.dim, self.heads, self.kv_heads, self.head_dim,
                self.layers, self.hidden, self.rope_dim]
        if 0 in dims:
            raise ValueError("every dimension must be positive")
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        if self.rope_dim > self.head_dim or self.rope_dim % 2:
            raise ValueError(f"rope_dim {self.rope_dim} must be even and at most head_dim {self.head_dim}")
        for v in (self.eps, self.rope_base):
            if not np.isfinite(v) or v <= 0:
                raise ValueError("eps and rope_base must be finite and positive")


LLAMA_MATS = ("wq", "wk", "wv", "wo", "gate", "up", "down")


@dataclass
class LlamaBlock:
    attn_norm: np.ndarray
    wq: np.ndarray
    wk: np.ndarray
    wv: np.ndarray
    wo: np.ndarray
    ffn_norm: np.ndarray
    gate: np.ndarray
    up: np.ndarray
    down: np.ndarray
    bq: np.ndarray | None = None
    bk: np.ndarray | None = None
    bv: np.ndarray | None = None


@dataclass
class Llama:
    cfg: LlamaConfig
    tok: np.ndarray
    blocks: list
    out_norm: np.ndarray
    head: np.ndarray
    tied: bool = False
    _keep: list = field(default_factory=list, repr=False)

    def mat_shape(self, name: str):
        c = self.cfg
        return {"wq": (c.dim, c.q_dim), "wk": (c.dim, c.kv_dim), "wv": (c.dim, c.kv_dim),
                "wo": (c.q_dim, c.dim), "gate": (c.dim, c.hidden), "up": (c.dim, c.hidden),
                "down": (c.hidden, c.dim), "head": (c.dim, c.vocab)}[name]

    def num_matrix_params(self) -> int:
        c = self.cfg
        per = c.dim * (c.q_dim + 2 * c.kv_dim) + c.q_dim * c.dim + 3 * c.dim * c.hidden
        return per * c.layers + c.dim * c.vocab

    def c_structs(self):
        """(FcLlamaConfig, FcLlamaWeights) pointing at this model's arrays (kept alive by self)."""
        c = self.cfg
        ff = None if c.freq_factors is None else _f32(c.freq_factors)
        cfg = _ffi.FcLlamaConfig(c.vocab, c.ctx, c.dim, c.heads, c.kv_heads, c.head_dim, c.layers,
                                 c.hidden, c.rope_dim, c.rope_type, c.rope_base, c.eps,
                                 c.rope_linear_factor, 0 if ff is None else ff.size, _ptr(ff),
                                 1 if self.tied else 0)
        arr = (_ffi.FcLlamaBlock * c.layers)()
        keep = [ff, arr]
        for i, b in enumerate(self.blocks):
            for name in _ffi.LLAMA_BLOCK_FIELDS:
                a = getattr(b, name)
                if a is not None:
                    a = _f32(a)
                    keep.append(a)
                setattr(arr[i], name, _ptr(a))
        tok, on, head = _f32(self.tok), _f32(self.out_norm), _f32(self.head)
        keep += [tok, on, head]
        w = _ffi.FcLlamaWeights(_ptr(tok), arr, _ptr(on), _ptr(head))
        self._keep = keep
        return cfg, w


@dataclass
class Gpt2Config:
    """`ferrum_ref::gpt2::Config` (models/gpt2/mod.rs:L15-L30)."""
    vocab: int
    ctx: int
    dim: int
    heads: int
    layers: int
    hidden: int

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads

    def validate(self) -> None:
        if 0 in (self.vocab, self.ctx, self.dim, self.heads, self.layers, self.hidden):
            raise ValueError("every dimension must be positive")
        if self.dim % self.heads:
            raise ValueError(f"dim {self.dim} is not divisible by heads {self.heads}")


GPT2_MATS = ("wq", "wk", "wv", "wo", "w1", "w2")


@dataclass
class Gpt2Block:
    ln1_g: np.ndarray
    ln1_b: np.ndarray
    wq: np.ndarray
    bq: np.ndarray
    wk: np.ndarray
    bk: np.ndarray
    wv: np.ndarray
    bv: np.ndarray
    wo: np.ndarray
    bo: np.ndarray
    ln2_g: np.ndarray
    ln2_b: np.ndarray
    w1: np.ndarray
    b1: np.ndarray
    w2: np.ndarray
    b2: np.ndarray


@dataclass
class Gpt2:
    cfg: Gpt2Config
    tok: np.ndarray
    pos: np.ndarray
    blocks: list
    lnf_g: np.ndarray
    lnf_b: np.ndarray
    head: np.ndarray
    _keep: list = field(default_factory=list, repr=False)

    def mat_shape(self, name: str):
        c = self.cfg
        return {"wq": (c.dim, c.dim), "wk": (c.dim, c.dim), "wv": (c.dim, c.dim),
                "wo": (c.dim, c.dim), "w1": (c.dim, c.hidden), "w2": (c.hidden, c.dim),
                "head": (c.dim, c.vocab)}[name]

    def num_matrix_params(self) -> int:
        c = self.cfg
        return (4 * c.dim * c.dim + 2 * c.dim * c.hidden) * c.layers + c.dim * c.vocab

    def c_structs(self):
        c = self.cfg
        cfg = _ffi.FcGpt2Config(c.vocab, c.ctx, c.dim, c.heads, c.layers, c.hidden)
        arr = (_ffi.FcGpt2Block * c.layers)()
        keep = [arr]
        for i, b in enumerate(self.blocks):
            for name in _ffi.GPT2_BLOCK_FIELDS:
                a = _f32(getattr(b, name))
                keep.append(a)
                setattr(arr[i], name, _ptr(a))
        tok, pos, g, bb, head = (_f32(self.tok), _f32(self.pos), _f32(self.lnf_g), _f32(self.lnf_b),
                                 _f32(self.head))
        keep += [tok, pos, g, bb, head]
        w = _ffi.FcGpt2Weights(_ptr(tok), _ptr(pos), arr, _ptr(g), _ptr(bb), _ptr(head))
        self._keep = keep
        return cfg, w


# ---- seeded synthetic weights --------------------------------------------------------------

def _normal(rng: np.random.Generator, n: int, std: float = 0.02) -> np.ndarray:
    return (rng.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float32)


def random_llama(cfg: LlamaConfig, seed: int, biases: bool = False, tied: bool = False,
                 std: float = 0.02, gain_jitter: float = 0.0) -> Llama:
    """Every matrix ~ N(0, std), norm gains 1 (+ optional jitter), q/k/v biases ~ N(0, std) or absent."""
    cfg.validate()
    rng = np.random.default_rng(seed)
    d, h, qd, kvd = cfg.dim, cfg.hidden, cfg.q_dim, cfg.kv_dim

    def gain(n):
        g = np.ones(n, dtype=np.float32)
        if gain_jitter:
            g += np.float32(gain_jitter) * rng.uniform(-1, 1, n).astype(np.float32)
        return g

    tok = _normal(rng, cfg.vocab * d, std)
    blocks = []
    for _ in range(cfg.layers):
        blocks.append(LlamaBlock(
            attn_norm=gain(d), wq=_normal(rng, d * qd, std), wk=_normal(rng, d * kvd, std),
            wv=_normal(rng, d * kvd, std), wo=_normal(rng, qd * d, std), ffn_norm=gain(d),
            gate=_normal(rng, d * h, std), up=_normal(rng, d * h, std), down=_normal(rng, h * d, std),
            bq=_normal(rng, qd, std) if biases else None,
            bk=_normal(rng, kvd, std) if biases else None,
            bv=_normal(rng, kvd, std) if biases else None))
    out_norm = gain(d)
    if tied:
        head = np.ascontiguousarray(tok.reshape(cfg.vocab, d).T).reshape(-1)
    else:
        head = _normal(rng, d * cfg.vocab, std)
    return Llama(cfg, tok, blocks, out_norm, head, tied)


def random_gpt2(cfg: Gpt2Config, seed: int, tied: bool = False, std: float = 0.02,
                bias_std: float = 0.0, gain_jitter: float = 0.0) -> Gpt2:
    """Weights ~ N(0, std), LayerNorm gains 1 and shifts/biases 0 unless bias_std / jitter are given."""
    cfg.validate()
    rng = np.random.default_rng(seed)
    d, h = cfg.dim, cfg.hidden

    def gain(n):
        g = np.ones(n, dtype=np.float32)
        if gain_jitter:
            g += np.float32(gain_jitter) * rng.uniform(-1, 1, n).astype(np.float32)
        return g

    def bias(n):
        return _normal(rng, n, bias_std) if bias_std else np.zeros(n, dtype=np.float32)

    tok = _normal(rng, cfg.vocab * d, std)
    pos = _normal(rng, cfg.ctx * d, std)
    blocks = []
    for _ in range(cfg.layers):
        blocks.append(Gpt2Block(
            ln1_g=gain(d), ln1_b=bias(d), wq=_normal(rng, d * d, std), bq=bias(d),
            wk=_normal(rng, d * d, std), bk=bias(d), wv=_normal(rng, d * d, std), bv=bias(d),
            wo=_normal(rng, d * d, std), bo=bias(d), ln2_g=gain(d), ln2_b=bias(d),
            w1=_normal(rng, d * h, std), b1=bias(h), w2=_normal(rng, h * d, std), b2=bias(d)))
    lnf_g, lnf_b = gain(d), bias(d)
    if tied:
        head = np.ascontiguousarray(tok.reshape(cfg.vocab, d).T).reshape(-1)
    else:
        head = _normal(rng, d * cfg.vocab, std)
    return Gpt2(cfg, tok, pos, blocks, lnf_g, lnf_b, head)


def random_tokens(seed: int, n: int, vocab: int) -> np.ndarray:
    """Uniform-random token ids (int32)."""
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.int32)


# The benchmark configurations (shapes only; weights are synthetic).
def config_c1() -> Gpt2Config:
    """GPT-2-style, byte-level vocab 256, 6 layers, d_model 384, 6 heads, context 256."""
    return Gpt2Config(vocab=256, ctx=256, dim=384, heads=6, layers=6, hidden=1536)


def config_c3() -> LlamaConfig:
    """Llama-style: 12 layers, d_model 768, 12 query / 4 KV heads, SwiGLU 2048, vocab 32000."""
    return LlamaConfig(vocab=32000, ctx=1024, dim=768, heads=12, kv_heads=4, head_dim=64, layers=12,
                       hidden=2048, rope_dim=64, rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM,
                       eps=1e-5)


def config_c4() -> LlamaConfig:
    """Qwen2-style: 24 layers, d_model 1024, 16 query / 2 KV heads, SwiGLU 2816, vocab 151936."""
    return LlamaConfig(vocab=151936, ctx=2048, dim=1024, heads=16, kv_heads=2, head_dim=64,
                       layers=24, hidden=2816, rope_dim=64, rope_base=1e6,
                       rope_type=_ffi.FC_ROPE_NEOX, eps=1e-6)


def config_c5() -> Gpt2Config:
    """GPT-2-124M shape: 12 layers, d_model 768, 12 heads, context 1024, vocab 50257."""
    return Gpt2Config(vocab=50257, ctx=1024, dim=768, heads=12, layers=12, hidden=3072)
