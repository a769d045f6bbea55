"""TEST INFRASTRUCTURE - ctypes wrapper of the CPU oracle (oracle/ferrum_oracle.cpp).

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module. The
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.hostmodel import (GPT2_MATS, LLAMA_MATS, Gpt2, Gpt2Block, Llama, LlamaBlock)

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libferrum_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile."""
    src = os.path.join(HERE, "ferrum_oracle.cpp")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "libferrum_oracle.so"] + (["-B"] if force else []))
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB):
        build()
    L = C.CDLL(LIB)
    vp, sz, u64, i32, u32 = C.c_void_p, C.c_size_t, C.c_uint64, C.c_int32, C.c_uint32
    f, P = C.c_float, C.POINTER
    sig = {
        "or_f16_to_f32": (f, [C.c_uint16]), "or_f32_to_f16": (C.c_uint16, [f]),
        "or_fp8_decode": (f, [C.c_int, C.c_uint8]), "or_fp8_encode": (C.c_uint8, [C.c_int, f]),
        "or_mxfp4_half_scale": (f, [C.c_uint8]), "or_mxfp4_scale_byte": (C.c_uint8, [f]),
        "or_effective_kind": (C.c_int, [C.c_int, sz]), "or_q2k_nearest_int": (i32, [f]),
        "or_block_bytes": (sz, [C.c_int, sz]),
        "or_encode": (C.c_int, [C.c_int, vp, sz, vp]), "or_decode": (C.c_int, [C.c_int, vp, sz, vp]),
        "or_quantise_matrix": (C.c_int, [C.c_int, vp, sz, sz, vp]),
        "or_snap_matrix": (C.c_int, [C.c_int, vp, sz, sz, vp]),
        "or_snap_rows": (C.c_int, [C.c_int, vp, sz, vp]),
        "or_pack_reference_layout": (C.c_int, [C.c_int, vp, sz, sz, vp]),
        "or_transpose": (None, [vp, sz, sz, vp]),
        "or_matmul": (None, [vp, vp, sz, sz, sz, vp, C.c_int]),
        "or_matmul_tuned": (None, [vp, vp, sz, sz, sz, vp, C.c_int]),
        "or_set_tuned": (None, [C.c_int]),
        "or_llama_extend_last": (C.c_int, [vp, vp, u32, vp]),
        "or_rand_vec": (None, [sz, u64, vp]),
        "or_gelu": (f, [f]), "or_silu": (f, [f]),
        "or_layernorm": (None, [vp, vp, vp, sz, sz, vp]),
        "or_rmsnorm": (None, [vp, vp, sz, sz, f, vp]),
        "or_rope_tables": (None, [sz, sz, sz, f, vp, sz, f, vp, vp]),
        "or_apply_rope": (None, [vp, sz, sz, sz, sz, vp, vp, C.c_int]),
        "or_attend_row": (None, [vp, vp, vp, sz, sz, sz, sz, vp]),
        "or_attention": (None, [vp, vp, vp, sz, sz, sz, sz, vp]),
        "or_score": (None, [vp, vp, sz, sz, vp, vp]),
        "or_logprobs_f64": (None, [vp, vp, sz, sz, vp, vp]),
        "or_argmax": (i32, [vp, sz]),
        "or_sample": (i32, [vp, sz, f, sz, f, f, vp, sz, P(u64)]),
        "or_rng_new": (u64, [u64]), "or_rng_next_u64": (u64, [P(u64)]),
        "or_rng_next_f32": (f, [P(u64)]), "or_rng_below": (u64, [P(u64), u64]),
        "or_llama_create": (vp, [P(_ffi.FcLlamaConfig), P(_ffi.FcLlamaWeights), C.c_int]),
        "or_llama_destroy": (None, [vp]), "or_llama_reset": (None, [vp]),
        "or_llama_pos": (u32, [vp]),
        "or_llama_feed": (C.c_int, [vp, i32, vp]),
        "or_llama_forward_logits": (C.c_int, [vp, vp, u32, vp]),
        "or_llama_extend": (C.c_int, [vp, vp, u32, vp]),
        "or_gpt2_create": (vp, [P(_ffi.FcGpt2Config), P(_ffi.FcGpt2Weights), C.c_int]),
        "or_gpt2_destroy": (None, [vp]), "or_gpt2_reset": (None, [vp]), "or_gpt2_pos": (u32, [vp]),
        "or_gpt2_feed": (C.c_int, [vp, i32, vp]),
        "or_gpt2_forward_logits": (C.c_int, [vp, vp, u32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- codec ---------------------------------------------------------------------------------

def f16_to_f32(h: int) -> float:
    return lib().or_f16_to_f32(h)


def f32_to_f16(x: float) -> int:
    return lib().or_f32_to_f16(C.c_float(x))


def fp8_decode(kind: int, code: int) -> float:
    """`Fp8::decode` (ferrum_gguf/src/codec/fp8.rs:L41-L70); kind is FC_FP8_E4M3 or FC_FP8_E5M2."""
    return lib().or_fp8_decode(kind, code)


def fp8_encode(kind: int, x: float) -> int:
    """`Fp8::encode` (fp8.rs:L75-L109)."""
    return lib().or_fp8_encode(kind, C.c_float(x))


def mxfp4_half_scale(e: int) -> float:
    """`half_scale` (ferrum_gguf/src/codec/mxfp4.rs:L22-L28): 2^(e - 128)."""
    return lib().or_mxfp4_half_scale(e)


def mxfp4_scale_byte(amax: float) -> int:
    """`scale_byte` (mxfp4.rs:L49-L54)."""
    return lib().or_mxfp4_scale_byte(C.c_float(amax))


def effective_kind(kind: int, k: int) -> int:
    """`effective` (ferrum_wgpu/src/ops/quant.rs:L134-L144): Q2_K on a width of whole 32s only is Q4_0."""
    return lib().or_effective_kind(kind, k)


def q2k_nearest_int(x: float) -> int:
    """`nearest_int` (ferrum_gguf/src/codec/q2k.rs:L17-L20)."""
    return lib().or_q2k_nearest_int(C.c_float(x))


def block_bytes(kind: int, n: int) -> int:
    return lib().or_block_bytes(kind, n)


def encode(kind: int, data) -> np.ndarray:
    d = _f32(data).reshape(-1)
    if d.size % (256 if kind == _ffi.FC_Q2_K else 32):
        raise ValueError(f"{d.size} elements is not a multiple of the block size")
    out = np.empty(block_bytes(kind, d.size), dtype=np.uint8)
    assert lib().or_encode(kind, _p(d), d.size, _p(out)) == 0
    return out


def decode(kind: int, data: np.ndarray, n: int) -> np.ndarray:
    b = np.ascontiguousarray(data, dtype=np.uint8)
    if b.size != block_bytes(kind, n) or n % (256 if kind == _ffi.FC_Q2_K else 32):
        raise ValueError("tensor byte length does not match its type and element count")
    out = np.empty(n, dtype=np.float32)
    assert lib().or_decode(kind, _p(b), n, _p(out)) == 0
    return out


def quantise_matrix(kind: int, w, k: int, n: int) -> np.ndarray:
    """`[k, n]` f32 -> GGUF block bytes of the transposed `[n, k]` rows (ops/quant.rs:L238-L252)."""
    w = _f32(w).reshape(-1)
    if k % (256 if kind == _ffi.FC_Q2_K else 32) or k == 0 or w.size != k * n:
        raise ValueError(f"cannot quantise {w.size} elements as a {k} x {n} weight in whole blocks")
    out = np.empty(block_bytes(kind, k * n), dtype=np.uint8)
    assert lib().or_quantise_matrix(kind, _p(w), k, n, _p(out)) == 0
    return out


def snap_matrix(kind: int, w, k: int, n: int) -> np.ndarray:
    """What a quantised run computes with: dequantised `[k, n]` matrix (models/llama/mod.rs:L188-L199)."""
    w = _f32(w).reshape(-1)
    out = np.empty(k * n, dtype=np.float32)
    assert lib().or_snap_matrix(kind, _p(w), k, n, _p(out)) == 0
    return out


def snap_rows(kind: int, data) -> np.ndarray:
    d = _f32(data).reshape(-1)
    out = np.empty_like(d)
    assert lib().or_snap_rows(kind, _p(d), d.size, _p(out)) == 0
    return out


def pack_reference_layout(kind: int, data: np.ndarray, k: int, n: int) -> np.ndarray:
    words = (9 if kind == _ffi.FC_Q8_0 else 5) * (k // 32) * n
    out = np.zeros(words, dtype=np.uint32)
    b = np.ascontiguousarray(data, dtype=np.uint8)
    assert lib().or_pack_reference_layout(kind, _p(b), k, n, _p(out)) == 0
    return out


# ---- kernels -------------------------------------------------------------------------------

def transpose(data, rows: int, cols: int) -> np.ndarray:
    d = _f32(data).reshape(-1)
    out = np.empty_like(d)
    lib().or_transpose(_p(d), rows, cols, _p(out))
    return out


def matmul(a, b, m: int, k: int, n: int, threads: int = 1) -> np.ndarray:
    a, b = _f32(a).reshape(-1), _f32(b).reshape(-1)
    if a.size != m * k:
        raise ValueError(f"matmul: operand a has {a.size} elements, shape needs {m * k}")
    if b.size != k * n:
        raise ValueError(f"matmul: operand b has {b.size} elements, shape needs {k * n}")
    out = np.empty(m * n, dtype=np.float32)
    lib().or_matmul(_p(a), _p(b), m, k, n, _p(out), threads)
    return out


def matmul_tuned(a, b, m: int, k: int, n: int, threads: int = 1) -> np.ndarray:
    """`matmul_tuned` (ferrum_ref/src/kernels/tuned.rs:L99-L134): cache panels and a 4 x 8 register tile."""
    a, b = _f32(a), _f32(b)
    out = np.empty(m * n, dtype=np.float32)
    lib().or_matmul_tuned(_p(a), _p(b), m, k, n, _p(out), threads)
    return out


def set_tuned(on: bool):
    """Model passes multiply with the tuned kernel (the all-cores speed baseline) or the simple one."""
    lib().or_set_tuned(1 if on else 0)


def rand_vec(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().or_rand_vec(n, seed, _p(out))
    return out


def gelu(x: float) -> float:
    return lib().or_gelu(C.c_float(x))


def silu(x: float) -> float:
    return lib().or_silu(C.c_float(x))


def layernorm(x, g, b, rows: int, cols: int) -> np.ndarray:
    x, g, b = _f32(x).reshape(-1), _f32(g), _f32(b)
    y = np.empty_like(x)
    lib().or_layernorm(_p(x), _p(g), _p(b), rows, cols, _p(y))
    return y


def rmsnorm(x, g, rows: int, cols: int, eps: float) -> np.ndarray:
    x, g = _f32(x).reshape(-1), _f32(g)
    y = np.empty_like(x)
    lib().or_rmsnorm(_p(x), _p(g), rows, cols, C.c_float(eps), _p(y))
    return y


def rope_tables(start: int, n: int, rope_dim: int, base: float, freq_factors=None, linear: float = 1.0):
    half = rope_dim // 2
    cos, sin = np.empty(n * half, dtype=np.float32), np.empty(n * half, dtype=np.float32)
    ff = None if freq_factors is None else _f32(freq_factors)
    lib().or_rope_tables(start, n, rope_dim, C.c_float(base), None if ff is None else _p(ff),
                         0 if ff is None else ff.size, C.c_float(linear), _p(cos), _p(sin))
    return cos, sin


def apply_rope(x, rows, heads, hd, rope_dim, cos, sin, rope_type) -> np.ndarray:
    x = _f32(x).reshape(-1).copy()
    cos, sin = _f32(cos), _f32(sin)
    lib().or_apply_rope(_p(x), rows, heads, hd, rope_dim, _p(cos), _p(sin), rope_type)
    return x


def attend_row(q, k, v, length, heads, kv_heads, hd) -> np.ndarray:
    q, k, v = _f32(q).reshape(-1), _f32(k).reshape(-1), _f32(v).reshape(-1)
    out = np.empty(heads * hd, dtype=np.float32)
    lib().or_attend_row(_p(q), _p(k), _p(v), length, heads, kv_heads, hd, _p(out))
    return out


def attention(q, k, v, batch, t, heads, hd) -> np.ndarray:
    q, k, v = _f32(q).reshape(-1), _f32(k).reshape(-1), _f32(v).reshape(-1)
    out = np.empty(batch * t * heads * hd, dtype=np.float32)
    lib().or_attention(_p(q), _p(k), _p(v), batch, t, heads, hd, _p(out))
    return out


def score(logits, targets, vocab: int):
    lg = _f32(logits).reshape(-1)
    tg = np.ascontiguousarray(targets, dtype=np.int32)
    lp, gr = np.empty(tg.size, dtype=np.float32), np.empty(tg.size, dtype=np.uint8)
    lib().or_score(_p(lg), _p(tg), tg.size, vocab, _p(lp), _p(gr))
    return lp, gr.astype(bool)


def logprobs_f64(logits, targets, vocab: int):
    lg = _f32(logits).reshape(-1)
    tg = np.ascontiguousarray(targets, dtype=np.int32)
    lp, gr = np.empty(tg.size, dtype=np.float64), np.empty(tg.size, dtype=np.uint8)
    lib().or_logprobs_f64(_p(lg), _p(tg), tg.size, vocab, _p(lp), _p(gr))
    return lp, gr.astype(bool)


def argmax(v) -> int:
    v = _f32(v).reshape(-1)
    return lib().or_argmax(_p(v), v.size)


def sample(logits, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, recent=(), rng=None) -> int:
    """`ferrum_model::sampling::sample` (sampling.rs:L42-L100); `rng` is an `Rng` and advances by one draw
    unless the call is greedy or has no candidate."""
    v = _f32(logits).reshape(-1)
    rec = np.ascontiguousarray(np.asarray(list(recent), dtype=np.int64))
    state = rng.s if rng is not None else C.c_uint64(lib().or_rng_new(1))
    return lib().or_sample(_p(v), v.size, float(temperature), int(top_k), float(top_p), float(repetition_penalty),
                           rec.ctypes.data if rec.size else None, rec.size, C.byref(state))


class Rng:
    """`ferrum_ref::rng::Rng` (kernels/rng.rs:L7-L41)."""

    def __init__(self, seed: int):
        self.s = C.c_uint64(lib().or_rng_new(seed))

    def next_u64(self) -> int:
        return lib().or_rng_next_u64(C.byref(self.s))

    def next_f32(self) -> float:
        return lib().or_rng_next_f32(C.byref(self.s))

    def below(self, n: int) -> int:
        return lib().or_rng_below(C.byref(self.s), n)


# ---- models --------------------------------------------------------------------------------

def dequantised_llama(m: Llama, kind: int, snap_embedding: bool = True) -> Llama:
    """The f32 model a quantised run computes with.

    Block matrices and head are snapped as `dequantised()` does (models/llama/mod.rs:L188-L213).
    With `snap_embedding` the token table is also round-tripped along its rows, which is what
    loading a Q8_0/Q4_0 GGUF gives (gguf/llama/mod.rs:L297-L316); a tied head is then rebuilt as
    the transpose of the snapped table, which equals its own snap.
    """
    c = m.cfg
    blocks = []
    for b in m.blocks:
        kw = {f: getattr(b, f) for f in _ffi.LLAMA_BLOCK_FIELDS}
        for name in LLAMA_MATS:
            k, n = m.mat_shape(name)
            kw[name] = snap_matrix(kind, kw[name], k, n)
        blocks.append(LlamaBlock(**kw))
    tok = snap_rows(kind, m.tok) if snap_embedding and c.dim % 32 == 0 else _f32(m.tok)
    if m.tied:
        head = transpose(tok, c.vocab, c.dim)
    else:
        head = snap_matrix(kind, m.head, c.dim, c.vocab)
    return Llama(c, tok, blocks, _f32(m.out_norm), head, m.tied)


def dequantised_gpt2(m: Gpt2, kind: int, tied: bool = False, snap_embedding: bool = True) -> Gpt2:
    """GPT-2 counterpart (the reference's CPU form is `Gpt2::fake_quantize`, training/qat.rs:L56-L76):
    token embedding, block matrices and head snapped; positions, biases and norms stay f32."""
    c = m.cfg
    blocks = []
    for b in m.blocks:
        kw = {f: getattr(b, f) for f in _ffi.GPT2_BLOCK_FIELDS}
        for name in GPT2_MATS:
            k, n = m.mat_shape(name)
            kw[name] = snap_matrix(kind, kw[name], k, n)
        blocks.append(Gpt2Block(**kw))
    tok = snap_rows(kind, m.tok) if snap_embedding and c.dim % 32 == 0 else _f32(m.tok)
    head = transpose(tok, c.vocab, c.dim) if tied else snap_matrix(kind, m.head, c.dim, c.vocab)
    return Gpt2(c, tok, _f32(m.pos), blocks, _f32(m.lnf_g), _f32(m.lnf_b), head)


class OracleLlama:
    """`ferrum_ref::llama::Llama` forward passes with an owned `Cache` (models/llama/mod.rs:L186-L259)."""

    def __init__(self, model: Llama, threads: int = 1):
        self.model = model
        cfg, w = model.c_structs()
        self.h = lib().or_llama_create(C.byref(cfg), C.byref(w), threads)
        self.vocab = model.cfg.vocab

    def __del__(self):
        if getattr(self, "h", None):
            lib().or_llama_destroy(self.h)
            self.h = None

    def reset(self):
        lib().or_llama_reset(self.h)

    def pos(self) -> int:
        return lib().or_llama_pos(self.h)

    def feed(self, token: int) -> np.ndarray:
        out = np.empty(self.vocab, dtype=np.float32)
        rc = lib().or_llama_feed(self.h, int(token), _p(out))
        _raise(rc, self.model.cfg, token)
        return out

    def extend(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(ids.size * self.vocab, dtype=np.float32)
        rc = lib().or_llama_extend(self.h, _p(ids), ids.size, _p(out))
        _raise(rc, self.model.cfg, None)
        return out.reshape(ids.size, self.vocab)

    def extend_last(self, ids) -> np.ndarray:
        """`extend`, returning the logits of the last new position only."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(self.vocab, dtype=np.float32)
        rc = lib().or_llama_extend_last(self.h, _p(ids), ids.size, _p(out))
        _raise(rc, self.model.cfg, None)
        return out

    def forward_logits(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(ids.size * self.vocab, dtype=np.float32)
        rc = lib().or_llama_forward_logits(self.h, _p(ids), ids.size, _p(out))
        if rc == _ffi.FC_ERR_SHAPE:
            raise ValueError(f"sequence length {ids.size} must be in 1..={self.model.cfg.ctx}")
        _raise(rc, self.model.cfg, None)
        return out.reshape(ids.size, self.vocab)

    def score(self, ids):
        """`GpuLlama::score` semantics on the CPU: forward over ids[:-1], nn::score vs ids[1:]."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lg = self.forward_logits(ids[:-1])
        return score(lg, ids[1:], self.vocab)


class OracleGpt2:
    """`ferrum_ref::gpt2::Gpt2::{forward_logits, feed}` (models/gpt2/mod.rs:L203-L230, decode.rs:L57-L116)."""

    def __init__(self, model: Gpt2, threads: int = 1):
        self.model = model
        cfg, w = model.c_structs()
        self.h = lib().or_gpt2_create(C.byref(cfg), C.byref(w), threads)
        self.vocab = model.cfg.vocab

    def __del__(self):
        if getattr(self, "h", None):
            lib().or_gpt2_destroy(self.h)
            self.h = None

    def reset(self):
        lib().or_gpt2_reset(self.h)

    def pos(self) -> int:
        return lib().or_gpt2_pos(self.h)

    def feed(self, token: int) -> np.ndarray:
        out = np.empty(self.vocab, dtype=np.float32)
        rc = lib().or_gpt2_feed(self.h, int(token), _p(out))
        _raise(rc, self.model.cfg, token)
        return out

    def forward_logits(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(ids.size * self.vocab, dtype=np.float32)
        rc = lib().or_gpt2_forward_logits(self.h, _p(ids), ids.size, _p(out))
        if rc == _ffi.FC_ERR_SHAPE:
            raise ValueError(f"sequence length {ids.size} must be in 1..={self.model.cfg.ctx}")
        _raise(rc, self.model.cfg, None)
        return out.reshape(ids.size, self.vocab)

    def score(self, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lg = self.forward_logits(ids[:-1])
        return score(lg, ids[1:], self.vocab)


def _raise(rc: int, cfg, token):
    if rc == _ffi.FC_OK:
        return
    if rc == _ffi.FC_ERR_CONTEXT_FULL:
        raise RuntimeError(f"context of {cfg.ctx} tokens is full")
    if rc == _ffi.FC_ERR_RANGE:
        raise IndexError(f"token {token} is out of range for vocab {cfg.vocab}")
    raise RuntimeError(f"oracle error {rc}")


def max_rel_err(got, want) -> float:
    """`ferrum_wgpu::tolerance::max_rel_err` (tolerance.rs:L14-L26): max |g-w| / max(|w|, 1)."""
    g, w = np.asarray(got, dtype=np.float32).reshape(-1), np.asarray(want, dtype=np.float32).reshape(-1)
    if g.size != w.size:
        return float("inf")
    if g.size == 0:
        return 0.0
    e = np.abs(g - w) / np.maximum(np.abs(w), np.float32(1.0))
    if np.isnan(e).any():
        return float("inf")
    return float(e.max())
