"""Resident models: the host-side mirror of `GpuLlama` / `GpuGpt2`
(ferrum_wgpu/src/models/llama/{mod,forward}.rs, models/gpt2.rs): `feed`, `forward_all`, `score`,
`reset`, `pos`, `config`, `quant`, with multi-stream decode and batched scoring added."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .device import CudaError, Device
from .hostmodel import Gpt2, Llama
from .quant import Mode, QKind


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


class ResidentModel:
    def __init__(self, dev: Device, handle, cfg, quant: QKind | None, max_streams: int):
        self.dev, self._h, self._lib = dev, handle, _ffi.load()
        self.cfg, self._quant, self.max_streams = cfg, quant, max_streams
        dev.adopt(self)

    # -- reference interface ------------------------------------------------------------------
    def config(self):
        return self.cfg

    def quant(self):
        """The quantisation requested at upload (ineligible matrices stay f32)."""
        return self._quant

    def pos(self, stream: int = 0) -> int:
        p = C.c_uint32()
        self.dev.check(self._lib.fc_model_pos(self._h, stream, C.byref(p)))
        return p.value

    def reset(self, stream: int = 0):
        self.dev.check(self._lib.fc_model_reset(self._h, stream))

    def feed(self, token: int, stream: int = 0) -> np.ndarray:
        """Consume one token at the next position and return its next-token logits row."""
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self.dev.check(self._lib.fc_model_feed(self._h, stream, int(token), out.ctypes.data, None))
        return out

    def feed_greedy(self, token: int, stream: int = 0) -> int:
        """`feed` with the argmax taken on the device (first maximum); no logits leave the GPU."""
        a = C.c_int32()
        self.dev.check(self._lib.fc_model_feed(self._h, stream, int(token), None, C.byref(a)))
        return a.value

    def topk(self, k: int, row: int = 0, repetition_penalty: float = 1.0, recent=()):
        """The candidates `sampling::sample` keeps for top_k = k from the logits row the last decode step left on
        the device, in its order (descending, ties lower index first, NaN dropped), after its repetition
        penalty over `recent`: (indices int32[n], values float32[n]) with n <= k. No logits row is read back."""
        idx = np.empty(k, dtype=np.int32)
        val = np.empty(k, dtype=np.float32)
        rec = np.ascontiguousarray(np.asarray(list(recent), dtype=np.int32))
        n = C.c_uint32()
        self.dev.check(self._lib.fc_model_topk(self._h, row, k, float(repetition_penalty),
                                               rec.ctypes.data if rec.size else None, rec.size, idx.ctypes.data,
                                               val.ctypes.data, C.byref(n)))
        return idx[:n.value], val[:n.value]

    def feed_batch(self, tokens, streams=None, want_logits: bool = False):
        """One decode step for several streams; returns (argmax[n], logits[n, vocab] | None)."""
        tokens = _i32(tokens)
        n = tokens.size
        streams = np.arange(n, dtype=np.uint32) if streams is None else np.ascontiguousarray(streams, dtype=np.uint32)
        am = np.empty(n, dtype=np.int32)
        lg = np.empty((n, self.cfg.vocab), dtype=np.float32) if want_logits else None
        self.dev.check(self._lib.fc_model_feed_batch(self._h, n, streams.ctypes.data, tokens.ctypes.data,
                                                     lg.ctypes.data if want_logits else None, am.ctypes.data))
        return am, lg

    def decode_greedy(self, tokens, steps: int, streams=None) -> np.ndarray:
        """`steps` greedy steps of several streams in one call, chained on the device: step 0 feeds `tokens`,
        every further step the previous picks. Returns the picks `[steps, n]` - what `steps` calls of
        `feed_batch` would return."""
        tokens = _i32(tokens)
        n = tokens.size
        streams = np.arange(n, dtype=np.uint32) if streams is None else np.ascontiguousarray(streams, dtype=np.uint32)
        out = np.empty((steps, n), dtype=np.int32)
        self.dev.check(self._lib.fc_model_decode_greedy(self._h, n, streams.ctypes.data, tokens.ctypes.data, steps,
                                                        out.ctypes.data))
        return out

    def prefill(self, ids, stream: int = 0, mode: Mode = Mode.EXACT_F32) -> np.ndarray:
        """Feed a whole prompt in one batched pass; returns the last position's logits."""
        ids = _i32(ids)
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self.dev.check(self._lib.fc_model_prefill(self._h, stream, ids.ctypes.data, ids.size, out.ctypes.data,
                                                  None, int(mode)))
        return out

    def forward_all(self, ids, mode: Mode = Mode.EXACT_F32) -> np.ndarray:
        """Stateless full causal forward; every position's logits `[len, vocab]`."""
        ids = _i32(ids)
        out = np.empty((ids.size, self.cfg.vocab), dtype=np.float32)
        self.dev.check(self._lib.fc_model_forward_all(self._h, ids.ctypes.data, ids.size, out.ctypes.data, int(mode)))
        return out

    def score(self, ids, mode: Mode = Mode.EXACT_F32):
        """For each i < len-1: (log-probability of ids[i+1] given ids[..=i], it is the first argmax)."""
        ids = _i32(ids).reshape(1, -1)
        lp, gr, _ = self.score_batch(ids, mode)
        return lp[0], gr[0]

    def score_batch(self, ids, mode: Mode = Mode.EXACT_F32):
        """Scores `[n_seqs, seq_len]` ids: (logprob[n, L-1], greedy[n, L-1], nll_sum[n] in f64)."""
        ids = _i32(ids)
        if ids.ndim != 2:
            raise CudaError(_ffi.FC_ERR_SHAPE, "score_batch takes [n_seqs, seq_len] ids")
        n, L = ids.shape
        if L < 2:
            raise CudaError(_ffi.FC_ERR_SHAPE, "scoring needs at least 2 tokens")
        lp = np.empty((n, L - 1), dtype=np.float32)
        gr = np.empty((n, L - 1), dtype=np.uint8)
        nll = np.empty(n, dtype=np.float64)
        self.dev.check(self._lib.fc_model_score(self._h, ids.ctypes.data, n, L, int(mode), lp.ctypes.data,
                                                gr.ctypes.data, nll.ctypes.data))
        return lp, gr.astype(bool), nll

    def score_ragged(self, seqs, mode: Mode = Mode.EXACT_F32):
        """Scores sequences of different lengths in batched passes (the server's concurrent requests,
        serving/routes.rs:L301-L309): per sequence (logprob[len-1], greedy[len-1]) as `score` gives them, and the
        f64 NLL sums `[n]`."""
        seqs = [_i32(s).reshape(-1) for s in seqs]
        offsets = np.zeros(len(seqs) + 1, dtype=np.uint32)
        offsets[1:] = np.cumsum([s.size for s in seqs])
        flat = np.concatenate(seqs) if seqs else np.zeros(0, dtype=np.int32)
        n_out = max(int(offsets[-1]) - len(seqs), 0)
        lp = np.empty(n_out, dtype=np.float32)
        gr = np.empty(n_out, dtype=np.uint8)
        nll = np.empty(len(seqs), dtype=np.float64)
        self.dev.check(self._lib.fc_model_score_ragged(self._h, flat.ctypes.data, offsets.ctypes.data, len(seqs), int(mode),
                                                       lp.ctypes.data, gr.ctypes.data, nll.ctypes.data))
        cut = (offsets - np.arange(len(seqs) + 1, dtype=np.uint32)).astype(np.int64)
        return ([lp[cut[i]:cut[i + 1]] for i in range(len(seqs))],
                [gr[cut[i]:cut[i + 1]].astype(bool) for i in range(len(seqs))], nll)

    def token_logprobs(self, streams, from_=None, mode: Mode = Mode.EXACT_F32):
        """`serving::score::token_logprobs` (serving/score.rs:L27-L49) for several id streams at once, every
        window of every stream in one ragged batch: [(logprob f64, n_tokens, greedy)] per stream."""
        streams = [_i32(s).reshape(-1) for s in streams]
        offsets = np.zeros(len(streams) + 1, dtype=np.uint32)
        offsets[1:] = np.cumsum([s.size for s in streams])
        flat = np.concatenate(streams) if streams else np.zeros(0, dtype=np.int32)
        frm = None if from_ is None else np.ascontiguousarray(from_, dtype=np.uint32)
        lp = np.empty(len(streams), dtype=np.float64)
        nt = np.empty(len(streams), dtype=np.uint64)
        gr = np.empty(len(streams), dtype=np.uint8)
        self.dev.check(self._lib.fc_model_token_logprobs(self._h, flat.ctypes.data, offsets.ctypes.data,
                                                         None if frm is None else frm.ctypes.data, len(streams),
                                                         int(mode), lp.ctypes.data, nt.ctypes.data, gr.ctypes.data))
        return [(float(lp[i]), int(nt[i]), bool(gr[i])) for i in range(len(streams))]

    # -- device-pointer variants (benchmark, multi-GPU) -----------------------------------------
    def score_dev(self, ids_ptr: int, n_seqs: int, seq_len: int, mode: Mode, logprob_ptr: int, greedy_ptr: int,
                  nll_ptr: int):
        self.dev.check(self._lib.fc_model_score_dev(self._h, ids_ptr, n_seqs, seq_len, int(mode), logprob_ptr or None,
                                                    greedy_ptr or None, nll_ptr or None))

    def set_head_shard(self, shard: int, n_shards: int):
        self.dev.check(self._lib.fc_model_set_head_shard(self._h, shard, n_shards))

    def trunk_dev(self, ids_ptr: int, n_seqs: int, seq_len: int, mode: Mode, hidden_ptr: int):
        self.dev.check(self._lib.fc_model_trunk_dev(self._h, ids_ptr, n_seqs, seq_len, int(mode), hidden_ptr))

    def head_partial_dev(self, hidden_ptr: int, targets_ptr: int, rows: int, mode: Mode, partial_ptr: int):
        self.dev.check(self._lib.fc_model_head_partial_dev(self._h, hidden_ptr, targets_ptr, rows, int(mode),
                                                           partial_ptr))

    def weight_bytes(self) -> int:
        b = C.c_uint64()
        self.dev.check(self._lib.fc_model_info(self._h, None, None, None, None, C.byref(b)))
        return b.value

    def close(self):
        if self._h:
            self._lib.fc_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _kind(quant) -> int:
    return int(QKind.F32 if quant is None else quant)


class CudaLlama(ResidentModel):
    """`GpuLlama::new(gpu, model, quant, budget)` (models/llama/mod.rs:L219-L314). `packed` (from `pack_model`, or
    the tensors of a quantised file): matrices that arrive as GGUF blocks of `packed_kind` (default `quant`) and are
    repacked as they are."""

    def __init__(self, dev: Device, model: Llama, quant: QKind | None = None, budget: int | None = None,
                 max_streams: int = 1, packed: dict | None = None, packed_kind: QKind | None = None):
        h = C.c_void_p()
        if packed is None:
            cfg, w = model.c_structs()
            dev.check(_ffi.load().fc_llama_create(dev.handle, C.byref(cfg), C.byref(w), _kind(quant), max_streams,
                                                  budget or 0, C.byref(h)))
        else:
            cfg, w, keep = _tensor_structs(model, packed_kind or quant, packed)
            dev.check(_ffi.load().fc_llama_create_from_tensors(dev.handle, C.byref(cfg), C.byref(w), _kind(quant),
                                                               max_streams, budget or 0, C.byref(h)))
            del keep
        super().__init__(dev, h, model.cfg, quant, max_streams)


def pack_model(dev: Device, model, kind: QKind) -> dict:
    """The model's matrices as GGUF block bytes, the way a quantised file holds them (token table, block matrices
    and head; ferrum_model/src/gguf/llama/mod.rs:L297-L316): {name or (layer, name): uint8 array}. Encoded by the
    device encoder, which is bit-identical to `ferrum_gguf::quant::encode`."""
    from .quant import upload_quantised
    c = model.cfg
    out = {}

    def blocks_of(w, k, n):
        q = upload_quantised(dev, kind, w, k, n)
        b = q.blocks()
        q.close()
        return b

    # the table is quantised along its rows of `dim`: as an [in, out] matrix that is its transpose
    tok_t = np.ascontiguousarray(np.asarray(model.tok, dtype=np.float32).reshape(c.vocab, c.dim).T)
    out["tok"] = blocks_of(tok_t, c.dim, c.vocab)
    out["head"] = blocks_of(model.head, c.dim, c.vocab)
    names = _ffi.LLAMA_MATS if isinstance(model, Llama) else _ffi.GPT2_MATS
    for i, b in enumerate(model.blocks):
        for name in names:
            k, n = model.mat_shape(name)
            out[(i, name)] = blocks_of(getattr(b, name), k, n)
    return out


def _tensor_structs(model, kind: QKind, packed: dict):
    """(config, FcLlamaTensors | FcGpt2Tensors, keep-alive list) with every matrix found in `packed` handed over as
    blocks of `kind` and the rest as f32."""
    c = model.cfg
    keep = []

    def tensor(key, f32_array):
        if key in packed:
            a = np.ascontiguousarray(packed[key], dtype=np.uint8)
            keep.append(a)
            return _ffi.FcTensor(a.ctypes.data, int(kind))
        a = np.ascontiguousarray(f32_array, dtype=np.float32)
        keep.append(a)
        return _ffi.FcTensor(a.ctypes.data, _ffi.FC_F32)

    def f32p(a):
        if a is None:
            return None
        a = np.ascontiguousarray(a, dtype=np.float32)
        keep.append(a)
        return a.ctypes.data_as(_ffi.f32p)

    llama = isinstance(model, Llama)
    cfg, _ = model.c_structs()
    mats = _ffi.LLAMA_MATS if llama else _ffi.GPT2_MATS
    fields = _ffi.LLAMA_BLOCK_FIELDS if llama else _ffi.GPT2_BLOCK_FIELDS
    arr = ((_ffi.FcLlamaBlockT if llama else _ffi.FcGpt2BlockT) * c.layers)()
    keep.append(arr)
    for i, b in enumerate(model.blocks):
        for name in fields:
            if name in mats:
                setattr(arr[i], name, tensor((i, name), getattr(b, name)))
            else:
                setattr(arr[i], name, f32p(getattr(b, name)))
    if llama:
        w = _ffi.FcLlamaTensors(tensor("tok", model.tok), arr, f32p(model.out_norm), tensor("head", model.head))
    else:
        w = _ffi.FcGpt2Tensors(tensor("tok", model.tok), f32p(model.pos), arr, f32p(model.lnf_g), f32p(model.lnf_b),
                               tensor("head", model.head))
    return cfg, w, keep


class CudaGpt2(ResidentModel):
    """`GpuGpt2::new` (models/gpt2.rs:L134-L190), with quantised weights added."""

    def __init__(self, dev: Device, model: Gpt2, quant: QKind | None = None, budget: int | None = None,
                 max_streams: int = 1, packed: dict | None = None, packed_kind: QKind | None = None):
        h = C.c_void_p()
        if packed is None:
            cfg, w = model.c_structs()
            dev.check(_ffi.load().fc_gpt2_create(dev.handle, C.byref(cfg), C.byref(w), _kind(quant), max_streams,
                                                 budget or 0, C.byref(h)))
        else:
            cfg, w, keep = _tensor_structs(model, packed_kind or quant, packed)
            dev.check(_ffi.load().fc_gpt2_create_from_tensors(dev.handle, C.byref(cfg), C.byref(w), _kind(quant),
                                                              max_streams, budget or 0, C.byref(h)))
            del keep
        super().__init__(dev, h, model.cfg, quant, max_streams)


def plan_bytes(cfg, quant: QKind | None = None, max_streams: int = 1) -> int:
    """`models::llama::plan` total (models/llama/mod.rs:L108-L182): device bytes a model needs."""
    lib = _ffi.load()
    if hasattr(cfg, "kv_heads"):
        c = _ffi.FcLlamaConfig(cfg.vocab, cfg.ctx, cfg.dim, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.layers,
                               cfg.hidden, cfg.rope_dim, cfg.rope_type, cfg.rope_base, cfg.eps,
                               cfg.rope_linear_factor, 0, None, 0)
        return lib.fc_llama_plan_bytes(C.byref(c), _kind(quant), max_streams)
    c = _ffi.FcGpt2Config(cfg.vocab, cfg.ctx, cfg.dim, cfg.heads, cfg.layers, cfg.hidden)
    return lib.fc_gpt2_plan_bytes(C.byref(c), _kind(quant), max_streams)
