"""Scoring over 1/2/4/8 GPUs of one box: one process per GPU, each a rank of an `FcGroup` of the C ABI
(`fc_group_create` / `fc_group_score`), which owns the NCCL communicators and does the whole exchange.
This module only carries the rendezvous token between the processes (a `torch.distributed` broadcast) and
mirrors the partition rules for the host-side tests.

Sequences are independent (so are the server's sliding windows, serving/score.rs:L27-L49), so the default
partition is by sequence with no data-path collective: every rank holds a replica of the packed weights and
scores its own sequences; only the per-sequence NLL sums are combined at the end. With `vocab_shards > 1` the
ranks form `world / vocab_shards` sequence groups of `vocab_shards` ranks that split the head by vocabulary
rows - `Lin::Sharded`'s column blocks (ferrum_wgpu/src/models/llama/lin.rs:L41-L53,L76-L90) on different GPUs.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _ffi
from .quant import Mode, QKind

ID_BYTES = 128


def seq_slice(n_seqs: int, rank: int, world: int) -> range:
    """Sequences `rank, rank + world, ...` of `n_seqs` (`fc_group_sequences`)."""
    return range(rank, n_seqs, world)


def vocab_rows(vocab: int, shard: int, n_shards: int):
    """Head rows of one shard: ceil(vocab / n_shards) each, the last one short (may be empty)."""
    per = -(-vocab // n_shards)
    v0 = min(per * shard, vocab)
    return v0, min(v0 + per, vocab)


def layout(world: int, vocab_shards: int):
    """(sequence groups, ranks of each group): rank r is shard r % vocab_shards of group r // vocab_shards."""
    if vocab_shards < 1 or world % vocab_shards:
        raise ValueError(f"{world} ranks cannot form groups of {vocab_shards} vocabulary shards")
    groups = world // vocab_shards
    return groups, [list(range(g * vocab_shards, (g + 1) * vocab_shards)) for g in range(groups)]


def exchange_id(make) -> bytes:
    """The rendezvous token of `fc_group_unique_id`, made on rank 0 and broadcast over the process group that
    `torch.distributed` already has (any backend); a single process just makes it."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return make()
    box = [make() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class GroupScorer:
    """One rank of a multi-GPU scoring job. Construct after `torch.distributed.init_process_group` (or alone)."""

    def __init__(self, model, quant: QKind, vocab_shards: int = 1, mode: Mode = Mode.TENSOR_F16):
        import torch.distributed as dist
        from .device import Device
        from .hostmodel import Llama
        from .resident import CudaGpt2, CudaLlama

        self._lib = _ffi.load()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.local = int(os.environ.get("LOCAL_RANK", self.rank))
        self.vocab_shards, self.mode = vocab_shards, mode
        self.n_groups, _ = layout(self.world, vocab_shards)
        self.group_id, self.shard = self.rank // vocab_shards, self.rank % vocab_shards
        self.dev = Device.open(self.local)
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        self.model = cls(self.dev, model, quant)
        self.cfg = model.cfg

        def make() -> bytes:
            buf = (C.c_uint8 * ID_BYTES)()
            self.dev.check(self._lib.fc_group_unique_id(buf, ID_BYTES))
            return bytes(buf)

        token = exchange_id(make)
        buf = (C.c_uint8 * ID_BYTES).from_buffer_copy(token)
        h = C.c_void_p()
        self.dev.check(self._lib.fc_group_create(self.dev.handle, self.model._h, self.rank, self.world, vocab_shards,
                                                 buf, ID_BYTES, C.byref(h)))
        self._h = h

    def close(self):
        if self._h:
            self._lib.fc_group_destroy(self._h)
            self._h = None
        self.model.close()
        self.dev.close()

    def score(self, ids: np.ndarray) -> np.ndarray:
        """Total NLL of every sequence of `ids` ([n_seqs, seq_len] int32, the same array on every rank);
        returns the `[n_seqs]` f64 sums on every rank."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        n_seqs, seq_len = ids.shape
        out = np.zeros(n_seqs, dtype=np.float64)
        self.dev.check(self._lib.fc_group_score(self._h, ids.ctypes.data, n_seqs, seq_len, int(self.mode),
                                                out.ctypes.data))
        return out

    def exchange_ms(self):
        """Device milliseconds of the last `score` call's exchanges: (hidden states, partials, NLL sums)."""
        ms = (C.c_float * 3)()
        self.dev.check(self._lib.fc_group_last_exchange_ms(self._h, ms))
        return tuple(ms)
