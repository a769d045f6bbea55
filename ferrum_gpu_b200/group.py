"""Scoring over 1/2/4/8 GPUs of one box: one process per GPU, `torch.distributed` for the plumbing.

Sequences are independent (so are the server's sliding windows, serving/score.rs:L27-L49), so the
default partition is by sequence with no data-path collective: every rank holds a replica of the packed
weights and scores its own sequences; only the per-sequence NLL sums are gathered at the end.

With `vocab_shards > 1` the ranks form `world / vocab_shards` sequence groups of `vocab_shards` ranks. The
precedent is `Lin::Sharded`, which splits a `[k, n]` weight by output columns, each block multiplied on
its own (ferrum_wgpu/src/models/llama/lin.rs:L41-L53,L76-L90); here the blocks of the head live on
different GPUs. Inside a group the trunk is sequence-parallel, the final hidden states are all-gathered
into local HBM (NCCL), every rank runs the fused head over its vocabulary rows and the per-row
(max, sum-exp, target logit, first argmax) partials are all-gathered and merged: one exchange of hidden
states and one of 16 bytes per row. Remote data always lands in local memory before a kernel reads it.
"""
from __future__ import annotations

import os

import numpy as np

from .quant import Mode, QKind


def seq_slice(n_seqs: int, rank: int, world: int) -> range:
    """Sequences `rank, rank + world, ...` of `n_seqs`."""
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


class GroupScorer:
    """One rank of a multi-GPU scoring job. Construct after `torch.distributed.init_process_group`."""

    def __init__(self, model, quant: QKind, vocab_shards: int = 1, mode: Mode = Mode.TENSOR_F16):
        import torch
        import torch.distributed as dist
        from .device import Device
        from .hostmodel import Llama
        from .resident import CudaGpt2, CudaLlama

        self.torch, self.dist = torch, dist
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.local = int(os.environ.get("LOCAL_RANK", self.rank))
        self.vocab_shards, self.mode = vocab_shards, mode
        self.n_groups, groups = layout(self.world, vocab_shards)
        self.group_id, self.shard = self.rank // vocab_shards, self.rank % vocab_shards
        self.pg = None
        if vocab_shards > 1:
            for ranks in groups:  # every rank must create every group
                pg = dist.new_group(ranks)
                if self.rank in ranks:
                    self.pg = pg
        torch.cuda.set_device(self.local)
        self.dev = Device.open(self.local)
        self.stream = torch.cuda.ExternalStream(self.dev.stream(), device=self.local)
        cls = CudaLlama if isinstance(model, Llama) else CudaGpt2
        self.model = cls(self.dev, model, quant)
        self.cfg = model.cfg
        if vocab_shards > 1:
            self.model.set_head_shard(self.shard, vocab_shards)

    def close(self):
        self.model.close()
        self.dev.close()

    def score(self, ids: np.ndarray) -> np.ndarray:
        """Total NLL of every sequence of `ids` ([n_seqs, seq_len] int32, the same array on every rank);
        returns the `[n_seqs]` f64 sums on every rank."""
        torch, dist = self.torch, self.dist
        n_seqs, seq_len = ids.shape
        device = f"cuda:{self.local}"
        out = torch.zeros(n_seqs, dtype=torch.float64, device=device)
        with torch.cuda.stream(self.stream):
            if self.vocab_shards == 1:
                mine = list(seq_slice(n_seqs, self.rank, self.world))
                if mine:
                    d_ids = torch.from_numpy(np.ascontiguousarray(ids[mine])).to(device)
                    nll = torch.zeros(len(mine), dtype=torch.float64, device=device)
                    self.model.score_dev(d_ids.data_ptr(), len(mine), seq_len, self.mode, 0, 0, nll.data_ptr())
                    out[torch.tensor(mine, device=device)] = nll
            else:
                self._score_split(ids, out)
            if self.world > 1:
                dist.all_reduce(out)  # disjoint slots: a sum is a gather
            self.stream.synchronize()
        return out.cpu().numpy()

    def _score_split(self, ids: np.ndarray, out):
        torch, dist = self.torch, self.dist
        device = f"cuda:{self.local}"
        n_seqs, seq_len = ids.shape
        t = seq_len - 1
        group_seqs = list(seq_slice(n_seqs, self.group_id, self.n_groups))
        if not group_seqs:
            return
        vs = self.vocab_shards
        per = -(-len(group_seqs) // vs)                      # sequences per rank inside the group (padded)
        padded = group_seqs + [group_seqs[-1]] * (per * vs - len(group_seqs))
        mine = padded[self.shard * per:(self.shard + 1) * per]
        half = self.mode == Mode.TENSOR_F16
        hdt = torch.float16 if half else torch.float32
        d_in = torch.from_numpy(np.ascontiguousarray(ids[mine][:, :t])).to(device)
        hidden = torch.empty(per * t, self.cfg.dim, dtype=hdt, device=device)
        self.model.trunk_dev(d_in.data_ptr(), per, t, self.mode, hidden.data_ptr())
        all_hidden = torch.empty(vs * per * t, self.cfg.dim, dtype=hdt, device=device)
        dist.all_gather_into_tensor(all_hidden, hidden, group=self.pg)      # lands in local HBM
        targets = torch.from_numpy(np.ascontiguousarray(ids[padded][:, 1:]).reshape(-1)).to(device)
        rows = vs * per * t
        partial = torch.empty(rows, 4, dtype=torch.float32, device=device)
        self.model.head_partial_dev(all_hidden.data_ptr(), targets.data_ptr(), rows, self.mode, partial.data_ptr())
        all_partial = torch.empty(vs, rows, 4, dtype=torch.float32, device=device)
        dist.all_gather_into_tensor(all_partial, partial, group=self.pg)
        lp = torch.empty(rows, dtype=torch.float32, device=device)
        nll = torch.empty(vs * per, dtype=torch.float64, device=device)
        from . import _ffi
        self.dev.check(_ffi.load().fc_score_combine_dev(self.dev.handle, all_partial.data_ptr(), vs, targets.data_ptr(),
                                                        vs * per, t, lp.data_ptr(), None, nll.data_ptr()))
        if self.shard == 0:  # one rank of the group reports its sequences
            idx = torch.tensor(group_seqs, device=device)
            out[idx] = nll[:len(group_seqs)]
