"""Host-side logic of the multi-GPU scoring driver on CPU: partitions, group layout, and the gather of
per-sequence sums over a world_size-2 gloo process group."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferrum_gpu_b200.group import layout, seq_slice, vocab_rows


def test_sequences_are_partitioned_exactly_once():
    for n, world in [(256, 1), (256, 2), (256, 8), (7, 4), (3, 8), (0, 2)]:
        seen = sorted(i for r in range(world) for i in seq_slice(n, r, world))
        assert seen == list(range(n))


def test_vocabulary_rows_cover_the_head_with_a_short_last_shard():
    for vocab, shards in [(50257, 2), (50257, 4), (50257, 8), (32000, 8), (17, 4), (5, 8)]:
        rows = [vocab_rows(vocab, s, shards) for s in range(shards)]
        assert rows[0][0] == 0 and rows[-1][1] == vocab
        for (a0, a1), (b0, b1) in zip(rows, rows[1:]):
            assert a1 == b0 and a0 <= a1
        assert max(v1 - v0 for v0, v1 in rows) == -(-vocab // shards)
    assert vocab_rows(50257, 1, 2) == (25129, 50257)  # uneven: 25129 + 25128


def test_group_layout():
    assert layout(8, 1) == (8, [[r] for r in range(8)])
    assert layout(8, 2) == (4, [[0, 1], [2, 3], [4, 5], [6, 7]])
    assert layout(8, 4) == (2, [[0, 1, 2, 3], [4, 5, 6, 7]])
    with pytest.raises(ValueError):
        layout(8, 3)


def _worker(rank, world, port, n_seqs, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # what GroupScorer.score does around the device work: own slots filled, the rest zero, then a sum
        truth = torch.arange(n_seqs, dtype=torch.float64) * 1.5 + 0.25
        out = torch.zeros(n_seqs, dtype=torch.float64)
        mine = list(seq_slice(n_seqs, rank, world))
        out[mine] = truth[mine]
        dist.all_reduce(out)
        ok = bool(torch.equal(out, truth))
        # the vocabulary-split exchange: each rank contributes its shard's (max, sumexp, target, argmax)
        rows = 5
        logits = torch.from_numpy(np.random.default_rng(3).standard_normal((rows, 11)).astype(np.float32))
        v0, v1 = vocab_rows(11, rank, world)
        part = torch.stack([logits[:, v0:v1].max(1).values,
                            torch.exp(logits[:, v0:v1] - logits[:, v0:v1].max(1, keepdim=True).values).sum(1),
                            torch.full((rows,), float("-inf")), (logits[:, v0:v1].argmax(1) + v0).float()], dim=1)
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part.contiguous())
        mx = torch.stack([g[:, 0] for g in gathered]).max(0).values
        se = sum(g[:, 1] * torch.exp(g[:, 0] - mx) for g in gathered)
        lse = mx + torch.log(se)
        ok = ok and bool(torch.allclose(lse, torch.logsumexp(logits, 1), atol=1e-5))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_gather_and_split_head_exchange_over_gloo_world_size_2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 9, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
