"""Multi-GPU scoring (one process per GPU, NCCL): sequence sharding with a gathered NLL vector, and the
vocabulary-split head whose log-softmax is merged from per-shard (max, sum-exp, target, argmax)
partials. Both must reproduce the single-GPU result. Skipped on a box with one GPU."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _model():
    from ferrum_gpu_b200 import _ffi
    from ferrum_gpu_b200.hostmodel import LlamaConfig, random_llama
    cfg = LlamaConfig(vocab=104, ctx=160, dim=128, heads=2, kv_heads=1, head_dim=64, layers=2, hidden=192, rope_dim=64,
                      rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
    return cfg, random_llama(cfg, seed=5, std=0.05, gain_jitter=0.1)


def _ids(cfg, n=10, length=131):
    from ferrum_gpu_b200.hostmodel import random_tokens
    return np.stack([random_tokens(300 + i, length, cfg.vocab) for i in range(n)])


def _worker(rank, world, port, vocab_shards, mode_value, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from ferrum_gpu_b200 import Mode, QKind
    from ferrum_gpu_b200.group import GroupScorer
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # carries the rendezvous token only: the group owns its NCCL
    try:
        cfg, model = _model()
        gs = GroupScorer(model, QKind.Q4_0, vocab_shards=vocab_shards, mode=Mode(mode_value))
        nll = gs.score(_ids(cfg))
        gs.close()
        q.put((rank, nll.tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("vocab_shards", [1, 2])
@pytest.mark.parametrize("mode_name", ["EXACT_F32", "TENSOR_F16"])
def test_two_gpus_reproduce_the_single_gpu_scores(dev, vocab_shards, mode_name):
    import torch
    import torch.multiprocessing as mp
    from ferrum_gpu_b200 import CudaLlama, Mode, QKind
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mode = Mode[mode_name]
    cfg, model = _model()
    single = CudaLlama(dev, model, QKind.Q4_0)
    _, _, want = single.score_batch(_ids(cfg), mode)
    single.close()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, vocab_shards, int(mode), q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    tol = 1e-3 if mode == Mode.EXACT_F32 else 5e-2  # per-sequence NLL sums over 130 positions
    for r in range(2):
        got = np.array(results[r])
        assert np.abs(got - want).max() < tol, (vocab_shards, mode_name, r, np.abs(got - want).max())
    assert results[0] == results[1], "every rank holds the same gathered vector"
