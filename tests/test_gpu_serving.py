"""Scoring callers on the GPU: unequal-length batches, the sliding windows of a long id stream (both against the
CPU oracle, window by window), and a one-rank group of the C ABI (the NCCL path without a second GPU)."""
import numpy as np
import pytest

from ferrum_gpu_b200 import CudaLlama, Mode, QKind
from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.group import GroupScorer
from ferrum_gpu_b200.hostmodel import LlamaConfig, random_llama, random_tokens
from ferrum_gpu_b200.serving import ModelDecoder, rolling, token_logprobs, windows
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _model(ctx=48):
    cfg = LlamaConfig(vocab=97, ctx=ctx, dim=128, heads=2, kv_heads=1, head_dim=64, layers=2, hidden=192, rope_dim=64,
                      rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
    return cfg, random_llama(cfg, seed=21, std=0.2, gain_jitter=0.1)


def test_unequal_lengths_score_like_each_sequence_alone(dev):
    """serving/routes.rs:L301-L309 runs requests one after another; one batched pass must give every request
    what it would get alone (models/llama/tests.rs:L176-L194 bounds: 1e-4 per log-probability, same flags)."""
    cfg, m = _model()
    ref = orc.dequantised_llama(m, int(QKind.Q8_0), snap_embedding=False)
    g = CudaLlama(dev, m, QKind.Q8_0)
    lens = [2, 49, 17, 48, 3, 33, 49, 12, 40, 41]
    seqs = [random_tokens(100 + i, n, cfg.vocab) for i, n in enumerate(lens)]
    lps, grs, nll = g.score_ragged(seqs)
    for i, s in enumerate(seqs):
        wlp, wgr = orc.OracleLlama(ref).score(s)
        assert lps[i].shape == (len(s) - 1,)
        assert np.abs(lps[i] - wlp).max() < 1e-4, i
        assert np.array_equal(grs[i], wgr), i
        assert abs(nll[i] + wlp.astype(np.float64).sum()) < 1e-3
        alone_lp, alone_gr = g.score(s)
        assert np.abs(lps[i] - alone_lp).max() < 1e-4 and np.array_equal(grs[i], alone_gr)  # (another batch shape, other kernels)
    from ferrum_gpu_b200 import CudaError
    with pytest.raises(CudaError, match="at least 2 tokens"):
        g.score_ragged([seqs[0], [1]])
    with pytest.raises(CudaError, match="must be in 1..="):
        g.score_ragged([random_tokens(1, cfg.ctx + 2, cfg.vocab)])
    g.close()


@pytest.mark.parametrize("mode", [Mode.EXACT_F32, Mode.TENSOR_F16])
def test_sliding_windows_sum_to_the_oracle_scored_window_by_window(dev, mode):
    """serving/score.rs:L27-L49 over a stream of several contexts: the f64 sum, the count and the flag equal the
    CPU oracle's, scored one window at a time the way the reference does."""
    cfg, m = _model(ctx=64)
    ref = orc.dequantised_llama(m, int(QKind.Q4_0), snap_embedding=False)
    g = CudaLlama(dev, m, QKind.Q4_0)
    streams = [random_tokens(7, 300, cfg.vocab), random_tokens(8, 65, cfg.vocab), random_tokens(9, 66, cfg.vocab),
               random_tokens(10, 2, cfg.vocab), random_tokens(11, 1, cfg.vocab)]
    frm = [1, 1, 40, 1, 1]
    got = g.token_logprobs(streams, frm, mode)
    oracle = orc.OracleLlama(ref)
    for j, ids in enumerate(streams):
        want_lp, want_n, want_greedy, flips = 0.0, 0, True, 0
        for s, e, f in windows(len(ids), frm[j], cfg.ctx):
            lp, gr = oracle.score(ids[s:e])
            for t in range(f, e):
                want_lp += float(lp[t - s - 1])
                want_n += 1
                want_greedy &= bool(gr[t - s - 1])
        lp_g, n_g, greedy_g = got[j]
        assert n_g == want_n, j
        tol = 1e-4 * max(want_n, 1) if mode == Mode.EXACT_F32 else 5e-3 * max(want_n, 1)  # (std 0.2 weights: logits an order above the benchmark models')
        assert abs(lp_g - want_lp) < tol, (j, lp_g, want_lp)
        if mode == Mode.EXACT_F32:
            assert greedy_g == want_greedy
    # the Python mirror over the same model: one ragged batch per text, same sums
    d = ModelDecoder(g, encode=lambda text: [b % cfg.vocab for b in text.encode()], bos=0, mode=mode)
    s = token_logprobs(d, streams[0].tolist(), 1)
    assert s.n_tokens == got[0][1] and abs(s.logprob - got[0][0]) < 1e-3  # (its windows alone: another batch shape)
    r = rolling(d, "a long enough text to need more than one window of sixty-four positions " * 3)
    assert r.n_tokens == len(("a long enough text to need more than one window of sixty-four positions " * 3).encode())
    g.close()


def test_a_one_rank_group_scores_like_the_model(dev):
    """fc_group_create / fc_group_score with world 1: the communicator, the scatter and the all-reduce run on one
    GPU and must return fc_model_score's sums."""
    cfg, m = _model(ctx=40)
    ids = np.stack([random_tokens(50 + i, 33, cfg.vocab) for i in range(6)])
    single = CudaLlama(dev, m, QKind.Q4_0)
    _, _, want = single.score_batch(ids, Mode.EXACT_F32)
    single.close()
    gs = GroupScorer(m, QKind.Q4_0, vocab_shards=1, mode=Mode.EXACT_F32)
    got = gs.score(ids)
    assert np.array_equal(got, want)
    assert len(gs.exchange_ms()) == 3
    gs.close()
