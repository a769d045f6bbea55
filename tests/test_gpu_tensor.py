"""The bf16 tensor-core scoring path (tcgen05 product, flash attention, fused head log-sum-exp) against
the f32 CPU oracle over dequantised weights. Tolerances are the stated ones for this path: 2e-2 max-abs
per logit and 1e-3 mean NLL; structural tests use inputs whose products are exact in bf16 so any
layout or descriptor mistake shows as a non-zero difference."""
import numpy as np
import pytest

from ferrum_gpu_b200 import CudaGpt2, CudaLlama, Mode, QKind, linear_q, upload_quantised
from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.hostmodel import (Gpt2Config, LlamaConfig, config_c3, random_gpt2, random_llama,
                                       random_tokens)
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2   # max-abs per logit
NLL_TOL = 1e-3     # mean NLL


def exact_weights(kind, k, n, seed):
    """A `[k, n]` matrix that quantises without error: every block holds multiples of a power of two
    with the block's extreme present, so d is a power of two and d*q is exact in bf16."""
    rng = np.random.default_rng(seed)
    if kind == QKind.Q8_0:
        q = rng.integers(-127, 128, size=(n, k)).astype(np.float32)
        q[:, ::32] = 127.0
        rows = q * np.float32(2.0 ** -7)
    elif kind == QKind.Q4_0:
        q = rng.integers(-8, 8, size=(n, k)).astype(np.float32)
        q[:, ::32] = -8.0
        rows = q * np.float32(2.0 ** -6)
    else:
        rows = rng.integers(-8, 8, size=(n, k)).astype(np.float32) * np.float32(2.0 ** -6)
    return np.ascontiguousarray(rows.T).reshape(-1)  # [k, n]


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0, QKind.F32])
@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (128, 128, 128), (256, 192, 384), (130, 768, 264), (1, 64, 8),
                                   (517, 2048, 1000)])
def test_tensor_product_is_exact_on_exactly_representable_inputs(dev, kind, m, k, n):
    w = exact_weights(kind, k, n, 3)
    x = np.random.default_rng(4).integers(-3, 4, size=m * k).astype(np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    if kind != QKind.F32:
        assert np.array_equal(qw.dequantised().T.reshape(-1), w), "the weights must survive quantisation exactly"
    got = linear_q(dev, x, qw, m, Mode.TENSOR_F16)
    want = orc.matmul(x, w, m, k, n, threads=8).reshape(m, n)
    bad = np.argwhere(got != want)
    assert bad.size == 0, (kind, m, k, n, bad[:5], got[tuple(bad[0])], want[tuple(bad[0])])
    qw.close()


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0])
@pytest.mark.parametrize("m,k,n", [(512, 768, 768), (300, 2048, 2816), (4096, 768, 1280)])
def test_tensor_product_within_tolerance_on_gaussian_inputs(dev, kind, m, k, n):
    """X ~ N(0, 1), W ~ N(0, 0.02): the shapes of the isolated sweep's scoring rows."""
    rng = np.random.default_rng(7)
    w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal(m * k, dtype=np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    got = linear_q(dev, x, qw, m, Mode.TENSOR_F16)
    want = orc.matmul(x, orc.snap_matrix(int(kind), w, k, n), m, k, n, threads=8).reshape(m, n)
    err = np.abs(got - want).max()
    assert err < LOGIT_TOL and err < 0.02 * np.abs(want).max(), (kind, m, k, n, err, np.abs(want).max())
    qw.close()


def llama_tc_cfg(**kw):
    base = dict(vocab=96, ctx=256, dim=128, heads=2, kv_heads=1, head_dim=64, layers=2, hidden=192, rope_dim=64,
                rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
    base.update(kw)
    return LlamaConfig(**base)


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0, QKind.F16, QKind.FP8_E4M3, QKind.FP8_E5M2, QKind.MXFP4])
@pytest.mark.parametrize("variant", ["norm-gqa", "neox-bias-tied", "mha"])
def test_llama_tensor_forward_and_score_match_the_f32_oracle(dev, kind, variant):
    cfg = {"norm-gqa": llama_tc_cfg(), "neox-bias-tied": llama_tc_cfg(rope_type=_ffi.FC_ROPE_NEOX, rope_base=1e6, vocab=104),
           "mha": llama_tc_cfg(kv_heads=2, hidden=128)}[variant]
    biases, tied = variant == "neox-bias-tied", variant == "neox-bias-tied"
    m = random_llama(cfg, seed=5, biases=biases, tied=tied, std=0.05, gain_jitter=0.1)
    ref = orc.dequantised_llama(m, int(kind), snap_embedding=False)
    if tied:
        ref.head = orc.snap_matrix(int(kind), m.head, cfg.dim, cfg.vocab)
    oracle = orc.OracleLlama(ref, threads=8)
    g = CudaLlama(dev, m, kind)
    ids = random_tokens(9, 150, cfg.vocab)
    want = oracle.forward_logits(ids)
    got = g.forward_all(ids, Mode.TENSOR_F16)
    # the reference's metric |g - w| / max(|w|, 1): these test weights give logits up to ~4
    err, scale = orc.max_rel_err(got, want), np.abs(want).max()
    assert err < LOGIT_TOL and np.abs(got - want).max() < 0.03 * scale, (variant, kind, err, scale)
    # the exact path on the same (gate/up interleaved) weights stays at 1e-5
    assert orc.max_rel_err(g.forward_all(ids[:40]), want[:40]) < 1e-5
    seqs = np.stack([random_tokens(20 + i, 131, cfg.vocab) for i in range(3)])
    lp, gr, nll = g.score_batch(seqs, Mode.TENSOR_F16)
    for s in range(3):
        wlp, wgr = oracle.score(seqs[s])
        assert abs(float(np.mean(lp[s] - wlp))) < NLL_TOL, (variant, kind, s)
        assert np.abs(lp[s] - wlp).max() < 2 * LOGIT_TOL
        assert (gr[s] != wgr).mean() < 0.05  # argmax may flip only on near-ties
        assert abs(nll[s] + float(lp[s].astype(np.float64).sum())) < 1e-6 * max(1.0, abs(nll[s]))
    g.close()


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0])
def test_gpt2_tensor_forward_and_score_match_the_f32_oracle(dev, kind):
    cfg = Gpt2Config(vocab=80, ctx=200, dim=128, heads=2, layers=2, hidden=256)
    m = random_gpt2(cfg, seed=6, std=0.05, bias_std=0.05, gain_jitter=0.1)
    ref = orc.dequantised_gpt2(m, int(kind), snap_embedding=False)
    oracle = orc.OracleGpt2(ref, threads=8)
    g = CudaGpt2(dev, m, kind)
    ids = random_tokens(10, 140, cfg.vocab)
    want = oracle.forward_logits(ids)
    got = g.forward_all(ids, Mode.TENSOR_F16)
    err, scale = orc.max_rel_err(got, want), np.abs(want).max()
    assert err < LOGIT_TOL and np.abs(got - want).max() < 0.03 * scale, (kind, err, scale)
    lp, gr = g.score(ids, Mode.TENSOR_F16)
    wlp, _ = oracle.score(ids)
    assert abs(float(np.mean(lp - wlp))) < NLL_TOL
    g.close()


def test_config3_shape_scoring_within_tolerance(dev):
    """The Llama-style scoring configuration (12 layers, d_model 768, 12q/4kv, SwiGLU 2048, vocab 32000,
    Q4_0, N(0, 0.02) weights) on a 192-token slice: every logit within 2e-2, mean NLL within 1e-3."""
    cfg = config_c3()
    m = random_llama(cfg, seed=1)
    ref = orc.dequantised_llama(m, _ffi.FC_Q4_0, snap_embedding=True)
    m.tok = ref.tok
    oracle = orc.OracleLlama(ref, threads=8)
    g = CudaLlama(dev, m, QKind.Q4_0)
    ids = random_tokens(3, 193, cfg.vocab)
    want = oracle.forward_logits(ids[:-1])
    got = g.forward_all(ids[:-1], Mode.TENSOR_F16)
    assert np.abs(got - want).max() < LOGIT_TOL
    wlp, _ = orc.score(want, ids[1:], cfg.vocab)
    lp, _ = g.score(ids, Mode.TENSOR_F16)
    assert abs(float(np.mean(lp - wlp))) < NLL_TOL
    lp32, _ = g.score(ids, Mode.EXACT_F32)
    assert np.abs(lp32 - wlp).max() < 1e-4
    g.close()


def test_long_sequences_cross_several_query_blocks_and_key_tiles(dev):
    """520 tokens: three blocks of 256 query rows (the last one ragged, its second half idle) and up to five
    key tiles per block in the tcgen05 attention kernel, two sequences and two KV groups per launch."""
    cfg = llama_tc_cfg(ctx=600, heads=4, kv_heads=2, dim=256, hidden=256)
    m = random_llama(cfg, seed=8, std=0.05, gain_jitter=0.1)
    ref = orc.dequantised_llama(m, int(QKind.Q8_0), snap_embedding=False)
    oracle = orc.OracleLlama(ref, threads=8)
    g = CudaLlama(dev, m, QKind.Q8_0)
    seqs = np.stack([random_tokens(40 + i, 520, cfg.vocab) for i in range(2)])
    lp, gr, nll = g.score_batch(seqs, Mode.TENSOR_F16)
    for s in range(2):
        wlp, wgr = oracle.score(seqs[s])
        assert abs(float(np.mean(lp[s] - wlp))) < NLL_TOL, s
        assert np.abs(lp[s] - wlp).max() < 2 * LOGIT_TOL
        assert (gr[s] != wgr).mean() < 0.05
    g.close()


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0])
def test_largest_sweep_shapes_on_sampled_output_columns(dev, kind):
    """The far corner of the isolated sweep (K = 4096, N in {11008, 32000}, M in {1, 8, 64, 512, 4096}) is too big
    for the scalar oracle, so 48 sampled output columns are recomputed in float64 from the oracle's snapped weights:
    decode-side rows (exact path) within 1e-5 by the reference's metric, scoring-side rows (tensor path) within
    2e-2 - its per-logit bound; outputs here have standard deviation ~1.3."""
    k = 4096
    rng = np.random.default_rng(7)
    for n in (11008, 32000):
        w = (rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02))
        cols = np.sort(rng.choice(n, 48, replace=False))
        wq = orc.snap_matrix(int(kind), np.ascontiguousarray(w[:, cols]).reshape(-1), k, cols.size).reshape(k, cols.size)
        qw = upload_quantised(dev, kind, w.reshape(-1), k, n)
        del w
        for m, mode, tol in ((1, Mode.EXACT_F32, 1e-5), (8, Mode.EXACT_F32, 1e-5), (64, Mode.EXACT_F32, 1e-5),
                             (512, Mode.TENSOR_F16, LOGIT_TOL), (4096, Mode.TENSOR_F16, LOGIT_TOL)):
            x = rng.standard_normal((m, k), dtype=np.float32)
            got = linear_q(dev, x.reshape(-1), qw, m, mode).reshape(m, n)[:, cols]
            want = x.astype(np.float64) @ wq.astype(np.float64)
            err = (np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max()
            assert err < tol, (kind, n, m, mode, err)
        qw.close()


@pytest.mark.parametrize("hidden", [512, 320])
def test_q2k_llama_decode_scoring_and_tensor_forward_match_the_oracle(dev, hidden):
    """Q2_K needs input widths of whole 256s: with hidden = 320 the down projection is stored as Q4_0 instead
    (`effective`, ops/quant.rs:L134-L144), the rest stays Q2_K. The oracle computes with the same dequantised
    weights; the exact path stays at 1e-5, the tensor path at the scoring tolerances."""
    cfg = LlamaConfig(vocab=96, ctx=256, dim=256, heads=4, kv_heads=2, head_dim=64, layers=2, hidden=hidden, rope_dim=64,
                      rope_base=10000.0, rope_type=_ffi.FC_ROPE_NORM, eps=1e-5)
    m = random_llama(cfg, seed=5, std=0.05, gain_jitter=0.1)
    ref = orc.dequantised_llama(m, int(QKind.Q2_K), snap_embedding=False)
    oracle = orc.OracleLlama(ref, threads=8)
    g = CudaLlama(dev, m, QKind.Q2_K, max_streams=12)
    ids = random_tokens(9, 150, cfg.vocab)
    want = oracle.forward_logits(ids)
    assert orc.max_rel_err(g.forward_all(ids[:40]), want[:40]) < 1e-5
    got = g.forward_all(ids, Mode.TENSOR_F16)
    err, scale = orc.max_rel_err(got, want), np.abs(want).max()
    assert err < LOGIT_TOL and np.abs(got - want).max() < 0.03 * scale, (hidden, err, scale)
    seqs = np.stack([random_tokens(20 + i, 131, cfg.vocab) for i in range(2)])
    lp, gr, nll = g.score_batch(seqs, Mode.TENSOR_F16)
    for s in range(2):
        wlp, wgr = oracle.score(seqs[s])
        assert abs(float(np.mean(lp[s] - wlp))) < NLL_TOL and np.abs(lp[s] - wlp).max() < 2 * LOGIT_TOL
    # token-by-token decode, one stream and twelve (the 9..64-row products fall back to the exact tiled kernel)
    o1 = orc.OracleLlama(ref)
    for t in ids[:6]:
        assert orc.max_rel_err(g.feed(int(t)), o1.feed(int(t))) < 1e-5
    g.reset()
    toks = np.stack([random_tokens(50 + s, 3, cfg.vocab) for s in range(12)])
    oracles = [orc.OracleLlama(ref) for _ in range(12)]
    for i in range(3):
        am, lg = g.feed_batch(toks[:, i], want_logits=True)
        for s in range(12):
            assert orc.max_rel_err(lg[s], oracles[s].feed(int(toks[s, i]))) < 2e-5
            assert am[s] == orc.argmax(lg[s])
    g.close()


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0])
def test_tensor_core_prefill_fills_the_cache_and_decode_continues_from_it(dev, kind):
    """A prompt through the scoring kernels (`prefill(..., Mode.TENSOR_F16)`) leaves its k and v in the f32
    cache: the last position's logits and the logits of the exactly decoded tokens that follow stay within
    the scoring tolerance of the f32 oracle, on a second stream while the first holds another context."""
    cfg = llama_tc_cfg(rope_type=_ffi.FC_ROPE_NEOX, rope_base=1e6, vocab=104, kv_heads=1)
    m = random_llama(cfg, seed=5, biases=True, std=0.05, gain_jitter=0.1)
    ref = orc.dequantised_llama(m, int(kind), snap_embedding=False)
    g = CudaLlama(dev, m, kind, max_streams=2)
    g.prefill(random_tokens(3, 9, cfg.vocab), stream=0)  # an unrelated context in the other stream
    ids = random_tokens(9, 140, cfg.vocab)
    oracle = orc.OracleLlama(ref, threads=8)
    want = [oracle.feed(int(t)) for t in ids]
    got = g.prefill(ids[:131], stream=1, mode=Mode.TENSOR_F16)
    assert g.pos(1) == 131 and g.pos(0) == 9
    scale = max(1.0, float(np.abs(want[130]).max()))
    assert np.abs(got - want[130]).max() < LOGIT_TOL * scale
    for i in range(131, 140):
        lg = g.feed(int(ids[i]), stream=1)
        assert np.abs(lg - want[i]).max() < LOGIT_TOL * max(1.0, float(np.abs(want[i]).max())), i
    with pytest.raises(Exception, match="empty stream"):
        g.prefill(ids[:4], stream=1, mode=Mode.TENSOR_F16)
    # the exact prefill of the same prompt agrees with the tensor one to the same tolerance
    g.reset(1)
    exact = g.prefill(ids[:131], stream=1)
    assert np.abs(exact - got).max() < LOGIT_TOL * scale and orc.max_rel_err(exact, want[130]) < 1e-5
    g.close()


def test_generate_with_a_tensor_core_prefill_continues_like_the_oracle(dev):
    """`GenOpts.prefill = Mode.TENSOR_F16`: the prompt runs through the scoring kernels, the new tokens through
    the exact decode path; on a model with well-separated logits the greedy continuation is the oracle's."""
    from ferrum_gpu_b200 import CudaBackend, GenOpts, generate_with
    cfg = llama_tc_cfg(vocab=64)
    m = random_llama(cfg, seed=12, std=0.3, gain_jitter=0.1)  # large weights: logits far apart
    oracle = orc.OracleLlama(orc.dequantised_llama(m, int(QKind.Q8_0), snap_embedding=False))
    prompt = [int(t) for t in random_tokens(4, 70, cfg.vocab)]
    want = generate_with(oracle.feed, cfg.ctx, prompt, GenOpts(max_new=6))
    got = CudaBackend(dev, QKind.Q8_0).generate(m, prompt, GenOpts(max_new=6, prefill=Mode.TENSOR_F16))
    assert len(got) == 6
    assert got == want
