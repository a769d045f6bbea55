"""Parity at the widths of the two benchmark configurations that the small-model tests do not reach: the
64-stream Qwen2-style decode (16 query / 2 KV heads, caches past 512 positions, a 151 936-row tied head) and the
GPT-2-124M scoring shape with its odd vocabulary of 50 257, whole and split in two shards on one device. Layers
are cut to 2 so that the CPU oracle finishes in seconds. Plus RoPE with a linear factor and with per-frequency
factors on the device. Mirrors ferrum_wgpu/src/models/llama/tests.rs:L63-L89,L196-L213."""
import numpy as np
import pytest

from ferrum_gpu_b200 import CudaGpt2, CudaLlama, Mode, QKind
from ferrum_gpu_b200 import _ffi
from ferrum_gpu_b200.hostmodel import config_c4, config_c5, random_gpt2, random_llama, random_tokens
from oracle import oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu

FORWARD = 1e-5  # ferrum_wgpu/src/tolerance.rs:L11


def test_config4_width_64_streams_past_512_positions_match_the_oracle(dev):
    """d 1024, 16 q / 2 kv heads of 64, FFN 2816, vocab 151936 tied, q/k/v biases, NEOX theta 1e6, Q8_0, 2 layers:
    64 streams prefilled to 600..663 positions (two context splits of the decode attention, different lengths
    per stream), then 3 single steps with logits and 5 chained greedy steps. Two of the streams are followed by
    the CPU oracle: logits within 2e-5 (1e-5 against exact arithmetic plus the oracle's own rounding) and the
    same greedy tokens."""
    cfg = config_c4()
    cfg.layers = 2
    m = random_llama(cfg, seed=31, biases=True, tied=True)
    ref = orc.dequantised_llama(m, int(QKind.Q8_0), snap_embedding=True)
    m.tok = ref.tok  # the file convention: the table is a round-tripped Q8_0 tensor, the head its transpose
    m.head = ref.head
    n_streams, watch = 64, (5, 40)
    g = CudaLlama(dev, m, QKind.Q8_0, max_streams=n_streams)
    prompts = [random_tokens(900 + s, 600 + s, cfg.vocab) for s in range(n_streams)]
    for s in range(n_streams):
        g.prefill(prompts[s], stream=s)
    oracles = {}
    for s in watch:
        o = orc.OracleLlama(ref, threads=8)
        o.extend_last(prompts[s])
        oracles[s] = o
    toks = random_tokens(77, n_streams, cfg.vocab)
    picks = []
    for step in range(3):
        am, lg = g.feed_batch(toks, want_logits=True)
        for s in watch:
            want = oracles[s].feed(int(toks[s]))
            assert orc.max_rel_err(lg[s], want) < 2 * FORWARD, (step, s)
            margin = np.partition(want, -2)[-2:]
            assert am[s] == orc.argmax(want) or margin[1] - margin[0] < 2 * FORWARD * max(1.0, abs(margin[1])), (step, s)
        for s in range(n_streams):
            assert am[s] == orc.argmax(lg[s])  # first maximum over the 151 936 entries, on several CTAs
        toks = am
        picks.append(am.copy())
    chain = g.decode_greedy(toks, 5)
    for s in watch:
        t = int(toks[s])
        for step in range(5):
            want = oracles[s].feed(t)
            margin = np.partition(want, -2)[-2:]
            assert chain[step, s] == orc.argmax(want) or margin[1] - margin[0] < 2 * FORWARD * max(1.0, abs(margin[1])), (step, s)
            t = int(chain[step, s])
    assert all(g.pos(s) == 600 + s + 8 for s in range(n_streams))
    g.close()


def test_config5_width_scores_the_odd_vocabulary_whole_and_in_two_shards(dev):
    """GPT-2-124M width (d 768, 12 heads, FFN 3072, ctx 1024, LayerNorm, GELU), vocab 50257 tied, Q4_0, 2 layers:
    2 x 256 tokens on the tensor path against the oracle (2e-2 per logit, 1e-3 mean NLL), then the same
    sequences through the split head with both shards on this device: (0, 2) and (1, 2) in turn, merged by
    fc_score_combine_dev - 25129 + 25128 rows, the second shard starting at an odd row."""
    import ctypes as C
    import torch
    cfg = config_c5()
    cfg.layers = 2
    m = random_gpt2(cfg, seed=41, tied=True)
    ref = orc.dequantised_gpt2(m, int(QKind.Q4_0), tied=True, snap_embedding=True)
    m.tok, m.head = ref.tok, ref.head
    ids = np.stack([random_tokens(500 + i, 256, cfg.vocab) for i in range(2)])
    g = CudaGpt2(dev, m, QKind.Q4_0)
    lp, gr, nll = g.score_batch(ids, Mode.TENSOR_F16)
    logits = g.forward_all(ids[0], Mode.TENSOR_F16)
    oracle = orc.OracleGpt2(ref, threads=8)
    for s in range(2):
        want_logits = oracle.forward_logits(ids[s][:-1])
        if s == 0:
            assert np.abs(logits[:-1] - want_logits).max() < 2e-2
        wlp, wgr = orc.score(want_logits, ids[s][1:], cfg.vocab)
        assert np.abs(lp[s] - wlp).max() < 2e-2
        assert abs(nll[s] / 255 + wlp.astype(np.float64).mean()) < 1e-3
    # split head, both shards on one device
    lib = _ffi.load()
    t = ids.shape[1] - 1
    rows = 2 * t
    d_in = torch.from_numpy(np.ascontiguousarray(ids[:, :t])).cuda()
    d_tgt = torch.from_numpy(np.ascontiguousarray(ids[:, 1:]).reshape(-1)).cuda()
    hidden = torch.empty(rows, cfg.dim, dtype=torch.float16, device="cuda")
    partials = torch.empty(2, rows, 4, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    g.trunk_dev(d_in.data_ptr(), 2, t, Mode.TENSOR_F16, hidden.data_ptr())
    for shard in range(2):
        g.set_head_shard(shard, 2)
        g.head_partial_dev(hidden.data_ptr(), d_tgt.data_ptr(), rows, Mode.TENSOR_F16, partials[shard].data_ptr())
    lp2 = torch.empty(rows, dtype=torch.float32, device="cuda")
    gr2 = torch.empty(rows, dtype=torch.uint8, device="cuda")
    nll2 = torch.empty(2, dtype=torch.float64, device="cuda")
    dev.check(lib.fc_score_combine_dev(dev.handle, partials.data_ptr(), 2, d_tgt.data_ptr(), 2, t, lp2.data_ptr(),
                                       gr2.data_ptr(), nll2.data_ptr()))
    dev.sync()
    lp2, nll2 = lp2.cpu().numpy().reshape(2, t), nll2.cpu().numpy()
    assert np.abs(lp2 - lp).max() < 1e-4, "the split head is the same arithmetic, merged across shards"
    assert np.abs(nll2 - nll).max() < 1e-2
    assert np.array_equal(gr2.cpu().numpy().reshape(2, t).astype(bool), gr)
    g.set_head_shard(0, 1)
    g.close()


@pytest.mark.parametrize("scaling", ["linear", "freq_factors", "both"])
def test_rope_scaling_on_the_device_matches_the_oracle(dev, scaling):
    """ferrum_ref/src/models/llama/ops.rs:L80-L101: theta = p * freq / ff * (1 / linear). The tables are built on
    the host by the library; decode, forward_all and the tensor path must all see the scaled angles."""
    cfg = helpers.tiny_llama_cfg(vocab=29, ctx=24, dim=128, heads=2, kv_heads=1, head_dim=64, hidden=128, rope_dim=64)
    if scaling in ("linear", "both"):
        cfg.rope_linear_factor = 2.0
    if scaling in ("freq_factors", "both"):
        cfg.freq_factors = (1.0 + 0.25 * np.arange(cfg.rope_dim // 2, dtype=np.float32)).astype(np.float32)
    m = helpers.ref_random_llama(cfg, 17, False, False)
    oracle = orc.OracleLlama(m)
    ids = [i % cfg.vocab for i in helpers_ids()]
    want = oracle.forward_logits(ids)
    plain = helpers.tiny_llama_cfg(vocab=29, ctx=24, dim=128, heads=2, kv_heads=1, head_dim=64, hidden=128, rope_dim=64)
    unscaled = orc.OracleLlama(helpers.ref_random_llama(plain, 17, False, False)).forward_logits(ids)
    assert np.abs(want - unscaled).max() > 1e-3, "the scaling must matter for this test to mean anything"
    g = CudaLlama(dev, m)
    for i, t in enumerate(ids):
        assert orc.max_rel_err(g.feed(t), want[i]) < 2 * FORWARD, (scaling, i)
    assert orc.max_rel_err(g.forward_all(ids), want) < 2 * FORWARD
    assert orc.max_rel_err(g.forward_all(ids, Mode.TENSOR_F16), want) < 2e-2
    g.close()


def helpers_ids():
    return [3, 16, 0, 9, 9, 4, 11, 2, 7, 5, 1, 8, 6, 10, 12, 15, 14, 13, 20, 28]
