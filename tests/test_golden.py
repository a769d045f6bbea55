"""The committed golden vectors (tests/golden/golden.npz, made by tests/golden/make_golden.py) against
the oracle on CPU and against the CUDA path on the GPU."""
import os

import numpy as np
import pytest

from ferrum_gpu_b200._ffi import FC_Q4_0, FC_Q8_0
from ferrum_gpu_b200.hostmodel import Gpt2Config
from oracle import oracle as orc
from tests import helpers

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
IDS = [3, 1, 4, 1, 5, 9, 2, 6]
K, N = 96, 14


def test_oracle_reproduces_the_golden_codec_vectors():
    w = helpers.nasty(K * N)
    assert np.array_equal(w.view(np.uint32), G["codec_w"].view(np.uint32))
    for name, kind in (("q8_0", FC_Q8_0), ("q4_0", FC_Q4_0)):
        b = orc.quantise_matrix(kind, w, K, N)
        assert np.array_equal(b, G[f"codec_{name}_blocks"])
        assert np.array_equal(orc.decode(kind, b, K * N).view(np.uint32), G[f"codec_{name}_rows"].view(np.uint32))


def test_oracle_reproduces_the_golden_logits():
    m = helpers.ref_random_llama(helpers.tiny_llama_cfg(), 3, True, False)
    assert np.array_equal(orc.OracleLlama(m).forward_logits(IDS), G["llama_tiny_logits"])
    g = helpers.ref_random_gpt2(Gpt2Config(vocab=11, ctx=10, dim=8, heads=2, layers=2, hidden=16), 1)
    assert np.array_equal(orc.OracleGpt2(g).forward_logits(IDS), G["gpt2_tiny_logits"])


@pytest.mark.gpu
def test_cuda_path_reproduces_the_golden_vectors(dev):
    from ferrum_gpu_b200 import CudaLlama, QKind, linear_q, upload_quantised
    w = G["codec_w"]
    for name, kind in (("q8_0", QKind.Q8_0), ("q4_0", QKind.Q4_0)):
        qw = upload_quantised(dev, kind, w, K, N)
        assert np.array_equal(qw.blocks(), G[f"codec_{name}_blocks"]), "device encoder vs golden blocks"
        assert np.array_equal(qw.dequantised().reshape(-1).view(np.uint32), G[f"codec_{name}_rows"].view(np.uint32))
        y = linear_q(dev, G["linear_x"], qw, 5)
        want = G[f"linear_{name}_y"]  # the stress weights span 1e-6 .. 3e4: compare on the scale of the result
        assert np.abs(y.reshape(-1) - want).max() < 1e-5 * np.abs(want).max()
        qw.close()
    cfg, biases, tied = helpers.gpu_llama_variants()[1][1:]
    g = CudaLlama(dev, helpers.ref_random_llama(cfg, 8, biases, tied), QKind.Q8_0)
    got = g.forward_all(IDS)
    assert orc.max_rel_err(got, G["llama_qwen_q8_0_logits"]) < 2e-5
    lp, gr = g.score(IDS)
    assert np.abs(lp - G["llama_qwen_q8_0_logprob"]).max() < 1e-4
    assert np.array_equal(gr, G["llama_qwen_q8_0_greedy"])
    g.close()
