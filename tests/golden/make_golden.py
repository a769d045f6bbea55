"""Regenerates tests/golden/golden.npz.

The reference is Rust and cannot be run in the build environment, so these vectors are outputs of the
CPU oracle (oracle/ferrum_oracle.cpp) at the commit that pinned it against the reference's known-answer
tests. They freeze the oracle: a later change to it that moves any of these bytes or logits fails
tests/test_golden.py. They also give the GPU tests inputs and expected outputs that do not need the
oracle at run time.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from ferrum_gpu_b200._ffi import FC_Q4_0, FC_Q8_0  # noqa: E402
from ferrum_gpu_b200.hostmodel import Gpt2Config  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tests import helpers  # noqa: E402

IDS = [3, 1, 4, 1, 5, 9, 2, 6]


def main():
    out = {}
    k, n = 96, 14
    w = helpers.nasty(k * n)
    out["codec_w"] = w
    for name, kind in (("q8_0", FC_Q8_0), ("q4_0", FC_Q4_0)):
        b = orc.quantise_matrix(kind, w, k, n)
        out[f"codec_{name}_blocks"] = b
        out[f"codec_{name}_rows"] = orc.decode(kind, b, k * n)
    x = orc.rand_vec(5 * k, 5)
    out["linear_x"] = x
    out["linear_q8_0_y"] = orc.matmul(x, orc.snap_matrix(FC_Q8_0, w, k, n), 5, k, n)
    out["linear_q4_0_y"] = orc.matmul(x, orc.snap_matrix(FC_Q4_0, w, k, n), 5, k, n)
    m = helpers.ref_random_llama(helpers.tiny_llama_cfg(), 3, True, False)
    out["llama_tiny_logits"] = orc.OracleLlama(m).forward_logits(IDS)
    cfg, biases, tied = helpers.gpu_llama_variants()[1][1:]
    mq = helpers.ref_random_llama(cfg, 8, biases, tied)
    ref = orc.dequantised_llama(mq, FC_Q8_0, snap_embedding=False)
    ref.head = orc.snap_matrix(FC_Q8_0, mq.head, cfg.dim, cfg.vocab)
    out["llama_qwen_q8_0_logits"] = orc.OracleLlama(ref).forward_logits(IDS)
    lp, gr = orc.OracleLlama(ref).score(IDS)
    out["llama_qwen_q8_0_logprob"], out["llama_qwen_q8_0_greedy"] = lp, gr
    g = helpers.ref_random_gpt2(Gpt2Config(vocab=11, ctx=10, dim=8, heads=2, layers=2, hidden=16), 1)
    out["gpt2_tiny_logits"] = orc.OracleGpt2(g).forward_logits(IDS)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
