"""The C++ mirror of the reference's interfaces (include/ferrum_cuda.hpp) compiled and run: a small program
(tests/cpp/mirror_main.cpp) builds a model from hashed weights and prints what feed / decode_greedy / score /
generate / linear_q return; the same calls through the ctypes mirror must give the same bits. The CPU half of the
suite checks that the header compiles and links against the built library without running anything."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "mirror_main.cpp")
LIBDIR = os.path.join(ROOT, "ferrum_gpu_b200")


def build(tmp_path) -> str:
    exe = str(tmp_path / "mirror_main")
    cuda_inc = "/usr/local/cuda/include"
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc, SRC, "-o", exe,
           "-L", LIBDIR, "-lferrum_cuda", f"-Wl,-rpath,{LIBDIR}", "-Wl,-rpath,/usr/local/cuda/lib64", "-L/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_the_cpp_mirror_compiles_and_links(tmp_path):
    assert os.path.exists(build(tmp_path))


def hashed(n, seed, scale):
    i = np.arange(n, dtype=np.uint64)
    h = ((i * np.uint64(2654435761) + np.uint64(seed * 40503)) & np.uint64(0xFFFFFFFF)) >> np.uint64(8) & np.uint64(0xFFFF)
    return ((h.astype(np.float32) / np.float32(65536.0) - np.float32(0.5)) * np.float32(scale)).astype(np.float32)


@pytest.mark.gpu
def test_the_cpp_mirror_returns_what_the_ctypes_mirror_returns(dev, tmp_path):
    from ferrum_gpu_b200 import CudaBackend, CudaLlama, GenOpts, QKind, linear_q, upload_quantised
    from ferrum_gpu_b200 import _ffi
    from ferrum_gpu_b200.hostmodel import Llama, LlamaBlock, LlamaConfig
    out = subprocess.run([build(tmp_path)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()

    cfg = LlamaConfig(vocab=40, ctx=16, dim=64, heads=2, kv_heads=1, head_dim=32, layers=2, hidden=96, rope_dim=32,
                      rope_base=10000.0, rope_type=_ffi.FC_ROPE_NEOX, eps=1e-5)
    d, qd, kvd, hid = 64, 64, 32, 96
    n = [0]

    def mk(size, scale):
        n[0] += 1
        return hashed(size, n[0], scale)

    def ones(size):
        n[0] += 1
        return np.ones(size, dtype=np.float32)

    blocks = []
    for _ in range(cfg.layers):
        an, fn = ones(d), ones(d)
        wq, wk, wv, wo = mk(d * qd, 0.4), mk(d * kvd, 0.4), mk(d * kvd, 0.4), mk(qd * d, 0.4)
        gate, up, down = mk(d * hid, 0.4), mk(d * hid, 0.4), mk(hid * d, 0.4)
        blocks.append(LlamaBlock(attn_norm=an, wq=wq, wk=wk, wv=wv, wo=wo, ffn_norm=fn, gate=gate, up=up, down=down,
                                 bq=None, bk=None, bv=None))
    tok = mk(cfg.vocab * d, 1.0)
    out_norm = ones(d)
    head = mk(d * cfg.vocab, 0.6)
    model = Llama(cfg, tok, blocks, out_norm, head, False)

    def bits(line, tag):
        assert line.startswith(tag + " "), line
        return np.array([int(x, 16) for x in line.split()[1:]], dtype=np.uint32)

    assert lines[0] == "kind cuda"
    g = CudaLlama(dev, model, QKind.Q8_0)
    ids = [3, 17, 0, 9, 9, 4, 11, 2]
    for i, t in enumerate(ids):
        assert np.array_equal(bits(lines[1 + i], "feed"), g.feed(t).view(np.uint32)), i
    assert lines[9] == "pos 8"
    assert lines[10] == "chain " + " ".join(str(t) for t in g.decode_greedy([5], 4)[:, 0])
    g.reset()
    lp, gr = g.score(ids)
    for i in range(7):
        assert lines[11 + i] == f"greedy {int(gr[i])}"
    assert np.array_equal(bits(lines[18], "score"), lp.view(np.uint32))
    gen = CudaBackend(dev, QKind.Q8_0).generate(model, [3, 17, 0], GenOpts(max_new=30))
    assert len(gen) == 13 and lines[19] == "generate " + " ".join(str(t) for t in gen)
    assert lines[20] == "error the prompt has 16 tokens but the context is 16"
    qw = upload_quantised(dev, QKind.Q4_0, hashed(64 * 48, 99, 0.1), 64, 48)
    assert np.array_equal(bits(lines[21], "linear"), linear_q(dev, hashed(3 * 64, 7, 2.0), qw, 3).reshape(-1).view(np.uint32))
    assert lines[22].startswith(f"range {_ffi.FC_ERR_RANGE} index 40 is out of range for 40 entries")
    g.close()
