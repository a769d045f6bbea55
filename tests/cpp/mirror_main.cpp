// Drives the C++ mirror of the reference's interfaces (include/ferrum_cuda.hpp) end to end on one GPU: a small
// Llama-style model with weights from an integer hash (the Python test builds the same arrays), quantised to Q8_0,
// then feed / decode_greedy / score / generate / a packed product. Every result is printed as the bit pattern of
// its floats, one record per line; tests/test_gpu_cpp_mirror.py compares them with the ctypes mirror's.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "ferrum_cuda.hpp"

static std::vector<float> hashed(size_t n, uint32_t seed, float scale) {
  std::vector<float> v(n);
  for (size_t i = 0; i < n; i++) {
    const uint32_t h = ((uint32_t)i * 2654435761u + seed * 40503u) >> 8 & 0xffffu;
    v[i] = ((float)h / 65536.0f - 0.5f) * scale;
  }
  return v;
}

static void dump(const char* tag, const std::vector<float>& v) {
  std::printf("%s", tag);
  for (float f : v) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    std::printf(" %08x", u);
  }
  std::printf("\n");
}

int main() {
  try {
    ferrum::CudaBackend be(0, ferrum::QKind::Q8_0);
    std::printf("kind %s\n", be.kind());
    FcLlamaConfig cfg{};
    cfg.vocab = 40, cfg.ctx = 16, cfg.dim = 64, cfg.heads = 2, cfg.kv_heads = 1, cfg.head_dim = 32, cfg.layers = 2, cfg.hidden = 96;
    cfg.rope_dim = 32, cfg.rope_type = FC_ROPE_NEOX, cfg.rope_base = 10000.0f, cfg.eps = 1e-5f, cfg.rope_linear_factor = 1.0f;
    const uint32_t d = cfg.dim, qd = cfg.heads * cfg.head_dim, kvd = cfg.kv_heads * cfg.head_dim, hid = cfg.hidden;
    std::vector<std::vector<float>> keep;
    auto mk = [&](size_t n, float scale) {
      keep.push_back(hashed(n, (uint32_t)keep.size() + 1, scale));
      return keep.back().data();
    };
    auto ones = [&](size_t n) {
      keep.push_back(std::vector<float>(n, 1.0f));
      return keep.back().data();
    };
    std::vector<FcLlamaBlock> blocks(cfg.layers);
    for (auto& b : blocks) {
      b = FcLlamaBlock{};
      b.attn_norm = ones(d), b.ffn_norm = ones(d);
      b.wq = mk((size_t)d * qd, 0.4f), b.wk = mk((size_t)d * kvd, 0.4f), b.wv = mk((size_t)d * kvd, 0.4f), b.wo = mk((size_t)qd * d, 0.4f);
      b.gate = mk((size_t)d * hid, 0.4f), b.up = mk((size_t)d * hid, 0.4f), b.down = mk((size_t)hid * d, 0.4f);
    }
    FcLlamaWeights w{};
    w.tok = mk((size_t)cfg.vocab * d, 1.0f), w.blocks = blocks.data(), w.out_norm = ones(d), w.head = mk((size_t)d * cfg.vocab, 0.6f);

    ferrum::CudaLlama m(be.gpu(), cfg, w, ferrum::QKind::Q8_0);
    const std::vector<int32_t> ids = {3, 17, 0, 9, 9, 4, 11, 2};
    for (int32_t t : ids) dump("feed", m.feed(t));
    std::printf("pos %u\n", m.pos());
    const auto chain = m.decode_greedy(5, 4);
    std::printf("chain");
    for (int32_t t : chain) std::printf(" %d", t);
    std::printf("\n");
    m.reset();
    std::vector<float> lp;
    for (auto [l, g] : m.score(ids)) lp.push_back(l), std::printf("greedy %d\n", g ? 1 : 0);
    dump("score", lp);
    const auto gen = be.generate(cfg, w, {3, 17, 0}, 30);  // stops when the 16-token context is full
    std::printf("generate");
    for (int32_t t : gen) std::printf(" %d", t);
    std::printf("\n");
    try {
      be.generate(cfg, w, std::vector<int32_t>(16, 1), 1);
      std::printf("no error\n");
    } catch (const ferrum::Error& e) {
      std::printf("error %s\n", e.what());
    }
    ferrum::QWeight qw(be.gpu(), ferrum::QKind::Q4_0, hashed((size_t)64 * 48, 99, 0.1f), 64, 48);
    dump("linear", ferrum::linear_q(qw, hashed((size_t)3 * 64, 7, 2.0f), 3));
    try {
      m.feed(40);
    } catch (const ferrum::Error& e) {
      std::printf("range %d %s\n", e.code, e.what());
    }
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "failed: %s\n", e.what());
    return 1;
  }
}
