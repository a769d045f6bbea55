// C++ mirror of the reference's interfaces for the quantised inference path, above the C ABI of
// ferrum_cuda.h. Header-only. Names, argument meaning and error behaviour follow the Rust items they
// stand in for; errors are `Result<_, String>` there and `ferrum::Error` (a std::runtime_error
// carrying the status code) here.
//
//   ferrum::Gpu          ferrum_wgpu::device::Gpu                  (device/mod.rs:L98-L176)
//   ferrum::QWeight      ferrum_wgpu::ops::quant::QWeight           (ops/quant.rs:L150-L183)
//   ferrum::linear_q     ferrum_wgpu::ops::quant::linear_q          (ops/quant.rs:L326-L335)
//   ferrum::CudaLlama    ferrum_wgpu::models::llama::GpuLlama       (models/llama/mod.rs:L215-L439, forward.rs)
//   ferrum::CudaGpt2     ferrum_wgpu::models::gpt2::GpuGpt2         (models/gpt2.rs:L134-L346)
//   ferrum::CudaBackend  impl Backend for GpuBackend                (ferrum_gpu_core/src/engine/{mod,gpu}.rs)
#pragma once

#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "ferrum_cuda.h"

namespace ferrum {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// ops::quant::QKind (ferrum_wgpu/src/ops/quant.rs:L27-L44), plus F32 for matrices kept unquantised
enum class QKind {
  F32 = FC_F32,
  Q8_0 = FC_Q8_0,
  Q4_0 = FC_Q4_0,
  F16 = FC_F16,
  Fp8E4M3 = FC_FP8_E4M3,
  Fp8E5M2 = FC_FP8_E5M2,
  Fp4 = FC_MXFP4,
  Q2K = FC_Q2_K,
};
enum class Mode { ExactF32 = FC_EXACT_F32, TensorF16 = FC_TENSOR_F16 };

class Gpu {
 public:
  explicit Gpu(int ordinal = 0) {
    int rc = fc_device_open(ordinal, &h_);
    if (rc != FC_OK) throw Error(rc, fc_last_error(nullptr));
  }
  ~Gpu() {
    if (h_) fc_device_close(h_);
  }
  Gpu(const Gpu&) = delete;
  Gpu& operator=(const Gpu&) = delete;
  FcDevice* raw() const { return h_; }
  void check(int rc) const {
    if (rc != FC_OK) throw Error(rc, fc_last_error(h_));
  }
  std::string name() const {
    char buf[256];
    check(fc_device_name(h_, buf, sizeof buf));
    return buf;
  }
  // Gpu::fail_after (device/runtime.rs:L214-L256); a negative count disarms the hook
  void fail_after(long long n) const { check(fc_debug_fail_after(h_, n)); }
  unsigned long long launches() const { return fc_device_launch_count(h_); }

 private:
  FcDevice* h_ = nullptr;
};

class QWeight {
 public:
  // upload_quantised (ops/quant.rs:L279-L288): `w` is the [k, n] ([in, out]) f32 matrix
  QWeight(const Gpu& gpu, QKind kind, const std::vector<float>& w, uint32_t k, uint32_t n) : gpu_(gpu) {
    if (w.size() != (size_t)k * n) throw Error(FC_ERR_SHAPE, "weight length does not match k x n");
    gpu.check(fc_qweight_create(gpu.raw(), (int)kind, w.data(), k, n, &h_));
    k_ = k, n_ = n, kind_ = kind;
  }
  ~QWeight() {
    if (h_) fc_qweight_destroy(h_);
  }
  QWeight(const QWeight&) = delete;
  QKind kind() const { return kind_; }
  uint32_t k() const { return k_; }
  uint32_t n() const { return n_; }
  uint64_t device_bytes() const {
    uint64_t b = 0;
    gpu_.check(fc_qweight_info(h_, nullptr, nullptr, nullptr, &b));
    return b;
  }
  std::vector<float> dequantised() const { // [n, k]
    std::vector<float> out((size_t)k_ * n_);
    gpu_.check(fc_dequant(h_, out.data(), out.size()));
    return out;
  }
  FcQWeight* raw() const { return h_; }
  const Gpu& gpu() const { return gpu_; }

 private:
  const Gpu& gpu_;
  FcQWeight* h_ = nullptr;
  uint32_t k_ = 0, n_ = 0;
  QKind kind_ = QKind::F32;
};

// y[rows, n] = x[rows, k] * W (ops/quant.rs:L326-L335)
inline std::vector<float> linear_q(const QWeight& w, const std::vector<float>& x, uint32_t rows,
                                   Mode mode = Mode::ExactF32) {
  if (x.size() != (size_t)rows * w.k()) throw Error(FC_ERR_SHAPE, "linear_q x has the wrong length");
  std::vector<float> y((size_t)rows * w.n());
  w.gpu().check(fc_qmatmul(w.raw(), x.data(), rows, y.data(), (int)mode));
  return y;
}

// Shared by both resident models.
class ResidentModel {
 public:
  virtual ~ResidentModel() {
    if (h_) fc_model_destroy(h_);
  }
  uint32_t pos(uint32_t stream = 0) const {
    uint32_t p = 0;
    gpu_.check(fc_model_pos(h_, stream, &p));
    return p;
  }
  void reset(uint32_t stream = 0) { gpu_.check(fc_model_reset(h_, stream)); }
  // feed (models/llama/mod.rs:L352-L438): one token in, the next-token logits row out
  std::vector<float> feed(int32_t token, uint32_t stream = 0) {
    std::vector<float> logits(vocab_);
    gpu_.check(fc_model_feed(h_, stream, token, logits.data(), nullptr));
    return logits;
  }
  int32_t feed_greedy(int32_t token, uint32_t stream = 0) {
    int32_t a = 0;
    gpu_.check(fc_model_feed(h_, stream, token, nullptr, &a));
    return a;
  }
  // `steps` greedy steps chained on the device: step 0 feeds `token`, every further step the previous pick
  // (the greedy branch of generate_with, engine/mod.rs:L230-L240, without a host round trip per token).
  std::vector<int32_t> decode_greedy(int32_t token, uint32_t steps, uint32_t stream = 0) {
    std::vector<int32_t> out(steps);
    gpu_.check(fc_model_decode_greedy(h_, 1, &stream, &token, steps, out.data()));
    return out;
  }
  // The candidates sampling::sample keeps for top_k = k (ferrum_model/src/sampling.rs:L44-L66) from the
  // logits row of the last decode step, selected on the device: (token, penalised logit) pairs in its order.
  std::vector<std::pair<int32_t, float>> topk(uint32_t k, uint32_t row = 0, float repetition_penalty = 1.0f,
                                              const std::vector<int32_t>& recent = {}) {
    std::vector<int32_t> idx(k);
    std::vector<float> val(k);
    uint32_t n = 0;
    gpu_.check(fc_model_topk(h_, row, k, repetition_penalty, recent.empty() ? nullptr : recent.data(),
                             (uint32_t)recent.size(), idx.data(), val.data(), &n));
    std::vector<std::pair<int32_t, float>> out(n);
    for (uint32_t i = 0; i < n; i++) out[i] = {idx[i], val[i]};
    return out;
  }
  // A whole prompt in one batched pass (the reference feeds it token by token, engine/mod.rs:L226-L229);
  // returns the last position's logits. Mode::TensorF16 needs an empty stream.
  std::vector<float> prefill(const std::vector<int32_t>& ids, uint32_t stream = 0, Mode mode = Mode::ExactF32) {
    std::vector<float> logits(vocab_);
    gpu_.check(fc_model_prefill(h_, stream, ids.data(), (uint32_t)ids.size(), logits.data(), nullptr, (int)mode));
    return logits;
  }
  // forward_all (models/llama/forward.rs:L13-L17)
  std::vector<float> forward_all(const std::vector<int32_t>& ids, Mode mode = Mode::ExactF32) {
    std::vector<float> logits(ids.size() * (size_t)vocab_);
    gpu_.check(fc_model_forward_all(h_, ids.data(), (uint32_t)ids.size(), logits.data(), (int)mode));
    return logits;
  }
  // score (models/llama/forward.rs:L74-L88): (log-probability, first-argmax flag) per position
  std::vector<std::pair<float, bool>> score(const std::vector<int32_t>& ids, Mode mode = Mode::ExactF32) {
    if (ids.size() < 2) throw Error(FC_ERR_SHAPE, "scoring needs at least 2 tokens");
    std::vector<float> lp(ids.size() - 1);
    std::vector<uint8_t> gr(ids.size() - 1);
    gpu_.check(fc_model_score(h_, ids.data(), 1, (uint32_t)ids.size(), (int)mode, lp.data(), gr.data(), nullptr));
    std::vector<std::pair<float, bool>> out;
    for (size_t i = 0; i < lp.size(); i++) out.emplace_back(lp[i], gr[i] != 0);
    return out;
  }
  FcModel* raw() const { return h_; }

 protected:
  explicit ResidentModel(const Gpu& gpu) : gpu_(gpu) {}
  const Gpu& gpu_;
  FcModel* h_ = nullptr;
  uint32_t vocab_ = 0;
};

class CudaLlama : public ResidentModel {
 public:
  // GpuLlama::new(gpu, model, quant, budget) (models/llama/mod.rs:L219-L314)
  CudaLlama(const Gpu& gpu, const FcLlamaConfig& cfg, const FcLlamaWeights& w, QKind quant, uint64_t budget = 0,
            uint32_t max_streams = 1)
      : ResidentModel(gpu) {
    gpu.check(fc_llama_create(gpu.raw(), &cfg, &w, (int)quant, max_streams, budget, &h_));
    vocab_ = cfg.vocab;
  }
};

class CudaGpt2 : public ResidentModel {
 public:
  CudaGpt2(const Gpu& gpu, const FcGpt2Config& cfg, const FcGpt2Weights& w, QKind quant, uint64_t budget = 0,
           uint32_t max_streams = 1)
      : ResidentModel(gpu) {
    gpu.check(fc_gpt2_create(gpu.raw(), &cfg, &w, (int)quant, max_streams, budget, &h_));
    vocab_ = cfg.vocab;
  }
};

// `Gpt2Feed<'a> = Box<dyn FnMut(usize) -> Result<Vec<f32>, String> + 'a>` (engine/mod.rs:L256)
using Feed = std::function<std::vector<float>(int32_t)>;

// impl Backend for a CUDA device (engine/mod.rs:L259-L312): kind / name / generate / decoders; train
// reports "not available" like the trait's defaults do.
class CudaBackend {
 public:
  explicit CudaBackend(int ordinal = 0, QKind weights = QKind::F32) : gpu_(ordinal), weights_(weights) {}
  const char* kind() const { return "cuda"; }
  std::string name() const { return gpu_.name(); }
  CudaBackend& with_weights(QKind q) {
    weights_ = q;
    return *this;
  }
  Feed llama_decoder(const FcLlamaConfig& cfg, const FcLlamaWeights& w) {
    auto m = std::make_shared<CudaLlama>(gpu_, cfg, w, weights_);
    return [m](int32_t t) { return m->feed(t); };
  }
  Feed gpt2_decoder(const FcGpt2Config& cfg, const FcGpt2Weights& w) {
    auto m = std::make_shared<CudaGpt2>(gpu_, cfg, w, weights_);
    return [m](int32_t t) { return m->feed(t); };
  }
  // generate_with (engine/mod.rs:L204-L242), greedy: feed each prompt token, then pick until `max_new` tokens are
  // out or the context is full; the last pick is not fed. Returns only the new tokens. The picks after the first
  // are chained on the device in one call.
  std::vector<int32_t> generate(const FcLlamaConfig& cfg, const FcLlamaWeights& w, const std::vector<int32_t>& prompt,
                                uint32_t max_new) {
    if (prompt.empty()) throw Error(FC_ERR_ARG, "the prompt is empty");
    if (prompt.size() >= cfg.ctx)
      throw Error(FC_ERR_CONTEXT_FULL, "the prompt has " + std::to_string(prompt.size()) + " tokens but the context is " +
                                           std::to_string(cfg.ctx));
    const uint32_t room = cfg.ctx - (uint32_t)prompt.size();
    if (max_new > room) max_new = room; // history reaches ctx: stop there
    CudaLlama m(gpu_, cfg, w, weights_);
    std::vector<int32_t> out;
    int32_t next = 0;
    for (int32_t t : prompt) next = m.feed_greedy(t);
    if (max_new == 0) return out;
    out.push_back(next);
    if (max_new > 1) {
      const auto rest = m.decode_greedy(next, max_new - 1);
      out.insert(out.end(), rest.begin(), rest.end());
    }
    return out;
  }
  [[noreturn]] void train() const { throw Error(FC_ERR_UNSUPPORTED, "training is not available on the cuda backend"); }
  const Gpu& gpu() const { return gpu_; }

 private:
  Gpu gpu_;
  QKind weights_;
};

} // namespace ferrum
