// Resident models: the CUDA counterpart of ferrum_wgpu's GpuLlama / GpuGpt2
// (ferrum_wgpu/src/models/llama/{mod,forward}.rs, models/gpt2.rs). One struct serves both
// architectures; `arch` switches the norm, the position treatment and the feed-forward.
#pragma once
#include "ops.cuh"

enum { ARCH_LLAMA = 0, ARCH_GPT2 = 1 };

struct Linear {
  FcQWeight* w = nullptr;
  float* bias = nullptr; // device, [n]; nullptr = none
};

struct Layer {
  float *norm1_g = nullptr, *norm1_b = nullptr, *norm2_g = nullptr, *norm2_b = nullptr;
  Linear qkv;  // rows: q heads, then k heads, then v heads
  Linear wo;
  Linear ff1;  // Llama: gate rows then up rows; GPT-2: w1
  Linear ff2;  // Llama: down; GPT-2: w2
  KvLayer kv;
};

// Grow-only device workspace for the batched passes.
struct Arena {
  char* base = nullptr;
  size_t cap = 0, off = 0;
};

struct FcModel {
  FcDevice* dev = nullptr;
  int arch = ARCH_LLAMA;
  int qkind = FC_F32;
  uint32_t vocab = 0, ctx = 0, dim = 0, heads = 0, kv_heads = 0, hd = 0, n_layers = 0, hidden = 0;
  float eps = 1e-5f;
  RopeParams rope;
  float *cos = nullptr, *sin = nullptr;
  float* tok = nullptr;       // [vocab][dim] f32 (stays f32: models/llama/mod.rs:L133,L303)
  float* pos_table = nullptr; // GPT-2 [ctx][dim]
  float *normf_g = nullptr, *normf_b = nullptr;
  Linear head;                // [vocab][dim]
  QMat head_view;             // the rows of `head` this rank owns
  uint32_t shard = 0, n_shards = 1, v0 = 0, v1 = 0;
  std::vector<Layer> layers;
  uint32_t gu_group = 0;      // gate/up rows of ff1 interleaved in groups of this many (0: not interleaved)
  uint32_t max_streams = 1;
  std::vector<uint32_t> pos;  // per stream
  uint64_t weight_bytes = 0;
  std::vector<void*> allocs;  // everything cudaMalloc'ed for this model except QWeights
  // decode scratch, sized for max_streams rows
  float *x = nullptr, *h = nullptr, *qkv = nullptr, *attn = nullptr, *ff = nullptr, *act = nullptr, *logits = nullptr;
  int32_t *d_ids = nullptr, *d_pos = nullptr, *d_streams = nullptr, *d_argmax = nullptr;
  void* argmax_scratch = nullptr; // keys and counters of the multi-CTA argmax, zero between launches
  // decode-step replay: one instantiated CUDA graph per batch width, inputs through a pinned buffer
  void* mma_scratch = nullptr; // scratch of the decode tensor product
  float* attn_scratch = nullptr; // per-split partials of the decode attention
  int32_t* pin_dec = nullptr;
  std::vector<cudaGraphExec_t> graphs;
  std::vector<uint64_t> graph_launches;
  std::vector<uint8_t> graph_warm;
  bool graph_ok = true;
  // device staging of fc_model_score's host buffers (ids up; log-probs, flags, sums down): kept between
  // calls and grown on demand - an allocation and a free per call cost more than the copies on some hosts
  void* score_stage = nullptr;
  size_t score_stage_bytes = 0;
  // chained greedy decode (fc_model_decode_greedy): the step that takes its tokens from the previous step's
  // argmax on the device, one graph per batch width; the tokens it consumed, in order; how many steps so far
  std::vector<cudaGraphExec_t> chain_graphs;
  std::vector<uint64_t> chain_launches;
  int32_t* d_chain_log = nullptr; // [ctx][max_streams]
  uint32_t* d_chain_cnt = nullptr;
  Arena arena;
  void* tc = nullptr; // state of the bf16 tensor-core path (built on first use)
  void* dc = nullptr; // state of the one-launch single-stream decode (decode_cluster.cu; probed on first use)

  uint32_t qd() const { return heads * hd; }
  uint32_t kvd() const { return kv_heads * hd; }
  uint32_t qkv_w() const { return qd() + 2 * kvd(); }
  uint32_t ff1_w() const { return arch == ARCH_LLAMA ? 2 * hidden : hidden; }
};

// Workspace helpers (model.cu)
int arena_reserve(FcModel* m, size_t bytes);
void* arena_take(FcModel* m, size_t bytes);

// Batched passes in exact f32 (model.cu).
// rows = n_seqs * t; ids/positions on the device; writes final-norm hidden states to `hidden_out`
// ([rows][dim]) when not NULL. Attention is stateless causal within each sequence.
int model_trunk_f32(FcModel* m, const int32_t* ids_dev, const int32_t* pos_dev, uint32_t n_seqs, uint32_t t,
                    float* hidden_out);

// bf16 tensor-core passes (model_tc.cu)
// `cache_stream` >= 0 (one sequence from position 0 only): every layer's rotated k and v also go into that
// stream's cache, so decode can continue from a prompt that went through the tensor-core passes.
int model_trunk_tc(FcModel* m, const int32_t* ids_dev, const int32_t* pos_dev, uint32_t n_seqs, uint32_t t,
                   __half* hidden_out, int32_t cache_stream = -1);
int model_head_partial_tc(FcModel* m, const __half* hidden, const int32_t* targets_dev, uint32_t rows,
                          float* partial);
int model_logits_tc(FcModel* m, const __half* hidden, uint32_t rows, float* logits);
void model_tc_free(FcModel* m);
size_t model_tc_trunk_bytes(const FcModel* m, size_t rows); // workspace model_trunk_tc takes from the arena
size_t model_tc_head_bytes(const FcModel* m, size_t rows);  // workspace model_head_partial_tc takes
int model_interleave_gate_up(FcDevice* dev, FcQWeight* w, uint32_t hidden, uint32_t group);
int tc_check_errors(FcDevice* dev);
// decode_cluster.cu: a small GPT-2-style model decodes one stream as one kernel per run of tokens
bool decode_cluster_ready(FcModel* m);
int k_decode_cluster(FcModel* m, uint32_t stream, uint32_t steps, bool chained);
void decode_cluster_free(FcModel* m);
