// Host entry points of the elementwise, attention and scoring kernels (f32 activations).
#pragma once
#include "common.cuh"

// K/V cache of one layer: [max_streams][kv_heads][ctx][hd] f32 each.
struct KvLayer {
  float* k = nullptr;
  float* v = nullptr;
};

struct RopeParams {
  const float* cos = nullptr; // [ctx][rope_dim/2], host-built (ferrum_ref/src/models/llama/ops.rs:L80-L101)
  const float* sin = nullptr;
  uint32_t rope_dim = 0;
  uint32_t type = FC_ROPE_NORM;
};

// elementwise.cu
int k_embed(FcDevice* dev, const float* tok, const float* pos_table /*nullable*/, const int32_t* ids,
            const int32_t* positions /*nullable unless pos_table*/, uint32_t rows, uint32_t d, float* x);
int k_rmsnorm(FcDevice* dev, const float* x, const float* g, uint32_t rows, uint32_t d, float eps, float* y);
int k_layernorm(FcDevice* dev, const float* x, const float* g, const float* b, uint32_t rows, uint32_t d, float* y);
int k_swiglu(FcDevice* dev, const float* gate_up /*[rows][2*hidden]*/, uint32_t rows, uint32_t hidden, uint32_t group, float* act);
int k_swiglu_split(FcDevice* dev, const float* gate_up, uint32_t rows, uint32_t mp, uint32_t hidden, uint32_t group, __half* xh,
                   __half* xl, const DeferredReduce* pending = nullptr); // gate_up's unfinished split-K sum: finished here
// Rotate q and k of the fused qkv rows in place (rope.type/rope_dim; skipped when rope.cos is
// NULL) and, when `kv` is given, store each row's k and v into the cache at (stream, position).
int k_rope_kv(FcDevice* dev, float* qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
              const RopeParams& rope, const int32_t* positions, const int32_t* streams /*nullable: row's cache slot*/,
              const KvLayer* kv, uint32_t ctx,
              const DeferredReduce* pending = nullptr); // an unfinished split-K sum of the qkv product: finished here
size_t argmax_scratch_bytes(uint32_t rows);
int k_argmax(FcDevice* dev, const float* logits, uint32_t rows, uint32_t vocab, int32_t* out, void* scratch = nullptr);
// nn::score on materialised logits in two steps: per-row partials over vocabulary columns
// [v0, v0 + vs) as (max, sum exp, target logit | -inf, first argmax), then the merge of n_shards.
int k_score_partial(FcDevice* dev, const float* logits, const int32_t* targets, uint32_t rows, uint32_t vs, uint32_t v0,
                    float* partial);
int k_score_combine(FcDevice* dev, const float* partials, uint32_t n_shards, uint32_t rows, const int32_t* targets,
                    float* logprob, uint8_t* greedy);
// Per-sequence -sum(logprob) in f64, ascending position.
int k_nll_sums(FcDevice* dev, const float* logprob, uint32_t n_seqs, uint32_t rows_per_seq, double* nll);

// attention.cu
// Decode: one query row per stream against that stream's cache, positions 0..=pos[row].
// `scratch` (attn_decode_scratch_bytes, nullable) enables the context-split kernel of
// attn_decode.cu; that kernel can write the result as the two fp16 terms [mp][heads*hd] of a following
// 9..64-row tensor-core product instead of `out` (xh, xl set).
int k_attn_decode(FcDevice* dev, const float* qkv, uint32_t q_stride, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                  uint32_t hd, const int32_t* positions, const int32_t* streams, const KvLayer& kv, uint32_t ctx,
                  float* out /*[rows][heads*hd]*/, float* scratch, __half* xh = nullptr, __half* xl = nullptr,
                  uint32_t mp = 0, bool append_kv = false,
                  // the context-split kernel only: fold the RoPE / cache launch into this one - finish the qkv
                  // product's pending split-K sum (nullable: none), rotate q and k by `rope`, append k and v
                  const DeferredReduce* qkv_pending = nullptr, const RopeParams* rope = nullptr);
// Whether k_attn_decode can store the rows' own k and v into the cache itself (`append_kv`): the
// context-split kernel does, for models whose k needs no rotation first.
bool attn_decode_appends(uint32_t heads, uint32_t kv_heads, uint32_t hd, const float* scratch);
// attn_decode.cu
bool attn_decode_split_supports(uint32_t heads, uint32_t kv_heads, uint32_t hd);
size_t attn_decode_scratch_bytes(const FcDevice* dev, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t ctx);
int k_attn_decode_split(FcDevice* dev, const float* qkv, uint32_t q_stride, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                        const int32_t* positions, const int32_t* streams, const KvLayer& kv, uint32_t ctx, float* scratch,
                        float* out, __half* xh, __half* xl, uint32_t mp, bool append, const DeferredReduce* qkv_pending = nullptr,
                        const RopeParams* rope = nullptr);
// Whether the launch can take the qkv product's pending sum and the rotation along (attn_decode.cu).
bool attn_decode_folds_rope(uint32_t heads, uint32_t kv_heads, uint32_t hd, const float* scratch, const DeferredReduce& pending,
                            const float* qkv, uint32_t rows);
// Stateless causal attention over `n_seqs` sequences of `t` rows in the fused qkv buffer (exact f32).
int k_attn_causal_f32(FcDevice* dev, const float* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                      uint32_t hd, float* out);
// Attention of `t` new rows of one stream over its cache (positions start..start+t), exact f32.
int k_attn_prefill_cache_f32(FcDevice* dev, const float* qkv, uint32_t t, uint32_t start, uint32_t heads,
                             uint32_t kv_heads, uint32_t hd, int32_t stream, const KvLayer& kv, uint32_t ctx, float* out);
