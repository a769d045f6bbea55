// Resident-model orchestration and its C ABI: upload (quantise + pack), KV-cached decode for one or
// many streams, batched prefill, stateless forward_all and scoring.
//
// Op order per layer follows the reference's resident models
// (ferrum_wgpu/src/models/llama/mod.rs:L352-L438, forward.rs:L18-L72, models/gpt2.rs:L192-L265)
// with the q/k/v products and the gate/up products each fused into one launch, bias / GELU /
// residual folded into the product's epilogue, and RoPE fused with the cache store:
//   norm -> qkv(+bias) -> rope+cache -> attention -> wo(+bias)+residual -> norm -> ff1(+bias, GELU)
//   [-> swiglu] -> ff2(+bias)+residual;   final norm -> head.
// That is 9 (Llama) / 8 (GPT-2) launches per layer against the reference's 18-21 / 15.
#include <cmath>
#include <cstring>

#include "model.cuh"

namespace {

int dev_alloc(FcModel* m, size_t bytes, void** out) {
  *out = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fc_fail(m->dev, FC_ERR_OOM, "cannot allocate %zu bytes: %s", bytes, cudaGetErrorString(e));
  }
  m->allocs.push_back(*out);
  return FC_OK;
}

int upload_f32(FcModel* m, const float* host, size_t n, float** out) {
  FC_TRY(dev_alloc(m, n * 4, (void**)out));
  FC_CUDA(m->dev, cudaMemcpyAsync(*out, host, n * 4, cudaMemcpyHostToDevice, m->dev->stream));
  FC_CUDA(m->dev, cudaStreamSynchronize(m->dev->stream));
  return FC_OK;
}

// Concatenated bias of fused projections; a missing part contributes zeros; all missing = none.
int upload_bias_concat(FcModel* m, const float* const* parts, const uint32_t* ns, int count, float** out) {
  *out = nullptr;
  bool any = false;
  size_t total = 0;
  for (int i = 0; i < count; i++) {
    any = any || parts[i];
    total += ns[i];
  }
  if (!any) return FC_OK;
  std::vector<float> hb(total, 0.0f);
  size_t off = 0;
  for (int i = 0; i < count; i++) {
    if (parts[i]) memcpy(hb.data() + off, parts[i], ns[i] * 4);
    off += ns[i];
  }
  return upload_f32(m, hb.data(), total, out);
}

void model_free(FcModel* m) {
  if (!m) return;
  cudaSetDevice(m->dev->ordinal);
  cudaStreamSynchronize(m->dev->stream);
  model_tc_free(m);
  decode_cluster_free(m);
  for (cudaGraphExec_t g : m->chain_graphs)
    if (g) cudaGraphExecDestroy(g);
  for (cudaGraphExec_t g : m->graphs)
    if (g) cudaGraphExecDestroy(g);
  if (m->pin_dec) cudaFreeHost(m->pin_dec);
  if (m->score_stage) cudaFree(m->score_stage);
  for (auto& l : m->layers) {
    qweight_free(l.qkv.w);
    qweight_free(l.wo.w);
    qweight_free(l.ff1.w);
    qweight_free(l.ff2.w);
  }
  qweight_free(m->head.w);
  for (void* p : m->allocs) cudaFree(p);
  if (m->arena.base) cudaFree(m->arena.base);
  delete m;
}

uint64_t matrix_bytes(int qkind, uint64_t k, uint64_t n) {
  qkind = effective_kind(qkind, k);
  if (qkind != FC_F32 && k % kind_block_elems(qkind) == 0) return qmat_qs_bytes(qkind, k, n) + qmat_sc_bytes(qkind, k, n);
  return k * n * 4;
}

struct Shape {
  int arch;
  uint64_t vocab, ctx, dim, heads, kv_heads, hd, layers, hidden, rope_dim;
};

// Named after models::llama::plan (ferrum_wgpu/src/models/llama/mod.rs:L108-L182): everything the
// resident model allocates.
uint64_t plan_bytes(const Shape& s, int qkind, uint64_t streams) {
  const uint64_t d = s.dim, qd = s.heads * s.hd, kvd = s.kv_heads * s.hd, hid = s.hidden;
  const uint64_t ff1 = s.arch == ARCH_LLAMA ? 2 * hid : hid;
  uint64_t b = s.vocab * d * 4;                                      // token table (f32)
  if (s.arch == ARCH_GPT2) b += s.ctx * d * 4;                       // position table
  if (s.arch == ARCH_LLAMA) b += 2 * s.ctx * (s.rope_dim / 2) * 4;   // rope tables
  uint64_t per = matrix_bytes(qkind, d, qd + 2 * kvd) + matrix_bytes(qkind, qd, d) + matrix_bytes(qkind, d, ff1) +
                 matrix_bytes(qkind, hid, d);
  per += 4 * d * 4 + (qd + 2 * kvd + d + ff1 + d) * 4;               // norms, biases (upper bound)
  per += 2 * streams * s.ctx * kvd * 4;                              // K and V caches
  b += per * s.layers;
  b += 2 * d * 4 + matrix_bytes(qkind, d, s.vocab);                  // final norm, head
  b += streams * (2 * d + (qd + 2 * kvd) + qd + ff1 + hid + s.vocab) * 4 + streams * 16; // decode scratch
  return b;
}

int check_budget(FcDevice* dev, uint64_t need, uint64_t budget) {
  size_t free_b = 0, total_b = 0;
  FC_CUDA(dev, cudaMemGetInfo(&free_b, &total_b));
  const uint64_t limit = budget ? budget : (uint64_t)free_b;
  if (need > limit)
    return fc_fail(dev, FC_ERR_OOM, "the model needs %llu bytes on the device, over the budget of %llu bytes",
                   (unsigned long long)need, (unsigned long long)limit);
  return FC_OK;
}

int alloc_common(FcModel* m) {
  const uint32_t s = m->max_streams;
  for (auto& l : m->layers) {
    const size_t kvb = (size_t)s * m->ctx * m->kvd() * 4;
    FC_TRY(dev_alloc(m, kvb, (void**)&l.kv.k));
    FC_TRY(dev_alloc(m, kvb, (void**)&l.kv.v));
    // caches start zeroed (models/llama/mod.rs:L266-L267)
    FC_CUDA(m->dev, cudaMemsetAsync(l.kv.k, 0, kvb, m->dev->stream));
    FC_CUDA(m->dev, cudaMemsetAsync(l.kv.v, 0, kvb, m->dev->stream));
  }
  FC_TRY(dev_alloc(m, (size_t)s * m->dim * 4, (void**)&m->x));
  FC_TRY(dev_alloc(m, (size_t)s * m->dim * 4, (void**)&m->h));
  FC_TRY(dev_alloc(m, (size_t)s * m->qkv_w() * 4, (void**)&m->qkv));
  FC_TRY(dev_alloc(m, (size_t)s * m->qd() * 4, (void**)&m->attn));
  FC_TRY(dev_alloc(m, (size_t)s * m->ff1_w() * 4, (void**)&m->ff));
  FC_TRY(dev_alloc(m, (size_t)s * m->hidden * 4, (void**)&m->act));
  FC_TRY(dev_alloc(m, (size_t)s * m->vocab * 4, (void**)&m->logits));
  FC_TRY(dev_alloc(m, (size_t)s * 4, (void**)&m->d_ids));
  FC_TRY(dev_alloc(m, (size_t)s * 4, (void**)&m->d_pos));
  FC_TRY(dev_alloc(m, (size_t)s * 4, (void**)&m->d_streams));
  FC_TRY(dev_alloc(m, (size_t)s * 4, (void**)&m->d_argmax));
  FC_TRY(dev_alloc(m, (size_t)m->ctx * s * 4, (void**)&m->d_chain_log));
  FC_TRY(dev_alloc(m, (size_t)s * 4 + 16, (void**)&m->d_chain_cnt));
  FC_TRY(dev_alloc(m, argmax_scratch_bytes(s), &m->argmax_scratch));
  FC_CUDA(m->dev, cudaMemsetAsync(m->argmax_scratch, 0, argmax_scratch_bytes(s), m->dev->stream));
  // partial results of the context-split decode attention: the largest need over every batch width
  if (attn_decode_split_supports(m->heads, m->kv_heads, m->hd)) {
    size_t need = 0;
    for (uint32_t rows = 1; rows <= s; rows++) {
      const size_t b = attn_decode_scratch_bytes(m->dev, rows, m->heads, m->kv_heads, m->ctx);
      need = b > need ? b : need;
    }
    FC_TRY(dev_alloc(m, need, (void**)&m->attn_scratch));
  }
  // scratch of the decode tensor product (x split + split-K partials), sized for the widest matrix
  {
    size_t need = qmatvec_mma_scratch_bytes(m->head.w->m.k, m->head.w->m.n);
    for (auto& l : m->layers)
      for (const FcQWeight* q : {l.qkv.w, l.wo.w, l.ff1.w, l.ff2.w}) {
        const size_t b = qmatvec_mma_scratch_bytes(q->m.k, q->m.n);
        need = b > need ? b : need;
      }
    // (the gate/up product may keep its partial sums behind the widest x terms: run_stack_f32)
    const size_t gu = qmatvec_mma_scratch_bytes(m->hidden > m->dim ? m->hidden : m->dim, m->ff1_w());
    need = gu > need ? gu : need;
    FC_TRY(dev_alloc(m, need, &m->mma_scratch));
  }
  m->pos.assign(s, 0);
  m->head_view = m->head.w->m;
  m->v0 = 0;
  m->v1 = m->vocab;
  m->weight_bytes = m->head.w->bytes;
  for (auto& l : m->layers) m->weight_bytes += l.qkv.w->bytes + l.wo.w->bytes + l.ff1.w->bytes + l.ff2.w->bytes;
  FC_CUDA(m->dev, cudaStreamSynchronize(m->dev->stream));
  return FC_OK;
}

// ---- the layer stack ------------------------------------------------------------------------------

enum AttnMode { ATTN_DECODE, ATTN_STATELESS, ATTN_PREFILL_CACHE };

struct PassBufs {
  float *x, *h, *qkv, *attn, *ff, *act;
};

// Run `rows` rows through embedding and all layers in exact f32; leaves the final-norm output in
// b.h (the residual stream in b.x when `final_norm` is false). ATTN_DECODE: each row is its own stream (streams[] = cache slots). ATTN_STATELESS: n_seqs
// sequences of t rows, no cache. ATTN_PREFILL_CACHE: t rows of one stream appended at `start`.
// "normalise the rows of x first" for a product (fused into the one-row matvec, a separate launch into
// b.h for the other kernels)
static void norm_before(const FcModel* m, Epilogue& e, const float* g, const float* bias, float* tmp) {
  e.norm = m->arch == ARCH_LLAMA ? NORM_RMS : NORM_LAYER;
  e.norm_g = g;
  e.norm_b = bias;
  e.norm_eps = m->eps;
  e.norm_tmp = tmp;
}

int run_stack_f32(FcModel* m, const PassBufs& b, const int32_t* ids, const int32_t* positions, const int32_t* streams,
                  uint32_t rows, AttnMode mode, uint32_t n_seqs, uint32_t t, uint32_t start, int32_t stream,
                  bool final_norm, DeferredReduce* tail = nullptr, bool embedded = false) {
  FcDevice* dev = m->dev;
  const uint32_t d = m->dim;
  if (!embedded) FC_TRY(k_embed(dev, m->tok, m->pos_table, ids, positions, rows, d, b.x)); // (else b.x holds the rows)
  // The two products that write the residual stream (wo, ff2) may leave their split-K sum to the norm
  // launch of the product that reads it next: `pend` is that unfinished sum, consumed (or finished on
  // its own) by the very next k_qlinear_f32.
  DeferredReduce pend, made;
  for (auto& l : m->layers) {
    Epilogue e_qkv;
    e_qkv.scratch = m->mma_scratch;
    e_qkv.bias = l.qkv.bias;
    e_qkv.pending = &pend;
    norm_before(m, e_qkv, l.norm1_g, l.norm1_b, b.h);
    DeferredReduce qkv_sum; // the RoPE / cache launch that follows finishes the qkv product's split-K sum
    e_qkv.defer_out = &qkv_sum;
    FC_TRY(k_qlinear_f32(dev, l.qkv.w->m, b.x, rows, b.qkv, e_qkv));
    pend = DeferredReduce();
    const bool to_cache = mode != ATTN_STATELESS;
    // Without RoPE the launch below would only copy k and v into the cache: the decode attention does that itself.
    const bool attn_appends =
        mode == ATTN_DECODE && !m->rope.cos && attn_decode_appends(m->heads, m->kv_heads, m->hd, m->attn_scratch);
    // With RoPE, the decode attention can take the rotation, the pending sum and the cache append along as well:
    // one launch less per layer.
    const bool attn_folds = mode == ATTN_DECODE && m->rope.cos &&
                            attn_decode_folds_rope(m->heads, m->kv_heads, m->hd, m->attn_scratch, qkv_sum, b.qkv, rows);
    if (attn_appends)
      FC_TRY(k_flush_deferred(dev, qkv_sum));
    else if (!attn_folds)
      FC_TRY(k_rope_kv(dev, b.qkv, rows, m->heads, m->kv_heads, m->hd, m->rope, positions, streams,
                       to_cache ? &l.kv : nullptr, m->ctx, &qkv_sum));
    Epilogue e_wo;
    if (mode == ATTN_DECODE) {
      __half *xh = nullptr, *xl = nullptr;
      uint32_t mp = 0;
      if (m->attn_scratch && qlinear_takes_wide_mma(l.wo.w->m, rows, m->mma_scratch)) {
        // the attention writes the output product's fp16 terms itself
        qmatvec_mma_split_ptrs(m->mma_scratch, rows, m->qd(), &xh, &xl, &mp);
        e_wo.presplit = true;
      }
      FC_TRY(k_attn_decode(dev, b.qkv, m->qkv_w(), rows, m->heads, m->kv_heads, m->hd, positions, streams, l.kv, m->ctx,
                           b.attn, m->attn_scratch, xh, xl, mp, attn_appends || attn_folds, attn_folds ? &qkv_sum : nullptr,
                           attn_folds ? &m->rope : nullptr));
    } else if (mode == ATTN_STATELESS)
      FC_TRY(k_attn_causal_f32(dev, b.qkv, n_seqs, t, m->heads, m->kv_heads, m->hd, b.attn));
    else
      FC_TRY(k_attn_prefill_cache_f32(dev, b.qkv, t, start, m->heads, m->kv_heads, m->hd, stream, l.kv, m->ctx, b.attn));
    e_wo.scratch = m->mma_scratch;
    e_wo.bias = l.wo.bias;
    e_wo.resid = b.x;
    made = DeferredReduce();
    e_wo.defer_out = &made;
    FC_TRY(k_qlinear_f32(dev, l.wo.w->m, b.attn, rows, b.x, e_wo));
    pend = made;
    Epilogue e_ff1;
    e_ff1.scratch = m->mma_scratch;
    e_ff1.bias = l.ff1.bias;
    e_ff1.act = m->arch == ARCH_GPT2 ? ACT_GELU : ACT_NONE;
    e_ff1.pending = &pend;
    norm_before(m, e_ff1, l.norm2_g, l.norm2_b, b.h);
    // When SwiGLU writes ff2's fp16 terms (below) it also finishes the gate/up product's split-K sum; the
    // partial sums then sit behind the widest x terms, clear of the ones SwiGLU writes.
    const bool swiglu_splits = m->arch == ARCH_LLAMA && qlinear_takes_wide_mma(l.ff2.w->m, rows, m->mma_scratch);
    DeferredReduce gu_sum;
    if (swiglu_splits) {
      e_ff1.defer_out = &gu_sum;
      const size_t widest = m->hidden > d ? m->hidden : d;
      e_ff1.partial_at = (float*)(((uintptr_t)m->mma_scratch + (size_t)2 * 64 * widest * 2 + 255) & ~(uintptr_t)255);
    }
    FC_TRY(k_qlinear_f32(dev, l.ff1.w->m, b.x, rows, b.ff, e_ff1));
    pend = DeferredReduce();
    const float* ff2_in = b.ff;
    Epilogue e_ff2;
    if (m->arch == ARCH_LLAMA) {
      if (swiglu_splits) { // SwiGLU writes the product's fp16 terms itself
        __half *xh, *xl;
        uint32_t mp;
        qmatvec_mma_split_ptrs(m->mma_scratch, rows, m->hidden, &xh, &xl, &mp);
        FC_TRY(k_swiglu_split(dev, b.ff, rows, mp, m->hidden, m->gu_group, xh, xl, &gu_sum));
        e_ff2.presplit = true;
      } else {
        FC_TRY(k_swiglu(dev, b.ff, rows, m->hidden, m->gu_group, b.act));
      }
      ff2_in = b.act;
    }
    e_ff2.scratch = m->mma_scratch;
    e_ff2.bias = l.ff2.bias;
    e_ff2.resid = b.x;
    made = DeferredReduce();
    e_ff2.defer_out = &made;
    FC_TRY(k_qlinear_f32(dev, l.ff2.w->m, ff2_in, rows, b.x, e_ff2));
    pend = made;
  }
  if (!final_norm && tail) { // the caller folds the norm, and the last unfinished sum, into the head product
    *tail = pend;
    return FC_OK;
  }
  FC_TRY(k_flush_deferred(dev, pend));
  if (!final_norm) return FC_OK;
  if (m->arch == ARCH_LLAMA)
    FC_TRY(k_rmsnorm(dev, b.x, m->normf_g, rows, d, m->eps, b.h));
  else
    FC_TRY(k_layernorm(dev, b.x, m->normf_g, m->normf_b, rows, d, b.h));
  return FC_OK;
}

int carve_pass(FcModel* m, uint32_t rows, PassBufs* b, size_t extra_bytes) {
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t need = al((size_t)rows * m->dim * 4) * 2 + al((size_t)rows * m->qkv_w() * 4) + al((size_t)rows * m->qd() * 4) +
                      al((size_t)rows * m->ff1_w() * 4) + al((size_t)rows * m->hidden * 4) + al(extra_bytes) + 4096;
  FC_TRY(arena_reserve(m, need));
  b->x = (float*)arena_take(m, (size_t)rows * m->dim * 4);
  b->h = (float*)arena_take(m, (size_t)rows * m->dim * 4);
  b->qkv = (float*)arena_take(m, (size_t)rows * m->qkv_w() * 4);
  b->attn = (float*)arena_take(m, (size_t)rows * m->qd() * 4);
  b->ff = (float*)arena_take(m, (size_t)rows * m->ff1_w() * 4);
  b->act = (float*)arena_take(m, (size_t)rows * m->hidden * 4);
  return FC_OK;
}

int check_ids(FcModel* m, const int32_t* ids, size_t n) {
  for (size_t i = 0; i < n; i++)
    if (ids[i] < 0 || (uint32_t)ids[i] >= m->vocab)
      return fc_fail(m->dev, FC_ERR_RANGE, "index %d is out of range for %u entries", ids[i], m->vocab);
  return FC_OK;
}

// positions 0..t-1 repeated n_seqs times, on the device
int upload_positions(FcModel* m, uint32_t n_seqs, uint32_t t, uint32_t start, int32_t* dst_dev) {
  void* pin;
  FC_TRY(fc_pinned(m->dev, (size_t)n_seqs * t * 4, &pin));
  int32_t* p = (int32_t*)pin;
  for (uint32_t s = 0; s < n_seqs; s++)
    for (uint32_t i = 0; i < t; i++) p[(size_t)s * t + i] = (int32_t)(start + i);
  FC_CUDA(m->dev, cudaMemcpyAsync(dst_dev, p, (size_t)n_seqs * t * 4, cudaMemcpyHostToDevice, m->dev->stream));
  FC_CUDA(m->dev, cudaStreamSynchronize(m->dev->stream)); // the pinned buffer is reused by the caller
  return FC_OK;
}

} // namespace

int arena_reserve(FcModel* m, size_t bytes) {
  m->arena.off = 0;
  if (bytes <= m->arena.cap) return FC_OK;
  FC_CUDA(m->dev, cudaStreamSynchronize(m->dev->stream));
  if (m->arena.base) cudaFree(m->arena.base);
  m->arena.base = nullptr;
  m->arena.cap = 0;
  cudaError_t e = cudaMalloc((void**)&m->arena.base, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fc_fail(m->dev, FC_ERR_OOM, "cannot allocate a %zu-byte workspace: %s", bytes, cudaGetErrorString(e));
  }
  m->arena.cap = bytes;
  return FC_OK;
}

void* arena_take(FcModel* m, size_t bytes) {
  void* p = m->arena.base + m->arena.off;
  m->arena.off += (bytes + 255) & ~(size_t)255;
  return p;
}

int model_trunk_f32(FcModel* m, const int32_t* ids_dev, const int32_t* pos_dev, uint32_t n_seqs, uint32_t t,
                    float* hidden_out) {
  // the caller has reserved the arena and carved nothing else after this call's buffers
  PassBufs b;
  const uint32_t rows = n_seqs * t;
  b.x = (float*)arena_take(m, (size_t)rows * m->dim * 4);
  b.h = hidden_out ? hidden_out : (float*)arena_take(m, (size_t)rows * m->dim * 4);
  b.qkv = (float*)arena_take(m, (size_t)rows * m->qkv_w() * 4);
  b.attn = (float*)arena_take(m, (size_t)rows * m->qd() * 4);
  b.ff = (float*)arena_take(m, (size_t)rows * m->ff1_w() * 4);
  b.act = (float*)arena_take(m, (size_t)rows * m->hidden * 4);
  return run_stack_f32(m, b, ids_dev, pos_dev, nullptr, rows, ATTN_STATELESS, n_seqs, t, 0, 0, true);
}

// ================================ C ABI ===========================================================

static bool valid_llama(const FcLlamaConfig* c) {
  if (!c) return false;
  const uint32_t dims[] = {c->vocab, c->ctx, c->dim, c->heads, c->kv_heads, c->head_dim, c->layers, c->hidden, c->rope_dim};
  for (uint32_t v : dims)
    if (v == 0) return false;
  if (c->heads % c->kv_heads) return false;
  if (c->rope_dim > c->head_dim || c->rope_dim % 2) return false;
  auto bad = [](float v) { return !std::isfinite(v) || v <= 0.0f; };
  if (bad(c->eps) || bad(c->rope_base) || bad(c->rope_linear_factor)) return false;
  if (c->n_freq_factors != 0 && (c->n_freq_factors != c->rope_dim / 2 || !c->freq_factors)) return false;
  return true;
}

static bool valid_gpt2(const FcGpt2Config* c) {
  if (!c) return false;
  const uint32_t dims[] = {c->vocab, c->ctx, c->dim, c->heads, c->layers, c->hidden};
  for (uint32_t v : dims)
    if (v == 0) return false;
  return c->dim % c->heads == 0;
}

FC_API uint64_t fc_llama_plan_bytes(const FcLlamaConfig* c, int qkind, uint32_t max_streams) {
  if (!valid_llama(c) || max_streams == 0) return 0;
  Shape s{ARCH_LLAMA, c->vocab, c->ctx, c->dim, c->heads, c->kv_heads, c->head_dim, c->layers, c->hidden, c->rope_dim};
  return plan_bytes(s, qkind, max_streams);
}

FC_API uint64_t fc_gpt2_plan_bytes(const FcGpt2Config* c, int qkind, uint32_t max_streams) {
  if (!valid_gpt2(c) || max_streams == 0) return 0;
  Shape s{ARCH_GPT2, c->vocab, c->ctx, c->dim, c->heads, c->heads, c->dim / c->heads, c->layers, c->hidden, 0};
  return plan_bytes(s, qkind, max_streams);
}

// The token table stays f32 on the device (models/llama/mod.rs:L133,L303): an f32 table is copied, a table that
// arrives as GGUF blocks is repacked and decoded there (bit-identical to quant::decode).
static int upload_table(FcModel* m, const FcTensor& t, uint32_t rows, uint32_t d, float** out) {
  if (t.kind == FC_F32) return upload_f32(m, (const float*)t.data, (size_t)rows * d, out);
  FcQWeight* q = nullptr;
  const WeightSrc src{t.data, t.kind};
  FC_TRY(qweight_from_parts(m->dev, t.kind, &src, &rows, 1, d, &q));
  int rc = dev_alloc(m, (size_t)rows * d * 4, (void**)out);
  if (rc == FC_OK) rc = k_dequant(m->dev, q->m, *out);
  if (rc == FC_OK && cudaStreamSynchronize(m->dev->stream) != cudaSuccess) rc = fc_fail(m->dev, FC_ERR_DEVICE, "decoding the token table failed");
  qweight_free(q);
  return rc;
}
static WeightSrc src_of(const FcTensor& t) { return WeightSrc{t.data, t.kind}; }

FC_API int fc_llama_create(FcDevice* dev, const FcLlamaConfig* c, const FcLlamaWeights* w, int qkind,
                           uint32_t max_streams, uint64_t budget_bytes, FcModel** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  if (!valid_llama(c)) return fc_fail(dev, FC_ERR_SHAPE, "invalid Llama configuration");
  if (!w || !w->tok || !w->blocks || !w->out_norm || !w->head) return fc_fail(dev, FC_ERR_ARG, "missing weights");
  std::vector<FcLlamaBlockT> blocks(c->layers);
  for (uint32_t i = 0; i < c->layers; i++) {
    const FcLlamaBlock& b = w->blocks[i];
    blocks[i] = FcLlamaBlockT{b.attn_norm, {b.wq, FC_F32}, b.bq, {b.wk, FC_F32}, b.bk, {b.wv, FC_F32}, b.bv, {b.wo, FC_F32},
                              b.ffn_norm,  {b.gate, FC_F32}, {b.up, FC_F32}, {b.down, FC_F32}};
  }
  const FcLlamaTensors t{{w->tok, FC_F32}, blocks.data(), w->out_norm, {w->head, FC_F32}};
  return fc_llama_create_from_tensors(dev, c, &t, qkind, max_streams, budget_bytes, out);
}

FC_API int fc_llama_create_from_tensors(FcDevice* dev, const FcLlamaConfig* c, const FcLlamaTensors* w, int qkind,
                                        uint32_t max_streams, uint64_t budget_bytes, FcModel** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  cudaSetDevice(dev->ordinal);
  if (!valid_llama(c)) return fc_fail(dev, FC_ERR_SHAPE, "invalid Llama configuration");
  if (!w || !w->tok.data || !w->blocks || !w->out_norm || !w->head.data) return fc_fail(dev, FC_ERR_ARG, "missing weights");
  if (max_streams == 0) return fc_fail(dev, FC_ERR_ARG, "max_streams must be positive");
  if (!kind_known(qkind)) return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", qkind);
  FC_TRY(check_budget(dev, fc_llama_plan_bytes(c, qkind, max_streams), budget_bytes)); // before any allocation
  FcModel* m = new FcModel();
  m->dev = dev;
  m->arch = ARCH_LLAMA;
  m->qkind = qkind;
  m->vocab = c->vocab, m->ctx = c->ctx, m->dim = c->dim, m->heads = c->heads, m->kv_heads = c->kv_heads;
  m->hd = c->head_dim, m->n_layers = c->layers, m->hidden = c->hidden, m->eps = c->eps;
  m->max_streams = max_streams;
  const uint32_t d = m->dim, qd = m->qd(), kvd = m->kvd(), hid = m->hidden;
  int rc = FC_OK;
  auto fail = [&](int code) {
    model_free(m);
    return code;
  };
  // RoPE tables on the host in the reference's precision (ferrum_ref/src/models/llama/ops.rs:L80-L101)
  {
    const uint32_t half = c->rope_dim / 2;
    std::vector<float> hc((size_t)c->ctx * half), hs((size_t)c->ctx * half);
    for (uint32_t p = 0; p < c->ctx; p++)
      for (uint32_t i = 0; i < half; i++) {
        const float freq = (float)std::pow((double)c->rope_base, -2.0 * (double)i / (double)c->rope_dim);
        const float ff = i < c->n_freq_factors ? c->freq_factors[i] : 1.0f;
        const float theta = (float)p * freq / ff * (1.0f / c->rope_linear_factor);
        hc[(size_t)p * half + i] = cosf(theta);
        hs[(size_t)p * half + i] = sinf(theta);
      }
    if ((rc = upload_f32(m, hc.data(), hc.size(), &m->cos)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, hs.data(), hs.size(), &m->sin)) != FC_OK) return fail(rc);
    m->rope.cos = m->cos, m->rope.sin = m->sin, m->rope.rope_dim = c->rope_dim, m->rope.type = c->rope_type;
  }
  if ((rc = upload_table(m, w->tok, c->vocab, d, &m->tok)) != FC_OK) return fail(rc);
  if ((rc = upload_f32(m, w->out_norm, d, &m->normf_g)) != FC_OK) return fail(rc);
  m->layers.resize(c->layers);
  for (uint32_t li = 0; li < c->layers; li++) {
    const FcLlamaBlockT& b = w->blocks[li];
    Layer& l = m->layers[li];
    if (!b.attn_norm || !b.wq.data || !b.wk.data || !b.wv.data || !b.wo.data || !b.ffn_norm || !b.gate.data || !b.up.data ||
        !b.down.data)
      return fail(fc_fail(dev, FC_ERR_ARG, "block %u is missing a tensor", li));
    if ((rc = upload_f32(m, b.attn_norm, d, &l.norm1_g)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.ffn_norm, d, &l.norm2_g)) != FC_OK) return fail(rc);
    const WeightSrc qkv_m[3] = {src_of(b.wq), src_of(b.wk), src_of(b.wv)};
    const uint32_t qkv_n[3] = {qd, kvd, kvd};
    if ((rc = qweight_from_parts(dev, qkind, qkv_m, qkv_n, 3, d, &l.qkv.w)) != FC_OK) return fail(rc);
    const float* qkv_b[3] = {b.bq, b.bk, b.bv};
    if ((rc = upload_bias_concat(m, qkv_b, qkv_n, 3, &l.qkv.bias)) != FC_OK) return fail(rc);
    const WeightSrc wo_m = src_of(b.wo), down_m = src_of(b.down);
    if ((rc = qweight_from_parts(dev, qkind, &wo_m, &d, 1, qd, &l.wo.w)) != FC_OK) return fail(rc);
    const WeightSrc gu_m[2] = {src_of(b.gate), src_of(b.up)};
    const uint32_t gu_n[2] = {hid, hid};
    if ((rc = qweight_from_parts(dev, qkind, gu_m, gu_n, 2, d, &l.ff1.w)) != FC_OK) return fail(rc);
    if (hid % 64 == 0) { // row 2i = gate i, row 2i + 1 = up i: the pair meets on neighbouring lanes of the tensor path's SwiGLU epilogue
      if ((rc = model_interleave_gate_up(dev, l.ff1.w, hid, 1)) != FC_OK) return fail(rc);
      m->gu_group = 1;
    }
    if ((rc = qweight_from_parts(dev, qkind, &down_m, &d, 1, hid, &l.ff2.w)) != FC_OK) return fail(rc);
  }
  {
    const WeightSrc head_m = src_of(w->head);
    const uint32_t vocab = c->vocab;
    if ((rc = qweight_from_parts(dev, qkind, &head_m, &vocab, 1, d, &m->head.w)) != FC_OK) return fail(rc);
  }
  if ((rc = alloc_common(m)) != FC_OK) return fail(rc);
  *out = m;
  return FC_OK;
}

FC_API int fc_gpt2_create(FcDevice* dev, const FcGpt2Config* c, const FcGpt2Weights* w, int qkind, uint32_t max_streams,
                          uint64_t budget_bytes, FcModel** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  if (!valid_gpt2(c)) return fc_fail(dev, FC_ERR_SHAPE, "invalid GPT-2 configuration");
  if (!w || !w->tok || !w->pos || !w->blocks || !w->lnf_g || !w->lnf_b || !w->head)
    return fc_fail(dev, FC_ERR_ARG, "missing weights");
  std::vector<FcGpt2BlockT> blocks(c->layers);
  for (uint32_t i = 0; i < c->layers; i++) {
    const FcGpt2Block& b = w->blocks[i];
    blocks[i] = FcGpt2BlockT{b.ln1_g, b.ln1_b, {b.wq, FC_F32}, b.bq, {b.wk, FC_F32}, b.bk, {b.wv, FC_F32}, b.bv, {b.wo, FC_F32}, b.bo,
                             b.ln2_g, b.ln2_b, {b.w1, FC_F32}, b.b1, {b.w2, FC_F32}, b.b2};
  }
  const FcGpt2Tensors t{{w->tok, FC_F32}, w->pos, blocks.data(), w->lnf_g, w->lnf_b, {w->head, FC_F32}};
  return fc_gpt2_create_from_tensors(dev, c, &t, qkind, max_streams, budget_bytes, out);
}

FC_API int fc_gpt2_create_from_tensors(FcDevice* dev, const FcGpt2Config* c, const FcGpt2Tensors* w, int qkind,
                                       uint32_t max_streams, uint64_t budget_bytes, FcModel** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  cudaSetDevice(dev->ordinal);
  if (!valid_gpt2(c)) return fc_fail(dev, FC_ERR_SHAPE, "invalid GPT-2 configuration");
  if (!w || !w->tok.data || !w->pos || !w->blocks || !w->lnf_g || !w->lnf_b || !w->head.data)
    return fc_fail(dev, FC_ERR_ARG, "missing weights");
  if (max_streams == 0) return fc_fail(dev, FC_ERR_ARG, "max_streams must be positive");
  if (!kind_known(qkind)) return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", qkind);
  FC_TRY(check_budget(dev, fc_gpt2_plan_bytes(c, qkind, max_streams), budget_bytes));
  FcModel* m = new FcModel();
  m->dev = dev;
  m->arch = ARCH_GPT2;
  m->qkind = qkind;
  m->vocab = c->vocab, m->ctx = c->ctx, m->dim = c->dim, m->heads = c->heads, m->kv_heads = c->heads;
  m->hd = c->dim / c->heads, m->n_layers = c->layers, m->hidden = c->hidden;
  m->max_streams = max_streams;
  const uint32_t d = m->dim, hid = m->hidden;
  int rc = FC_OK;
  auto fail = [&](int code) {
    model_free(m);
    return code;
  };
  if ((rc = upload_table(m, w->tok, c->vocab, d, &m->tok)) != FC_OK) return fail(rc);
  if ((rc = upload_f32(m, w->pos, (size_t)c->ctx * d, &m->pos_table)) != FC_OK) return fail(rc);
  if ((rc = upload_f32(m, w->lnf_g, d, &m->normf_g)) != FC_OK) return fail(rc);
  if ((rc = upload_f32(m, w->lnf_b, d, &m->normf_b)) != FC_OK) return fail(rc);
  m->layers.resize(c->layers);
  for (uint32_t li = 0; li < c->layers; li++) {
    const FcGpt2BlockT& b = w->blocks[li];
    Layer& l = m->layers[li];
    const void* need[] = {b.ln1_g, b.ln1_b, b.wq.data, b.bq, b.wk.data, b.bk, b.wv.data, b.bv, b.wo.data, b.bo, b.ln2_g, b.ln2_b,
                          b.w1.data, b.b1, b.w2.data, b.b2};
    for (const void* p : need)
      if (!p) return fail(fc_fail(dev, FC_ERR_ARG, "block %u is missing a tensor", li));
    if ((rc = upload_f32(m, b.ln1_g, d, &l.norm1_g)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.ln1_b, d, &l.norm1_b)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.ln2_g, d, &l.norm2_g)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.ln2_b, d, &l.norm2_b)) != FC_OK) return fail(rc);
    const WeightSrc qkv_m[3] = {src_of(b.wq), src_of(b.wk), src_of(b.wv)};
    const uint32_t qkv_n[3] = {d, d, d};
    if ((rc = qweight_from_parts(dev, qkind, qkv_m, qkv_n, 3, d, &l.qkv.w)) != FC_OK) return fail(rc);
    const float* qkv_b[3] = {b.bq, b.bk, b.bv};
    if ((rc = upload_bias_concat(m, qkv_b, qkv_n, 3, &l.qkv.bias)) != FC_OK) return fail(rc);
    const WeightSrc wo_m = src_of(b.wo), w1_m = src_of(b.w1), w2_m = src_of(b.w2);
    if ((rc = qweight_from_parts(dev, qkind, &wo_m, &d, 1, d, &l.wo.w)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.bo, d, &l.wo.bias)) != FC_OK) return fail(rc);
    if ((rc = qweight_from_parts(dev, qkind, &w1_m, &hid, 1, d, &l.ff1.w)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.b1, hid, &l.ff1.bias)) != FC_OK) return fail(rc);
    if ((rc = qweight_from_parts(dev, qkind, &w2_m, &d, 1, hid, &l.ff2.w)) != FC_OK) return fail(rc);
    if ((rc = upload_f32(m, b.b2, d, &l.ff2.bias)) != FC_OK) return fail(rc);
  }
  {
    const WeightSrc head_m = src_of(w->head);
    const uint32_t vocab = c->vocab;
    if ((rc = qweight_from_parts(dev, qkind, &head_m, &vocab, 1, d, &m->head.w)) != FC_OK) return fail(rc);
  }
  if ((rc = alloc_common(m)) != FC_OK) return fail(rc);
  *out = m;
  return FC_OK;
}

FC_API int fc_model_destroy(FcModel* m) {
  if (!m) return FC_ERR_ARG;
  model_free(m);
  return FC_OK;
}

FC_API int fc_model_pos(FcModel* m, uint32_t stream_id, uint32_t* pos_out) {
  if (!m || !pos_out) return FC_ERR_ARG;
  if (stream_id >= m->max_streams) return fc_fail(m->dev, FC_ERR_RANGE, "stream %u of %u", stream_id, m->max_streams);
  *pos_out = m->pos[stream_id];
  return FC_OK;
}

FC_API int fc_model_reset(FcModel* m, uint32_t stream_id) {
  if (!m) return FC_ERR_ARG;
  if (stream_id >= m->max_streams) return fc_fail(m->dev, FC_ERR_RANGE, "stream %u of %u", stream_id, m->max_streams);
  m->pos[stream_id] = 0;
  return FC_OK;
}

FC_API int fc_model_info(FcModel* m, uint32_t* vocab, uint32_t* ctx, uint32_t* max_streams, int* qkind,
                         uint64_t* weight_bytes) {
  if (!m) return FC_ERR_ARG;
  if (vocab) *vocab = m->vocab;
  if (ctx) *ctx = m->ctx;
  if (max_streams) *max_streams = m->max_streams;
  if (qkind) *qkind = m->qkind;
  if (weight_bytes) *weight_bytes = m->weight_bytes;
  return FC_OK;
}

FC_API int fc_model_feed_batch(FcModel* m, uint32_t n, const uint32_t* stream_ids, const int32_t* tokens,
                               float* logits_out, int32_t* argmax_out) {
  if (!m || !stream_ids || !tokens) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (n == 0) return FC_OK;
  if (n > m->max_streams) return fc_fail(dev, FC_ERR_SHAPE, "%u rows for a model of %u streams", n, m->max_streams);
  if (m->n_shards != 1) return fc_fail(dev, FC_ERR_UNSUPPORTED, "decode needs the whole head on this device");
  std::vector<uint8_t> seen(m->max_streams, 0);
  for (uint32_t i = 0; i < n; i++) {
    if (stream_ids[i] >= m->max_streams) return fc_fail(dev, FC_ERR_RANGE, "stream %u of %u", stream_ids[i], m->max_streams);
    if (seen[stream_ids[i]]) return fc_fail(dev, FC_ERR_ARG, "stream %u appears twice in one step", stream_ids[i]);
    seen[stream_ids[i]] = 1;
    if (m->pos[stream_ids[i]] >= m->ctx) return fc_fail(dev, FC_ERR_CONTEXT_FULL, "context of %u tokens is full", m->ctx);
  }
  FC_TRY(check_ids(m, tokens, n));
  // The step's variable inputs (token, position, cache slot per row) travel through one pinned
  // buffer owned by the model, so the whole step is a fixed sequence of launches and copies: after
  // one eager step per batch width it is captured into a CUDA graph and replayed (a decode step is
  // ~50-220 dependent launches of a few microseconds each, so launch overhead, not bandwidth, sets
  // its time at small widths). Fault injection and per-kernel profiling use the eager path.
  if (!m->pin_dec) FC_CUDA(dev, cudaMallocHost((void**)&m->pin_dec, (size_t)m->max_streams * 16));
  int32_t* p = m->pin_dec;
  for (uint32_t i = 0; i < n; i++) {
    p[i] = tokens[i];
    p[n + i] = (int32_t)m->pos[stream_ids[i]];
    p[2 * n + i] = (int32_t)stream_ids[i];
  }
  // One stream of a small GPT-2-style model: the whole step is one cluster kernel (decode_cluster.cu).
  if (n == 1 && m->n_shards == 1 && decode_cluster_ready(m)) {
    FC_CUDA(dev, cudaMemcpyAsync(m->d_ids, p, 4, cudaMemcpyHostToDevice, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(m->d_pos, p + 1, 4, cudaMemcpyHostToDevice, dev->stream));
    FC_TRY(k_decode_cluster(m, stream_ids[0], 1, false));
    FC_CUDA(dev, cudaMemcpyAsync(p + 3, m->d_argmax, 4, cudaMemcpyDeviceToHost, dev->stream));
    if (logits_out)
      FC_CUDA(dev, cudaMemcpyAsync(logits_out, m->logits, (size_t)m->vocab * 4, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (argmax_out) argmax_out[0] = p[3];
    m->pos[stream_ids[0]]++;
    return FC_OK;
  }
  auto enqueue_step = [&]() -> int {
    FC_CUDA(dev, cudaMemcpyAsync(m->d_ids, p, n * 4, cudaMemcpyHostToDevice, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(m->d_pos, p + n, n * 4, cudaMemcpyHostToDevice, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(m->d_streams, p + 2 * n, n * 4, cudaMemcpyHostToDevice, dev->stream));
    PassBufs b{m->x, m->h, m->qkv, m->attn, m->ff, m->act};
    DeferredReduce tail;
    FC_TRY(run_stack_f32(m, b, m->d_ids, m->d_pos, m->d_streams, n, ATTN_DECODE, 0, 0, 0, 0, false, &tail));
    Epilogue e_head;
    e_head.scratch = m->mma_scratch;
    e_head.pending = &tail;
    norm_before(m, e_head, m->normf_g, m->normf_b, m->h);
    FC_TRY(k_qlinear_f32(dev, m->head_view, m->x, n, m->logits, e_head));
    FC_TRY(k_argmax(dev, m->logits, n, m->vocab, m->d_argmax, m->argmax_scratch));
    FC_CUDA(dev, cudaMemcpyAsync(p + 3 * n, m->d_argmax, n * 4, cudaMemcpyDeviceToHost, dev->stream));
    return FC_OK;
  };
  if (m->graphs.size() <= n) {
    m->graphs.resize(n + 1, nullptr);
    m->graph_launches.resize(n + 1, 0);
    m->graph_warm.resize(n + 1, 0);
  }
  const bool graph_mode = m->graph_ok && dev->fail_after < 0 && !dev->profiling;
  if (graph_mode && m->graphs[n]) {
    FC_CUDA(dev, cudaGraphLaunch(m->graphs[n], dev->stream));
    dev->launches += m->graph_launches[n];
  } else if (graph_mode && m->graph_warm[n]) {
    const uint64_t l0 = dev->launches;
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
    int rc = ok ? enqueue_step() : FC_OK;
    if (ok) ok = cudaStreamEndCapture(dev->stream, &graph) == cudaSuccess && rc == FC_OK && graph;
    if (ok) ok = cudaGraphInstantiate(&m->graphs[n], graph, 0) == cudaSuccess;
    if (graph) cudaGraphDestroy(graph);
    if (ok) {
      m->graph_launches[n] = dev->launches - l0;
      FC_CUDA(dev, cudaGraphLaunch(m->graphs[n], dev->stream));
    } else { // capture is an optimisation: without it the step runs as plain launches
      cudaGetLastError();
      m->graphs[n] = nullptr;
      m->graph_ok = false;
      dev->launches = l0;
      FC_TRY(enqueue_step());
    }
  } else {
    FC_TRY(enqueue_step());
    m->graph_warm[n] = 1;
  }
  if (logits_out)
    FC_CUDA(dev, cudaMemcpyAsync(logits_out, m->logits, (size_t)n * m->vocab * 4, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (argmax_out) memcpy(argmax_out, p + 3 * n, n * 4);
  for (uint32_t i = 0; i < n; i++) m->pos[stream_ids[i]]++; // only a step that fully succeeded advances
  return FC_OK;
}

// The link of a chained greedy step: the previous step's picks become this step's tokens (and are logged),
// every row moves one position on.
__global__ void chain_advance_kernel(const int32_t* __restrict__ argmax, int32_t* __restrict__ ids, int32_t* __restrict__ pos,
                                     int32_t* __restrict__ log, uint32_t* __restrict__ cnt, uint32_t n) {
  const uint32_t r = threadIdx.x, step = *cnt;
  __syncthreads(); // everyone has read the counter before it moves
  if (r < n) {
    const int32_t tok = argmax[r];
    ids[r] = tok;
    pos[r] += 1;
    log[(size_t)step * n + r] = tok;
  }
  if (r == 0) *cnt = step + 1;
}

// The link for vocabularies one CTA scans quickly: it also takes the pick itself (first maximum, NaN never
// wins - the rule of argmax_kernel) from the previous step's logits and writes the embedding row, which
// saves the argmax and the embedding launch of every chained step. One CTA per row, one counter per row.
__global__ void __launch_bounds__(256)
    chain_link_kernel(const float* __restrict__ logits, uint32_t vocab, const float* __restrict__ tok_table,
                      const float* __restrict__ pos_table, uint32_t d, int32_t* __restrict__ argmax, int32_t* __restrict__ ids,
                      int32_t* __restrict__ pos, int32_t* __restrict__ log, uint32_t* __restrict__ cnt, uint32_t n,
                      float* __restrict__ x) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  __shared__ int s_tok, s_pos;
  const uint32_t r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best) best = v, idx = (int)i;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
  }
  if (lane == 0) bv[warp] = best, bi[warp] = idx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++)
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) best = bv[w], idx = bi[w];
    const int tok = idx == 0x7fffffff ? 0 : idx;
    const uint32_t step = cnt[r];
    cnt[r] = step + 1;
    argmax[r] = tok;
    ids[r] = tok;
    s_pos = pos[r] + 1;
    pos[r] = s_pos;
    log[(size_t)step * n + r] = tok;
    s_tok = tok;
  }
  __syncthreads();
  const float* src = tok_table + (size_t)s_tok * d;
  const float* ps = pos_table ? pos_table + (size_t)s_pos * d : nullptr;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)r * d + i] = ps ? src[i] + ps[i] : src[i];
}

FC_API int fc_model_decode_greedy(FcModel* m, uint32_t n, const uint32_t* stream_ids, const int32_t* first_tokens, uint32_t steps,
                                  int32_t* tokens_out) {
  if (!m || !stream_ids || !first_tokens || !tokens_out) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (n == 0 || steps == 0) return FC_OK;
  if (n > m->max_streams || n > 1024) return fc_fail(dev, FC_ERR_SHAPE, "%u rows for a model of %u streams", n, m->max_streams);
  for (uint32_t i = 0; i < n; i++) {
    if (stream_ids[i] >= m->max_streams) return fc_fail(dev, FC_ERR_RANGE, "stream %u of %u", stream_ids[i], m->max_streams);
    if ((uint64_t)m->pos[stream_ids[i]] + steps > m->ctx) // (64 bits: a step count near 2^32 must not wrap)
      return fc_fail(dev, FC_ERR_CONTEXT_FULL, "context of %u tokens is full", m->ctx);
  }
  // the first step takes its tokens from the host like any other (and checks streams and ids)
  FC_TRY(fc_model_feed_batch(m, n, stream_ids, first_tokens, nullptr, tokens_out));
  if (steps == 1) return FC_OK;
  if (n == 1 && m->n_shards == 1 && decode_cluster_ready(m)) {
    // the remaining steps in one launch: the kernel takes each pick as the next token itself
    FC_CUDA(dev, cudaMemsetAsync(m->d_chain_cnt, 0, 4, dev->stream));
    FC_TRY(k_decode_cluster(m, stream_ids[0], steps - 1, true));
    if (steps > 2)
      FC_CUDA(dev, cudaMemcpyAsync(tokens_out + 1, m->d_chain_log + 1, (size_t)(steps - 2) * 4, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(tokens_out + (steps - 1), m->d_argmax, 4, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    m->pos[stream_ids[0]] += steps - 1;
    return FC_OK;
  }
  const bool graph_mode = m->graph_ok && dev->fail_after < 0 && !dev->profiling;
  if (!graph_mode) { // fault injection and per-kernel profiling step on the host
    for (uint32_t s = 1; s < steps; s++)
      FC_TRY(fc_model_feed_batch(m, n, stream_ids, tokens_out + (size_t)(s - 1) * n, nullptr, tokens_out + (size_t)s * n));
    return FC_OK;
  }
  // Steps 1 .. steps-1 run back to back on the device: d_ids / d_pos / d_streams still hold step 0's rows and
  // d_argmax its picks; each further step starts with the link kernel instead of host copies, and the host
  // waits once at the end.
  const bool fused_link = m->vocab <= 8192; // the link scans the logits row itself
  auto enqueue_link = [&]() -> int {
    if (fused_link)
      FC_LAUNCH(dev, "chain_link",
                chain_link_kernel<<<n, 256, 0, dev->stream>>>(m->logits, m->vocab, m->tok, m->pos_table, m->dim, m->d_argmax, m->d_ids,
                                                              m->d_pos, m->d_chain_log, m->d_chain_cnt, n, m->x));
    else
      FC_LAUNCH(dev, "chain_advance",
                chain_advance_kernel<<<1, 1024, 0, dev->stream>>>(m->d_argmax, m->d_ids, m->d_pos, m->d_chain_log, m->d_chain_cnt, n));
    PassBufs b{m->x, m->h, m->qkv, m->attn, m->ff, m->act};
    DeferredReduce tail;
    FC_TRY(run_stack_f32(m, b, m->d_ids, m->d_pos, m->d_streams, n, ATTN_DECODE, 0, 0, 0, 0, false, &tail, fused_link));
    Epilogue e_head;
    e_head.scratch = m->mma_scratch;
    e_head.pending = &tail;
    norm_before(m, e_head, m->normf_g, m->normf_b, m->h);
    FC_TRY(k_qlinear_f32(dev, m->head_view, m->x, n, m->logits, e_head));
    if (!fused_link) FC_TRY(k_argmax(dev, m->logits, n, m->vocab, m->d_argmax, m->argmax_scratch));
    return FC_OK;
  };
  if (m->chain_graphs.size() <= n) {
    m->chain_graphs.resize(n + 1, nullptr);
    m->chain_launches.resize(n + 1, 0);
  }
  FC_CUDA(dev, cudaMemsetAsync(m->d_chain_cnt, 0, (size_t)m->max_streams * 4, dev->stream));
  uint32_t done = 1;
  if (!m->chain_graphs[n]) {
    const uint64_t l0 = dev->launches;
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
    int rc = ok ? enqueue_link() : FC_OK;
    if (ok) ok = cudaStreamEndCapture(dev->stream, &graph) == cudaSuccess && rc == FC_OK && graph;
    if (ok) ok = cudaGraphInstantiate(&m->chain_graphs[n], graph, 0) == cudaSuccess;
    if (graph) cudaGraphDestroy(graph);
    if (ok) {
      m->chain_launches[n] = dev->launches - l0;
      dev->launches = l0;
    } else { // without the graph the steps go through the host one by one
      cudaGetLastError();
      m->chain_graphs[n] = nullptr;
      dev->launches = l0;
      for (uint32_t s = 1; s < steps; s++)
        FC_TRY(fc_model_feed_batch(m, n, stream_ids, tokens_out + (size_t)(s - 1) * n, nullptr, tokens_out + (size_t)s * n));
      return FC_OK;
    }
  }
  for (; done < steps; done++) {
    FC_CUDA(dev, cudaGraphLaunch(m->chain_graphs[n], dev->stream));
    dev->launches += m->chain_launches[n];
  }
  // the log holds the tokens the links consumed: the picks of steps 0 .. steps-2; the last picks are in d_argmax
  if (fused_link) FC_TRY(k_argmax(dev, m->logits, n, m->vocab, m->d_argmax, m->argmax_scratch)); // (of the last step)
  if (steps > 2)
    FC_CUDA(dev, cudaMemcpyAsync(tokens_out + n, m->d_chain_log + n, (size_t)(steps - 2) * n * 4, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaMemcpyAsync(tokens_out + (size_t)(steps - 1) * n, m->d_argmax, (size_t)n * 4, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  for (uint32_t i = 0; i < n; i++) m->pos[stream_ids[i]] += steps - 1; // (step 0 advanced them once already)
  return FC_OK;
}

FC_API int fc_model_feed(FcModel* m, uint32_t stream_id, int32_t token, float* logits_out, int32_t* argmax_out) {
  return fc_model_feed_batch(m, 1, &stream_id, &token, logits_out, argmax_out);
}

// ids to the device workspace; returns the device pointer
static int upload_ids(FcModel* m, const int32_t* ids, size_t n, int32_t* dst_dev) {
  FC_CUDA(m->dev, cudaMemcpyAsync(dst_dev, ids, n * 4, cudaMemcpyHostToDevice, m->dev->stream));
  return FC_OK;
}

FC_API int fc_model_prefill(FcModel* m, uint32_t stream_id, const int32_t* ids, uint32_t n, float* logits_out,
                            int32_t* argmax_out, int mode) {
  if (!m || !ids) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (stream_id >= m->max_streams) return fc_fail(dev, FC_ERR_RANGE, "stream %u of %u", stream_id, m->max_streams);
  if (n == 0) return FC_OK;
  if (mode != FC_EXACT_F32 && mode != FC_TENSOR_F16) return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
  if (m->n_shards != 1) return fc_fail(dev, FC_ERR_UNSUPPORTED, "prefill needs the whole head on this device");
  const uint32_t start = m->pos[stream_id];
  if ((uint64_t)start + n > m->ctx) return fc_fail(dev, FC_ERR_CONTEXT_FULL, "context of %u tokens is full", m->ctx);
  FC_TRY(check_ids(m, ids, n));
  if (mode == FC_TENSOR_F16) {
    // The prompt goes through the scoring kernels (fp16 operands, f32 accumulation) and leaves its rotated
    // k and v in the stream's f32 cache; the stream must be empty (the causal kernel sees the prompt only).
    if (start != 0)
      return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-core prefill fills an empty stream: stream %u holds %u tokens", stream_id,
                     start);
    FC_TRY(arena_reserve(m, (size_t)n * 8 + 512 + (size_t)n * m->dim * 2 + 256 + model_tc_trunk_bytes(m, n) + 4096));
    int32_t* t_ids = (int32_t*)arena_take(m, (size_t)n * 4);
    int32_t* t_pos = (int32_t*)arena_take(m, (size_t)n * 4);
    __half* hid = (__half*)arena_take(m, (size_t)n * m->dim * 2);
    FC_TRY(upload_positions(m, 1, n, 0, t_pos));
    FC_TRY(upload_ids(m, ids, n, t_ids));
    FC_TRY(model_trunk_tc(m, t_ids, t_pos, 1, n, hid, (int32_t)stream_id));
    if (logits_out || argmax_out) {
      FC_TRY(model_logits_tc(m, hid + (size_t)(n - 1) * m->dim, 1, m->logits));
      if (argmax_out) {
        FC_TRY(k_argmax(dev, m->logits, 1, m->vocab, m->d_argmax, m->argmax_scratch));
        FC_CUDA(dev, cudaMemcpyAsync(argmax_out, m->d_argmax, 4, cudaMemcpyDeviceToHost, dev->stream));
      }
      if (logits_out)
        FC_CUDA(dev, cudaMemcpyAsync(logits_out, m->logits, (size_t)m->vocab * 4, cudaMemcpyDeviceToHost, dev->stream));
    }
    FC_TRY(tc_check_errors(dev));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    m->pos[stream_id] = n;
    return FC_OK;
  }
  PassBufs b;
  FC_TRY(carve_pass(m, n, &b, (size_t)n * 12 + 768));
  int32_t* d_ids = (int32_t*)arena_take(m, (size_t)n * 4);
  int32_t* d_pos = (int32_t*)arena_take(m, (size_t)n * 4);
  int32_t* d_slots = (int32_t*)arena_take(m, (size_t)n * 4); // every row writes the same stream's cache
  void* pin;
  FC_TRY(fc_pinned(dev, (size_t)n * 4, &pin));
  for (uint32_t i = 0; i < n; i++) ((int32_t*)pin)[i] = (int32_t)stream_id;
  FC_CUDA(dev, cudaMemcpyAsync(d_slots, pin, (size_t)n * 4, cudaMemcpyHostToDevice, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  FC_TRY(upload_positions(m, 1, n, start, d_pos));
  FC_TRY(upload_ids(m, ids, n, d_ids));
  FC_TRY(run_stack_f32(m, b, d_ids, d_pos, d_slots, n, ATTN_PREFILL_CACHE, 1, n, start, (int32_t)stream_id, true));
  if (logits_out || argmax_out) {
    FC_TRY(k_qlinear_f32(dev, m->head_view, b.h + (size_t)(n - 1) * m->dim, 1, m->logits, Epilogue()));
    if (argmax_out) {
      FC_TRY(k_argmax(dev, m->logits, 1, m->vocab, m->d_argmax, m->argmax_scratch));
      FC_CUDA(dev, cudaMemcpyAsync(argmax_out, m->d_argmax, 4, cudaMemcpyDeviceToHost, dev->stream));
    }
    if (logits_out)
      FC_CUDA(dev, cudaMemcpyAsync(logits_out, m->logits, (size_t)m->vocab * 4, cudaMemcpyDeviceToHost, dev->stream));
  }
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  m->pos[stream_id] = start + n;
  return FC_OK;
}

FC_API int fc_model_forward_all(FcModel* m, const int32_t* ids, uint32_t n, float* logits_out, int mode) {
  if (!m || !ids || !logits_out) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (n == 0 || n > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", n, m->ctx);
  if (m->n_shards != 1) return fc_fail(dev, FC_ERR_UNSUPPORTED, "forward_all needs the whole head on this device");
  FC_TRY(check_ids(m, ids, n));
  const size_t extra = (size_t)n * 8 + 512 + (size_t)n * m->vocab * 4 + 256 + (size_t)n * m->dim * 2 + 256 +
                       (mode == FC_TENSOR_F16 ? model_tc_trunk_bytes(m, n) : 0);
  PassBufs b;
  FC_TRY(carve_pass(m, n, &b, extra));
  int32_t* d_ids = (int32_t*)arena_take(m, (size_t)n * 4);
  int32_t* d_pos = (int32_t*)arena_take(m, (size_t)n * 4);
  float* logits = (float*)arena_take(m, (size_t)n * m->vocab * 4);
  FC_TRY(upload_positions(m, 1, n, 0, d_pos));
  FC_TRY(upload_ids(m, ids, n, d_ids));
  if (mode == FC_EXACT_F32) {
    FC_TRY(run_stack_f32(m, b, d_ids, d_pos, nullptr, n, ATTN_STATELESS, 1, n, 0, 0, true));
    FC_TRY(k_qlinear_f32(dev, m->head_view, b.h, n, logits, Epilogue()));
  } else if (mode == FC_TENSOR_F16) {
    __half* hid = (__half*)arena_take(m, (size_t)n * m->dim * 2);
    FC_TRY(model_trunk_tc(m, d_ids, d_pos, 1, n, hid));
    FC_TRY(model_logits_tc(m, hid, n, logits));
    FC_TRY(tc_check_errors(dev));
  } else {
    return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
  }
  FC_CUDA(dev, cudaMemcpyAsync(logits_out, logits, (size_t)n * m->vocab * 4, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FC_OK;
}

// Scoring of sequences already on the device. Sequences are processed in chunks that bound the
// workspace; every chunk runs trunk -> head partials -> combine.
FC_API int fc_model_score_dev(FcModel* m, const int32_t* ids_dev, uint32_t n_seqs, uint32_t seq_len, int mode,
                              float* logprob_dev, uint8_t* greedy_dev, double* nll_sum_dev);

FC_API int fc_model_score(FcModel* m, const int32_t* ids, uint32_t n_seqs, uint32_t seq_len, int mode,
                          float* logprob_out, uint8_t* greedy_out, double* nll_sum_out) {
  if (!m || !ids) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (seq_len < 2) return fc_fail(dev, FC_ERR_SHAPE, "scoring needs at least 2 tokens");
  if (seq_len - 1 > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", seq_len - 1, m->ctx);
  if (n_seqs == 0) return FC_OK;
  FC_TRY(check_ids(m, ids, (size_t)n_seqs * seq_len));
  const size_t rows = (size_t)n_seqs * (seq_len - 1);
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t b_ids = al((size_t)n_seqs * seq_len * 4), b_lp = al(rows * 4), b_gr = al(rows), b_nll = al((size_t)n_seqs * 8);
  const size_t need = b_ids + b_lp + b_gr + b_nll;
  if (need > m->score_stage_bytes) {
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (m->score_stage) cudaFree(m->score_stage);
    m->score_stage = nullptr;
    m->score_stage_bytes = 0;
    const cudaError_t e = cudaMalloc(&m->score_stage, need);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fc_fail(dev, FC_ERR_OOM, "cannot allocate scoring buffers: %s", cudaGetErrorString(e));
    }
    m->score_stage_bytes = need;
  }
  uint8_t* base = (uint8_t*)m->score_stage;
  int32_t* d_ids = (int32_t*)base;
  float* d_lp = (float*)(base + b_ids);
  uint8_t* d_gr = base + b_ids + b_lp;
  double* d_nll = (double*)(base + b_ids + b_lp + b_gr);
  int rc = FC_OK;
  if (cudaMemcpyAsync(d_ids, ids, (size_t)n_seqs * seq_len * 4, cudaMemcpyHostToDevice, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "upload of ids failed");
  if (rc == FC_OK) rc = fc_model_score_dev(m, d_ids, n_seqs, seq_len, mode, d_lp, d_gr, d_nll);
  if (rc == FC_OK && mode == FC_TENSOR_F16) rc = tc_check_errors(dev);
  if (rc == FC_OK) {
    if (logprob_out) cudaMemcpyAsync(logprob_out, d_lp, rows * 4, cudaMemcpyDeviceToHost, dev->stream);
    if (greedy_out) cudaMemcpyAsync(greedy_out, d_gr, rows, cudaMemcpyDeviceToHost, dev->stream);
    if (nll_sum_out) cudaMemcpyAsync(nll_sum_out, d_nll, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, dev->stream);
    if (cudaStreamSynchronize(dev->stream) != cudaSuccess) {
      dev->lost = true;
      rc = fc_fail(dev, FC_ERR_DEVICE, "scoring failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
  }
  return rc;
}
