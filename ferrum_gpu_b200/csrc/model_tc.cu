// f16 tensor-core passes of the resident model (scoring / forward_all with FC_TENSOR_F16).
//
// Per layer: norm (f32 residual stream -> f16) -> fused qkv product (f16 out, bias) -> RoPE on the
// f16 rows -> causal flash attention -> output product with the residual add in its epilogue ->
// norm -> feed-forward product with SwiGLU (gate/up rows interleaved at upload) or bias+GELU in its
// epilogue -> down product with the residual add. The residual stream stays f32. The head never
// writes logits for scoring: its epilogue reduces each 128-column tile to (max, sum exp, target
// logit, first argmax) and a small kernel merges the tiles (score.wgsl re-reads a materialised
// [rows, vocab] matrix instead: ferrum_wgpu/src/shaders/fwd/score.wgsl:L8-L24).
#include "gemm_tc.cuh"
#include "model.cuh"

namespace {
size_t al(size_t v) { return (v + 255) & ~(size_t)255; }

int check_tc_shapes(FcModel* m) {
  if (m->dim % 64 || m->qd() % 64 || m->hidden % 64 || m->hd != 64)
    return fc_fail(m->dev, FC_ERR_UNSUPPORTED,
                   "the tensor-core path needs dim, heads*head_dim and hidden to be multiples of 64 and head_dim 64 "
                   "(dim %u, q width %u, hidden %u, head_dim %u)",
                   m->dim, m->qd(), m->hidden, m->hd);
  if (m->arch == ARCH_LLAMA && m->gu_group != 1)
    return fc_fail(m->dev, FC_ERR_UNSUPPORTED, "the tensor-core path needs the gate and up rows of ff1 interleaved");
  return FC_OK;
}
} // namespace

size_t model_tc_trunk_bytes(const FcModel* m, size_t rows) {
  return al(rows * m->dim * 4) + al(rows * m->dim * 2) + al(rows * m->qkv_w() * 2) + al(rows * m->qd() * 2) +
         al(rows * m->hidden * 2) + 2048;
}
size_t model_tc_head_bytes(const FcModel* m, size_t rows) {
  const size_t tiles = (m->v1 - m->v0 + TC_BN - 1) / TC_BN;
  return al(rows * tiles * 16) + 1024;
}

// Re-order the fused gate/up weight into groups of `group` gate rows followed by their `group` up rows
// (group 1: rows alternate gate, up). Both planes are permuted by whole rows.
int model_interleave_gate_up(FcDevice* dev, FcQWeight* w, uint32_t hidden, uint32_t group) {
  const QMat& q = w->m;
  const size_t qs_row = qmat_qs_bytes(q.kind, q.k, 1), sc_row = qmat_sc_bytes(q.kind, q.k, 1);
  void *nqs = nullptr, *nsc = nullptr;
  cudaError_t e = cudaMalloc(&nqs, qs_row * q.n);
  if (e == cudaSuccess && sc_row) e = cudaMalloc(&nsc, sc_row * q.n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (nqs) cudaFree(nqs);
    return fc_fail(dev, FC_ERR_OOM, "cannot allocate the interleaved gate/up weight: %s", cudaGetErrorString(e));
  }
  int rc = k_permute_rows(dev, q.qs, (uint8_t*)nqs, q.n, (uint32_t)qs_row, hidden, group);
  if (rc == FC_OK && sc_row) rc = k_permute_rows(dev, (const uint8_t*)q.sc, (uint8_t*)nsc, q.n, (uint32_t)sc_row, hidden, group);
  if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) rc = fc_fail(dev, FC_ERR_DEVICE, "gate/up interleave failed");
  if (rc != FC_OK) {
    cudaFree(nqs);
    if (nsc) cudaFree(nsc);
    return rc;
  }
  cudaFree(w->qs_alloc);
  if (w->sc_alloc) cudaFree(w->sc_alloc);
  w->qs_alloc = nqs;
  w->sc_alloc = nsc;
  w->m.qs = (const uint8_t*)nqs;
  w->m.sc = (const __half*)nsc;
  return FC_OK;
}

int k_qgemm_tc(FcDevice* dev, FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev) {
  if (m == 0) return FC_OK;
  const size_t need = (size_t)m * w->m.k * 2;
  if (need > w->tc_cache_bytes) {
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (w->tc_cache) cudaFree(w->tc_cache);
    w->tc_cache = nullptr;
    w->tc_cache_bytes = 0;
    FC_CUDA(dev, cudaMalloc(&w->tc_cache, need));
    w->tc_cache_bytes = need;
  }
  __half* a = (__half*)w->tc_cache;
  FC_TRY(k_f32_to_f16(dev, x_dev, (size_t)m * w->m.k, a));
  TcArgs t;
  t.m = m;
  t.out_f32 = y_dev;
  t.ldo = w->m.n;
  return k_qgemm_tc_f16(dev, w->m, a, EPI_F32, t);
}

int model_trunk_tc(FcModel* m, const int32_t* ids, const int32_t* positions, uint32_t n_seqs, uint32_t t,
                   __half* hidden_out, int32_t cache_stream) {
  FcDevice* dev = m->dev;
  FC_TRY(check_tc_shapes(m));
  if (cache_stream >= 0 && n_seqs != 1) return fc_fail(dev, FC_ERR_ARG, "one sequence fills one stream's cache");
  const uint32_t rows = n_seqs * t, d = m->dim;
  float* x = (float*)arena_take(m, (size_t)rows * d * 4);
  __half* h = (__half*)arena_take(m, (size_t)rows * d * 2);
  __half* qkv = (__half*)arena_take(m, (size_t)rows * m->qkv_w() * 2);
  __half* attn = (__half*)arena_take(m, (size_t)rows * m->qd() * 2);
  __half* act = (__half*)arena_take(m, (size_t)rows * m->hidden * 2);
  const bool ln = m->arch == ARCH_GPT2;
  FC_TRY(k_embed(dev, m->tok, m->pos_table, ids, positions, rows, d, x));
  for (auto& l : m->layers) {
    FC_TRY(k_norm_f16(dev, ln, x, l.norm1_g, l.norm1_b, rows, d, m->eps, h));
    TcArgs a_qkv;
    a_qkv.m = rows, a_qkv.bias = l.qkv.bias, a_qkv.out_f16 = qkv, a_qkv.ldo = m->qkv_w();
    // (RoPE fused into this product's epilogue was measured at a third of the plain fp16 store's rate - the
    // table gathers - so the rotation runs as its own 16-byte-vectorised pass over the q and k columns.)
    FC_TRY(k_qgemm_tc_f16(dev, l.qkv.w->m, h, EPI_F16, a_qkv));
    FC_TRY(k_rope_f16(dev, qkv, rows, m->heads, m->kv_heads, m->hd, m->rope.cos, m->rope.sin, m->rope.rope_dim, m->rope.type,
                       positions));
    if (cache_stream >= 0)
      FC_TRY(k_kv_store_f16(dev, qkv, t, m->heads, m->kv_heads, m->hd, (uint32_t)cache_stream, 0, m->ctx, l.kv.k, l.kv.v));
    FC_TRY(k_attn_causal_f16(dev, qkv, n_seqs, t, m->heads, m->kv_heads, m->hd, attn));
    TcArgs a_wo;
    a_wo.m = rows, a_wo.bias = l.wo.bias, a_wo.out_f32 = x, a_wo.ldo = d;
    FC_TRY(k_qgemm_tc_f16(dev, l.wo.w->m, attn, EPI_RESID, a_wo));
    FC_TRY(k_norm_f16(dev, ln, x, l.norm2_g, l.norm2_b, rows, d, m->eps, h));
    TcArgs a_ff1;
    a_ff1.m = rows, a_ff1.bias = l.ff1.bias, a_ff1.out_f16 = act, a_ff1.ldo = m->hidden;
    if (m->arch == ARCH_LLAMA) {
      FC_TRY(k_qgemm_tc_f16(dev, l.ff1.w->m, h, EPI_SWIGLU, a_ff1));
    } else {
      a_ff1.act = ACT_GELU;
      FC_TRY(k_qgemm_tc_f16(dev, l.ff1.w->m, h, EPI_F16, a_ff1));
    }
    TcArgs a_ff2;
    a_ff2.m = rows, a_ff2.bias = l.ff2.bias, a_ff2.out_f32 = x, a_ff2.ldo = d;
    FC_TRY(k_qgemm_tc_f16(dev, l.ff2.w->m, act, EPI_RESID, a_ff2));
  }
  return k_norm_f16(dev, ln, x, m->normf_g, m->normf_b, rows, d, m->eps, hidden_out);
}

int model_head_partial_tc(FcModel* m, const __half* hidden, const int32_t* targets, uint32_t rows, float* partial) {
  const uint32_t tiles = (m->v1 - m->v0 + TC_BN - 1) / TC_BN;
  float* tile_partials = (float*)arena_take(m, (size_t)rows * tiles * 16);
  TcArgs a;
  a.m = rows, a.targets = targets, a.v0 = m->v0, a.partial = tile_partials;
  FC_TRY(k_qgemm_tc_f16(m->dev, m->head_view, hidden, EPI_LSE, a));
  return k_partial_merge(m->dev, tile_partials, tiles, rows, partial);
}

int model_logits_tc(FcModel* m, const __half* hidden, uint32_t rows, float* logits) {
  TcArgs a;
  a.m = rows, a.out_f32 = logits, a.ldo = m->v1 - m->v0;
  return k_qgemm_tc_f16(m->dev, m->head_view, hidden, EPI_F32, a);
}

void model_tc_free(FcModel*) {}
