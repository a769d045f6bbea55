// Scoring on the device: batched GpuLlama::score (ferrum_wgpu/src/models/llama/forward.rs:L74-L88)
// over many sequences, in chunks that bound the workspace, plus the pieces of the
// vocabulary-split head (trunk / head partials / combine) that the multi-GPU driver strings
// together around its collectives.
#include "model.cuh"

namespace {

// in_ids[s][i] = ids[s][i], targets[s][i] = ids[s][i+1], positions[s][i] = i, for i < seq_len-1
__global__ void score_prep_kernel(const int32_t* __restrict__ ids, uint32_t n_seqs, uint32_t seq_len,
                                  int32_t* __restrict__ in_ids, int32_t* __restrict__ targets,
                                  int32_t* __restrict__ positions) {
  const uint32_t t = seq_len - 1;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_seqs * t) return;
  const size_t s = i / t, p = i % t;
  in_ids[i] = ids[s * seq_len + p];
  targets[i] = ids[s * seq_len + p + 1];
  positions[i] = (int32_t)p;
}

size_t al(size_t v) { return (v + 255) & ~(size_t)255; }

// Workspace bytes of one chunk of `rows` rows (trunk buffers + ids + head scratch).
size_t chunk_bytes(const FcModel* m, size_t rows, int mode) {
  const size_t vs = m->v1 - m->v0;
  size_t b = al(rows * m->dim * 4) * 2 + al(rows * m->qkv_w() * 4) + al(rows * m->qd() * 4) + al(rows * m->ff1_w() * 4) +
             al(rows * m->hidden * 4) + 3 * al(rows * 4) + al(rows * 16) + al(rows * m->dim * 2) + 8192;
  if (mode == FC_EXACT_F32) b += al(rows * vs * 4); // materialised logits of the chunk
  else b += model_tc_head_bytes(m, rows);           // per-tile log-sum-exp partials
  return b;
}

} // namespace

// Exact-f32 head over this rank's vocabulary rows: logits of the chunk are materialised, then
// reduced to per-row partials.
static int head_partial_f32(FcModel* m, const float* hidden, const int32_t* targets, uint32_t rows, float* logits_ws,
                            float* partial) {
  FC_TRY(k_qlinear_f32(m->dev, m->head_view, hidden, rows, logits_ws, Epilogue()));
  return k_score_partial(m->dev, logits_ws, targets, rows, m->v1 - m->v0, m->v0, partial);
}

FC_API int fc_model_score_dev(FcModel* m, const int32_t* ids_dev, uint32_t n_seqs, uint32_t seq_len, int mode,
                              float* logprob_dev, uint8_t* greedy_dev, double* nll_sum_dev) {
  if (!m || !ids_dev) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (seq_len < 2) return fc_fail(dev, FC_ERR_SHAPE, "scoring needs at least 2 tokens");
  if (seq_len - 1 > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", seq_len - 1, m->ctx);
  if (mode != FC_EXACT_F32 && mode != FC_TENSOR_F16) return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
  if (m->n_shards != 1)
    return fc_fail(dev, FC_ERR_UNSUPPORTED, "this model holds one vocabulary shard: use the trunk / head_partial / combine calls");
  if (n_seqs == 0) return FC_OK;
  const uint32_t t = seq_len - 1;
  // chunk size: whole sequences, workspace bounded (2 GiB exact / 6 GiB tensor path)
  const size_t cap = mode == FC_EXACT_F32 ? ((size_t)2 << 30) : ((size_t)6 << 30);
  uint32_t per = n_seqs;
  while (per > 1 && chunk_bytes(m, (size_t)per * t, mode) > cap) per = (per + 1) / 2;
  const size_t rows_max = (size_t)per * t;
  const size_t lp_bytes = logprob_dev ? 0 : al((size_t)n_seqs * t * 4);
  FC_TRY(arena_reserve(m, chunk_bytes(m, rows_max, mode) + lp_bytes));
  float* lp_all = logprob_dev ? logprob_dev : (float*)arena_take(m, (size_t)n_seqs * t * 4);
  int32_t* in_ids = (int32_t*)arena_take(m, rows_max * 4);
  int32_t* targets = (int32_t*)arena_take(m, rows_max * 4);
  int32_t* positions = (int32_t*)arena_take(m, rows_max * 4);
  float* partial = (float*)arena_take(m, rows_max * 16);
  float* logits_ws = mode == FC_EXACT_F32 ? (float*)arena_take(m, rows_max * (m->v1 - m->v0) * 4) : nullptr;
  void* hidden = arena_take(m, rows_max * m->dim * 4); // f32 (exact) or bf16 (tensor)
  const size_t mark = m->arena.off;
  for (uint32_t s0 = 0; s0 < n_seqs; s0 += per) {
    const uint32_t ns = n_seqs - s0 < per ? n_seqs - s0 : per;
    const uint32_t rows = ns * t;
    m->arena.off = mark;
    FC_LAUNCH(dev, "score_prep",
              score_prep_kernel<<<(rows + 255) / 256, 256, 0, dev->stream>>>(ids_dev + (size_t)s0 * seq_len, ns, seq_len,
                                                                             in_ids, targets, positions));
    float* lp = lp_all + (size_t)s0 * t;
    uint8_t* gr = greedy_dev ? greedy_dev + (size_t)s0 * t : nullptr;
    if (mode == FC_EXACT_F32) {
      FC_TRY(model_trunk_f32(m, in_ids, positions, ns, t, (float*)hidden));
      FC_TRY(head_partial_f32(m, (const float*)hidden, targets, rows, logits_ws, partial));
    } else {
      FC_TRY(model_trunk_tc(m, in_ids, positions, ns, t, (__half*)hidden));
      FC_TRY(model_head_partial_tc(m, (const __half*)hidden, targets, rows, partial));
    }
    FC_TRY(k_score_combine(dev, partial, 1, rows, targets, lp, gr));
  }
  if (nll_sum_dev) FC_TRY(k_nll_sums(dev, lp_all, n_seqs, t, nll_sum_dev));
  return FC_OK;
}

// ---- vocabulary-split head ------------------------------------------------------------------------

FC_API int fc_model_set_head_shard(FcModel* m, uint32_t shard, uint32_t n_shards) {
  if (!m) return FC_ERR_ARG;
  if (n_shards == 0 || shard >= n_shards) return fc_fail(m->dev, FC_ERR_ARG, "shard %u of %u", shard, n_shards);
  const uint32_t per = (m->vocab + n_shards - 1) / n_shards;
  const uint32_t v0 = per * shard < m->vocab ? per * shard : m->vocab;
  const uint32_t v1 = v0 + per < m->vocab ? v0 + per : m->vocab;
  if (v1 <= v0) return fc_fail(m->dev, FC_ERR_SHAPE, "shard %u of %u holds no vocabulary rows", shard, n_shards);
  const QMat& full = m->head.w->m;
  QMat v = full;
  v.n = v1 - v0;
  v.qs = full.qs + qmat_qs_bytes(full.kind, full.k, v0);
  v.sc = full.sc ? (const __half*)((const uint8_t*)full.sc + qmat_sc_bytes(full.kind, full.k, v0)) : nullptr;
  m->head_view = v;
  m->shard = shard, m->n_shards = n_shards, m->v0 = v0, m->v1 = v1;
  return FC_OK;
}

FC_API int fc_model_trunk_dev(FcModel* m, const int32_t* ids_dev, uint32_t n_seqs, uint32_t seq_len, int mode,
                              void* hidden_dev) {
  if (!m || !ids_dev || !hidden_dev) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (seq_len == 0 || seq_len > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", seq_len, m->ctx);
  if (n_seqs == 0) return FC_OK;
  const size_t rows = (size_t)n_seqs * seq_len;
  FC_TRY(arena_reserve(m, chunk_bytes(m, rows, FC_TENSOR_F16)));
  int32_t* positions = (int32_t*)arena_take(m, rows * 4);
  // positions 0..seq_len-1 per sequence (score_prep with a virtual extra token would drop the
  // last row; here every row is kept)
  {
    void* pin;
    FC_TRY(fc_pinned(dev, rows * 4, &pin));
    for (size_t i = 0; i < rows; i++) ((int32_t*)pin)[i] = (int32_t)(i % seq_len);
    FC_CUDA(dev, cudaMemcpyAsync(positions, pin, rows * 4, cudaMemcpyHostToDevice, dev->stream));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  }
  if (mode == FC_EXACT_F32) return model_trunk_f32(m, ids_dev, positions, n_seqs, seq_len, (float*)hidden_dev);
  if (mode == FC_TENSOR_F16) return model_trunk_tc(m, ids_dev, positions, n_seqs, seq_len, (__half*)hidden_dev);
  return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
}

FC_API int fc_model_head_partial_dev(FcModel* m, const void* hidden_dev, const int32_t* targets_dev, uint32_t rows,
                                     int mode, float* partial_dev) {
  if (!m || !hidden_dev || !targets_dev || !partial_dev) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (rows == 0) return FC_OK;
  if (mode == FC_TENSOR_F16) {
    FC_TRY(arena_reserve(m, model_tc_head_bytes(m, rows)));
    return model_head_partial_tc(m, (const __half*)hidden_dev, targets_dev, rows, partial_dev);
  }
  if (mode != FC_EXACT_F32) return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
  // chunk the rows so the materialised logits stay under 2 GiB
  const size_t vs = m->v1 - m->v0;
  size_t per = rows;
  while (per > 1 && per * vs * 4 > ((size_t)2 << 30)) per = (per + 1) / 2;
  FC_TRY(arena_reserve(m, al(per * vs * 4) + 4096));
  float* logits_ws = (float*)arena_take(m, per * vs * 4);
  for (size_t r0 = 0; r0 < rows; r0 += per) {
    const uint32_t nr = (uint32_t)(rows - r0 < per ? rows - r0 : per);
    FC_TRY(head_partial_f32(m, (const float*)hidden_dev + r0 * m->dim, targets_dev + r0, nr, logits_ws,
                            partial_dev + r0 * 4));
  }
  return FC_OK;
}

FC_API int fc_score_combine_dev(FcDevice* dev, const float* partials_dev, uint32_t n_shards, const int32_t* targets_dev,
                                uint32_t n_seqs, uint32_t rows_per_seq, float* logprob_dev, uint8_t* greedy_dev,
                                double* nll_sum_dev) {
  if (!dev || !partials_dev || !targets_dev) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  if (n_shards == 0) return fc_fail(dev, FC_ERR_ARG, "n_shards must be positive");
  if (nll_sum_dev && !logprob_dev) return fc_fail(dev, FC_ERR_ARG, "nll sums need the logprob buffer");
  const uint32_t rows = n_seqs * rows_per_seq;
  FC_TRY(k_score_combine(dev, partials_dev, n_shards, rows, targets_dev, logprob_dev, greedy_dev));
  if (nll_sum_dev) FC_TRY(k_nll_sums(dev, logprob_dev, n_seqs, rows_per_seq, nll_sum_dev));
  return FC_OK;
}
