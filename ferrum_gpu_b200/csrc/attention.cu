// Attention over an f32 K/V cache.
//
// Decode (one query row per stream): one CTA per (stream, kv-head). The G = heads / kv_heads
// query heads that share the kv-head are served by a single pass over its K and V rows, so the
// cache - the dominant HBM traffic of batched decode - is read once per step. Replaces
// attn_gqd_probs.wgsl + attn_gqd_pv.wgsl (one thread per query head, serial over the context)
// and their MHA twins (ferrum_wgpu/src/ops/llama.rs:L150-L179, ops/mod.rs:L230-L252).
//
//   phase 1: thread t takes positions t, t+256, ...; reads the whole K row (hd floats, 16-byte
//            loads, many in flight) and dots it with the G query vectors held in shared memory;
//            scores go to shared memory [G][len].
//   phase 2: per query head: max, exp, sum (block reductions).
//   phase 3: thread (slice, e) accumulates sum_j p[g][j] * V[j][e] for its quarter of the
//            positions; V rows are read coalesced; slices are combined through shared memory.
//
// The exact-f32 causal kernels for stateless scoring / prefill follow the same three phases with
// one warp per (row, head).
#include "ops.cuh"

namespace {

constexpr int MAXG = 8; // query heads per pass; more are handled in further passes

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// smem: q [MAXG][hd] | red [32] | outp [4][MAXG][hd] | scores [gc][len_cap]
__global__ void __launch_bounds__(256)
    attn_decode_kernel(const float* __restrict__ qkv, uint32_t q_stride, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ streams, KvLayer kv,
                       uint32_t ctx, uint32_t gc, uint32_t len_cap, float* __restrict__ out) {
  extern __shared__ __align__(16) float sm[];
  float* qs = sm;
  float* red = qs + MAXG * hd;
  float* outp = red + 32;
  float* sc = outp + 4 * MAXG * hd;

  const uint32_t r = blockIdx.y, kvh = blockIdx.x;
  const uint32_t G = heads / kv_heads;
  const uint32_t len = (uint32_t)positions[r] + 1;
  const uint32_t slot = streams ? (uint32_t)streams[r] : 0;
  const float* kbase = kv.k + ((size_t)slot * kv_heads + kvh) * ctx * hd;
  const float* vbase = kv.v + ((size_t)slot * kv_heads + kvh) * ctx * hd;
  const float scale = 1.0f / sqrtf((float)hd);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t hd4 = hd / 4;

  for (uint32_t g0 = 0; g0 < G; g0 += gc) {
    const uint32_t gn = min(gc, G - g0);
    __syncthreads();
    for (uint32_t i = tid; i < gn * hd; i += blockDim.x)
      qs[i] = qkv[(size_t)r * q_stride + (size_t)(kvh * G + g0) * hd + i];
    __syncthreads();
    // phase 1: scores
    for (uint32_t j = tid; j < len; j += blockDim.x) {
      const float4* krow = reinterpret_cast<const float4*>(kbase + (size_t)j * hd);
      float dot[MAXG];
#pragma unroll
      for (int g = 0; g < MAXG; g++) dot[g] = 0.0f;
      for (uint32_t c = 0; c < hd4; c++) {
        const float4 kk = krow[c];
#pragma unroll
        for (int g = 0; g < MAXG; g++) {
          if (g < (int)gn) {
            const float4 qq = *reinterpret_cast<const float4*>(qs + g * hd + 4 * c);
            dot[g] = fmaf(qq.x, kk.x, dot[g]);
            dot[g] = fmaf(qq.y, kk.y, dot[g]);
            dot[g] = fmaf(qq.z, kk.z, dot[g]);
            dot[g] = fmaf(qq.w, kk.w, dot[g]);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < MAXG; g++)
        if (g < (int)gn) sc[(size_t)g * len_cap + j] = dot[g] * scale;
    }
    __syncthreads();
    // phase 2: softmax numerators and their sums, one query head at a time
    float inv_sum[MAXG];
    for (uint32_t g = 0; g < gn; g++) {
      float* s = sc + (size_t)g * len_cap;
      float mx = -INFINITY;
      for (uint32_t j = tid; j < len; j += blockDim.x) mx = fmaxf(mx, s[j]);
      mx = warp_max(mx);
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      mx = warp_max(lane < 8 ? red[lane] : -INFINITY);
      __syncthreads();
      float sum = 0.0f;
      for (uint32_t j = tid; j < len; j += blockDim.x) {
        const float p = expf(s[j] - mx);
        s[j] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) red[warp] = sum;
      __syncthreads();
      sum = warp_sum(lane < 8 ? red[lane] : 0.0f);
      __syncthreads();
      inv_sum[g] = 1.0f / sum;
    }
    // phase 3: out[g][e] = sum_j p[g][j] v[j][e]; (256 / hd) position slices
    const uint32_t slices = min(blockDim.x / hd, 4u); // hd <= 256 and divides 256 (checked on the host)
    const uint32_t e = tid % hd, sl = tid / hd;
    float acc[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; g++) acc[g] = 0.0f;
    if (sl < slices) {
      for (uint32_t j = sl; j < len; j += slices) {
        const float vv = vbase[(size_t)j * hd + e];
#pragma unroll
        for (int g = 0; g < MAXG; g++)
          if (g < (int)gn) acc[g] = fmaf(sc[(size_t)g * len_cap + j], vv, acc[g]);
      }
#pragma unroll
      for (int g = 0; g < MAXG; g++)
        if (g < (int)gn && sl < 4) outp[((size_t)sl * MAXG + g) * hd + e] = acc[g];
    }
    __syncthreads();
    if (sl == 0) {
      const uint32_t ns = min(slices, 4u);
      for (uint32_t g = 0; g < gn; g++) {
        float v = 0.0f;
        for (uint32_t s2 = 0; s2 < ns; s2++) v += outp[((size_t)s2 * MAXG + g) * hd + e];
        out[(size_t)r * heads * hd + (size_t)(kvh * G + g0 + g) * hd + e] = v * inv_sum[g];
      }
    }
  }
}

// One warp per (query row, head): causal attention over keys 0..=limit(row). K/V rows come either
// from the fused qkv buffer of the same sequence (stateless) or from a stream's cache.
// smem per warp: scores [t_cap].
template <bool FROM_CACHE>
__global__ void __launch_bounds__(256)
    attn_causal_kernel(const float* __restrict__ qkv, uint32_t t, uint32_t start, uint32_t heads, uint32_t kv_heads,
                       uint32_t hd, KvLayer kv, uint32_t slot, uint32_t ctx, uint32_t t_cap, float* __restrict__ out) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* s = sm + (size_t)warp * t_cap;
  const uint32_t qd = heads * hd, kvd = kv_heads * hd, stride = qd + 2 * kvd;
  const uint32_t G = heads / kv_heads;
  const uint32_t seq = blockIdx.z, h = blockIdx.y;
  const uint32_t i = blockIdx.x * 8 + warp; // row within the sequence
  if (i >= t) return;
  const uint32_t kvh = h / G;
  const uint32_t len = start + i + 1;
  const float* qrow = qkv + ((size_t)seq * t + i) * stride + (size_t)h * hd;
  const float* kb;
  const float* vb;
  size_t kstride;
  if (FROM_CACHE) {
    kb = kv.k + ((size_t)slot * kv_heads + kvh) * ctx * hd;
    vb = kv.v + ((size_t)slot * kv_heads + kvh) * ctx * hd;
    kstride = hd;
  } else {
    kb = qkv + (size_t)seq * t * stride + qd + (size_t)kvh * hd;
    vb = kb + kvd;
    kstride = stride;
  }
  const float scale = 1.0f / sqrtf((float)hd);
  float mx = -INFINITY;
  for (uint32_t j = lane; j < len; j += 32) {
    const float* krow = kb + (size_t)j * kstride;
    float dot = 0.0f;
    for (uint32_t c = 0; c < hd; c += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(krow + c);
      const float4 qq = *reinterpret_cast<const float4*>(qrow + c);
      dot = fmaf(qq.x, kk.x, dot);
      dot = fmaf(qq.y, kk.y, dot);
      dot = fmaf(qq.z, kk.z, dot);
      dot = fmaf(qq.w, kk.w, dot);
    }
    dot *= scale;
    s[j] = dot;
    mx = fmaxf(mx, dot);
  }
  mx = warp_max(mx);
  float sum = 0.0f;
  for (uint32_t j = lane; j < len; j += 32) {
    const float p = expf(s[j] - mx);
    s[j] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = 1.0f / sum;
  for (uint32_t e = lane; e < hd; e += 32) {
    float acc = 0.0f;
    for (uint32_t j = 0; j < len; j++) acc = fmaf(s[j], vb[(size_t)j * kstride + e], acc);
    out[((size_t)seq * t + i) * qd + (size_t)h * hd + e] = acc * inv;
  }
}

} // namespace

bool attn_decode_appends(uint32_t heads, uint32_t kv_heads, uint32_t hd, const float* scratch) {
  return scratch && attn_decode_split_supports(heads, kv_heads, hd);
}
bool attn_decode_folds_rope(uint32_t heads, uint32_t kv_heads, uint32_t hd, const float* scratch, const DeferredReduce& pending,
                            const float* qkv, uint32_t rows) {
  if (!attn_decode_appends(heads, kv_heads, hd, scratch)) return false;
  // Only with a pending sum: the kernel then builds the row from the partial sums, which nobody modifies, so the
  // several CTAs (splits) of a (row, kv-head) can each do it; rotating a finished row in place would not be
  // repeatable. The sum must be the qkv buffer's own, without a residual (the kernel adds none).
  if (!pending.splits) return false;
  return pending.y == qkv && pending.m == rows && pending.n == (heads + 2 * kv_heads) * hd && !pending.resid;
}

int k_attn_decode(FcDevice* dev, const float* qkv, uint32_t q_stride, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                  uint32_t hd, const int32_t* positions, const int32_t* streams, const KvLayer& kv, uint32_t ctx,
                  float* out, float* scratch, __half* xh, __half* xl, uint32_t mp, bool append_kv, const DeferredReduce* qkv_pending,
                  const RopeParams* rope) {
  if (!rows) return FC_OK;
  if (scratch && attn_decode_split_supports(heads, kv_heads, hd))
    return k_attn_decode_split(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, scratch, out, xh, xl, mp,
                               append_kv, qkv_pending, rope);
  if (xh || append_kv || rope) return fc_fail(dev, FC_ERR_ARG, "only the context-split decode attention writes fp16 terms or the cache");
  if (hd % 4 || hd > 256 || 256 % hd)
    return fc_fail(dev, FC_ERR_UNSUPPORTED, "decode attention needs head_dim in {4,8,...,256} dividing 256, not %u", hd);
  const uint32_t G = heads / kv_heads;
  uint32_t gc = G < MAXG ? G : MAXG;
  const size_t fixed = ((size_t)MAXG * hd + 32 + 4 * MAXG * hd) * 4;
  while (gc > 1 && fixed + (size_t)gc * ctx * 4 > 200 * 1024) gc--;
  const size_t smem = fixed + (size_t)gc * ctx * 4;
  if (smem > 220 * 1024) return fc_fail(dev, FC_ERR_UNSUPPORTED, "decode attention: context %u exceeds shared memory", ctx);
  static OncePerDevice attr_set;
  if (attr_set.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  }
  dim3 grid(kv_heads, rows);
  FC_LAUNCH(dev, "attn_decode",
            attn_decode_kernel<<<grid, 256, smem, dev->stream>>>(qkv, q_stride, heads, kv_heads, hd, positions, streams,
                                                                 kv, ctx, gc, ctx, out));
  return FC_OK;
}

static int attn_causal(FcDevice* dev, bool from_cache, const float* qkv, uint32_t n_seqs, uint32_t t, uint32_t start,
                       uint32_t heads, uint32_t kv_heads, uint32_t hd, const KvLayer& kv, uint32_t slot, uint32_t ctx,
                       float* out) {
  if (!n_seqs || !t) return FC_OK;
  if (hd % 4) return fc_fail(dev, FC_ERR_UNSUPPORTED, "attention needs head_dim %% 4 == 0, not %u", hd);
  const uint32_t t_cap = start + t;
  const size_t smem = (size_t)8 * t_cap * 4;
  if (smem > 220 * 1024) return fc_fail(dev, FC_ERR_UNSUPPORTED, "attention: %u positions exceed shared memory", t_cap);
  static OncePerDevice attr_set;
  if (attr_set.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(attn_causal_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    FC_CUDA(dev, cudaFuncSetAttribute(attn_causal_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  }
  dim3 grid((t + 7) / 8, heads, n_seqs);
  if (from_cache)
    FC_LAUNCH(dev, "attn_prefill_cache",
              attn_causal_kernel<true><<<grid, 256, smem, dev->stream>>>(qkv, t, start, heads, kv_heads, hd, kv, slot, ctx,
                                                                         t_cap, out));
  else
    FC_LAUNCH(dev, "attn_causal_f32",
              attn_causal_kernel<false><<<grid, 256, smem, dev->stream>>>(qkv, t, 0, heads, kv_heads, hd, kv, 0, ctx,
                                                                          t_cap, out));
  return FC_OK;
}

int k_attn_causal_f32(FcDevice* dev, const float* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                      uint32_t hd, float* out) {
  return attn_causal(dev, false, qkv, n_seqs, t, 0, heads, kv_heads, hd, KvLayer(), 0, 0, out);
}

int k_attn_prefill_cache_f32(FcDevice* dev, const float* qkv, uint32_t t, uint32_t start, uint32_t heads,
                             uint32_t kv_heads, uint32_t hd, int32_t stream, const KvLayer& kv, uint32_t ctx, float* out) {
  return attn_causal(dev, true, qkv, 1, t, start, heads, kv_heads, hd, kv, (uint32_t)stream, ctx, out);
}
