// The elementwise / row-reduction ops between the matrix products: embedding gather, RMSNorm,
// LayerNorm, RoPE + KV-cache store, SwiGLU, argmax and log-softmax scoring. One CTA per row where
// a row reduction is needed (the reference runs those on a single thread per row:
// rmsnorm.wgsl:L9-L18, layernorm.wgsl:L9-L26, score.wgsl:L8-L24).
#include "ops.cuh"

namespace {

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

// Sum over the CTA; every thread gets the result. `red` holds 32 floats.
__device__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.0f;
  return warp_sum(t);
}
__device__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

// gather.wgsl / embed.wgsl: x[r] = tok[ids[r]] (+ pos[position[r]])
__global__ void embed_kernel(const float* __restrict__ tok, const float* __restrict__ pos_table,
                             const int32_t* __restrict__ ids, const int32_t* __restrict__ positions, uint32_t d,
                             float* __restrict__ x) {
  const uint32_t r = blockIdx.x;
  const float* src = tok + (size_t)ids[r] * d;
  const float* ps = pos_table ? pos_table + (size_t)positions[r] * d : nullptr;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)r * d + i] = ps ? src[i] + ps[i] : src[i];
}

// ferrum_ref/src/models/llama/ops.rs:L55-L66: y = x * (1 / sqrt(mean(x^2) + eps)) * g
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ g, uint32_t d, float eps,
                               float* __restrict__ y) {
  __shared__ float red[32];
  const float* row = x + (size_t)blockIdx.x * d;
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) y[(size_t)blockIdx.x * d + i] = row[i] * inv * g[i];
}

// ferrum_ref/src/kernels/nn.rs:L31-L43: two-pass variance, eps = 1e-5 fixed
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ b,
                                 uint32_t d, float* __restrict__ y) {
  __shared__ float red[32];
  const float* row = x + (size_t)blockIdx.x * d;
  float s = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s += row[i];
  const float mean = block_sum(s, red) / (float)d;
  float vs = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
    const float dl = row[i] - mean;
    vs = fmaf(dl, dl, vs);
  }
  const float var = block_sum(vs, red) / (float)d;
  const float is = 1.0f / sqrtf(var + 1e-5f);
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x)
    y[(size_t)blockIdx.x * d + i] = (row[i] - mean) * is * g[i] + b[i];
}

// ferrum_ref/src/models/llama/ops.rs:L69-L76: silu(g) * u with silu(x) = x / (1 + exp(-x))
// `group` > 0: the fused product's columns come as `group` gate columns followed by the matching
// `group` up columns (the layout the tensor-core SwiGLU epilogue wants); 0: all gate, then all up.
__global__ void swiglu_kernel(const float* __restrict__ gu, uint32_t rows, uint32_t hidden, uint32_t group,
                              float* __restrict__ act) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * hidden) return;
  const size_t r = i / hidden, c = i % hidden;
  const size_t gi = group ? (c / group) * 2 * group + c % group : c;
  const float g = gu[r * 2 * hidden + gi], u = gu[r * 2 * hidden + gi + (group ? group : hidden)];
  act[i] = g / (1.0f + expf(-g)) * u;
}

// rope.wgsl + the two cache copies of feed (ferrum_ref/src/models/llama/ops.rs:L105-L127,
// ferrum_wgpu/src/models/llama/mod.rs:L393-L399). One CTA per row; thread i handles pair i of a head.
__global__ void rope_kv_kernel(float* __restrict__ qkv, uint32_t heads, uint32_t kv_heads, uint32_t hd, RopeParams rope,
                               const int32_t* __restrict__ positions, const int32_t* __restrict__ streams,
                               KvLayer kv, bool has_kv, uint32_t ctx, DeferredReduce pend) {
  const uint32_t r = blockIdx.x;
  const uint32_t qd = heads * hd, kvd = kv_heads * hd;
  float* row = qkv + (size_t)r * (qd + 2 * kvd);
  if (pend.splits) {
    // the qkv product left its split-K partial sums apart: add them in ascending order and apply the bias,
    // exactly as its own reduce launch would, then carry on with the finished row
    const uint32_t w = qd + 2 * kvd; // (a multiple of 4: the host checks)
    const size_t split_stride = (size_t)pend.m * w;
    const float* prow = pend.partial + (size_t)r * w;
    for (uint32_t i = threadIdx.x * 4; i < w; i += blockDim.x * 4) {
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
      for (uint32_t s = 0; s < pend.splits; s++) {
        const float4 p = *reinterpret_cast<const float4*>(prow + s * split_stride + i);
        v.x += p.x, v.y += p.y, v.z += p.z, v.w += p.w;
      }
      if (pend.bias) {
        const float4 bb = *reinterpret_cast<const float4*>(pend.bias + i);
        v.x += bb.x, v.y += bb.y, v.z += bb.z, v.w += bb.w;
      }
      *reinterpret_cast<float4*>(row + i) = v;
    }
    __syncthreads();
  }
  const uint32_t pos = (uint32_t)positions[r];
  if (rope.cos) {
    const uint32_t half = rope.rope_dim / 2;
    const float* cs = rope.cos + (size_t)pos * half;
    const float* sn = rope.sin + (size_t)pos * half;
    const uint32_t total = (heads + kv_heads) * half; // q heads then k heads are contiguous in the row
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
      const uint32_t h = i / half, p = i % half;
      float* base = row + (size_t)h * hd;
      const uint32_t ia = rope.type == FC_ROPE_NORM ? 2 * p : p;
      const uint32_t ib = rope.type == FC_ROPE_NORM ? 2 * p + 1 : p + half;
      const float c = cs[p], s = sn[p], a = base[ia], b = base[ib];
      base[ia] = a * c - b * s;
      base[ib] = a * s + b * c;
    }
  }
  if (has_kv) {
    __syncthreads();
    const uint32_t slot = streams ? (uint32_t)streams[r] : 0;
    for (uint32_t i = threadIdx.x; i < kvd; i += blockDim.x) {
      const uint32_t h = i / hd, e = i % hd;
      const size_t dst = (((size_t)slot * kv_heads + h) * ctx + pos) * hd + e;
      kv.k[dst] = row[qd + i];
      kv.v[dst] = row[qd + kvd + i];
    }
  }
}

// ferrum_model/src/sampling.rs:L32-L40: strictly greater wins, first maximum, NaN never wins
__global__ void argmax_kernel(const float* __restrict__ logits, uint32_t vocab, int32_t* __restrict__ out) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const float* row = logits + (size_t)blockIdx.x * vocab;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { // ascending i per thread keeps the first maximum
      best = v;
      idx = (int)i;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? bv[lane] : -INFINITY;
    idx = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx; // nothing beat -inf: index 0
  }
}

// ferrum_ref/src/kernels/nn.rs:L117-L129 on materialised logits, split in two so a vocabulary
// shard can be scored on its own: per row (max, sum exp(l - max), target logit or -inf, first
// argmax as a global index) over columns [v0, v0 + vs) ...
__global__ void score_partial_kernel(const float* __restrict__ logits, const int32_t* __restrict__ targets,
                                     uint32_t vs, uint32_t v0, float* __restrict__ partial) {
  __shared__ float red[32];
  __shared__ int first_s;
  const float* row = logits + (size_t)blockIdx.x * vs;
  float mx = -INFINITY;
  for (uint32_t i = threadIdx.x; i < vs; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, red);
  float se = 0.0f;
  int first = 0x7fffffff;
  for (uint32_t i = threadIdx.x; i < vs; i += blockDim.x) {
    const float v = row[i];
    se += expf(v - mx);
    if (v == mx && (int)i < first) first = (int)i;
  }
  se = block_sum(se, red);
  if (threadIdx.x == 0) first_s = 0x7fffffff;
  __syncthreads();
  if (first != 0x7fffffff) atomicMin(&first_s, first);
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = targets[blockIdx.x] - (int)v0;
    float* o = partial + (size_t)blockIdx.x * 4;
    o[0] = mx;
    o[1] = se;
    o[2] = (t >= 0 && t < (int)vs) ? row[t] : -INFINITY;
    o[3] = (float)((first_s == 0x7fffffff ? 0 : first_s) + (int)v0);
  }
}

// ... and the merge of n_shards partials: logprob = target - max - ln(sum), greedy = target is the
// first index holding the global maximum.
__global__ void score_combine_kernel(const float* __restrict__ partials, uint32_t n_shards, uint32_t rows,
                                     const int32_t* __restrict__ targets, float* __restrict__ logprob,
                                     uint8_t* __restrict__ greedy) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float mx = -INFINITY, tl = -INFINITY;
  for (uint32_t s = 0; s < n_shards; s++) {
    const float* p = partials + ((size_t)s * rows + r) * 4;
    mx = fmaxf(mx, p[0]);
    tl = fmaxf(tl, p[2]);
  }
  float se = 0.0f;
  int first = 0;
  bool found = false;
  for (uint32_t s = 0; s < n_shards; s++) { // shards are in ascending vocabulary order
    const float* p = partials + ((size_t)s * rows + r) * 4;
    se += n_shards == 1 ? p[1] : p[1] * expf(p[0] - mx);
    if (!found && p[0] == mx) {
      first = (int)p[3];
      found = true;
    }
  }
  if (logprob) logprob[r] = tl - mx - logf(se);
  if (greedy) greedy[r] = first == targets[r];
}

// serving/decoder.rs:L69-L83 sums in f64; ascending position, one thread per sequence
__global__ void nll_sums_kernel(const float* __restrict__ logprob, uint32_t n_seqs, uint32_t rows_per_seq,
                                double* __restrict__ nll) {
  const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seqs) return;
  double acc = 0.0;
  for (uint32_t i = 0; i < rows_per_seq; i++) acc -= (double)logprob[(size_t)s * rows_per_seq + i];
  nll[s] = acc;
}

// the same, written as the two fp16 terms the 9..64-row decode product multiplies (rows >= `rows` of the
// padded block are zero): saves that product's own split launch
// With `pend` the gate/up product's split-K partial sums are still apart: an element is then their sum in
// ascending split order plus the bias (what that product's reduce launch computes), and `gu` is not read.
__global__ void swiglu_split_kernel(const float* __restrict__ gu, uint32_t rows, uint32_t mp, uint32_t hidden, uint32_t group,
                                    __half* __restrict__ xh, __half* __restrict__ xl, DeferredReduce pend) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)mp * hidden) return;
  const size_t r = i / hidden, c = i % hidden;
  float v = 0.0f;
  if (r < rows) {
    const size_t gi = group ? (c / group) * 2 * group + c % group : c;
    const size_t ui = gi + (group ? group : hidden);
    float g, u;
    if (pend.splits) {
      const size_t stride = (size_t)pend.m * 2 * hidden;
      const float* p = pend.partial + r * 2 * hidden;
      g = 0.0f, u = 0.0f;
      for (uint32_t s = 0; s < pend.splits; s++) {
        g += p[s * stride + gi];
        u += p[s * stride + ui];
      }
      if (pend.bias) g += pend.bias[gi], u += pend.bias[ui];
    } else {
      g = gu[r * 2 * hidden + gi], u = gu[r * 2 * hidden + ui];
    }
    v = g / (1.0f + expf(-g)) * u;
  }
  v = fminf(fmaxf(v, -65504.0f), 65504.0f);
  const __half h = __float2half_rn(v);
  xh[i] = h;
  xl[i] = __float2half_rn(v - __half2float(h));
}

} // namespace

int k_swiglu_split(FcDevice* dev, const float* gate_up, uint32_t rows, uint32_t mp, uint32_t hidden, uint32_t group, __half* xh,
                   __half* xl, const DeferredReduce* pending) {
  const size_t total = (size_t)mp * hidden;
  DeferredReduce pend;
  if (pending && pending->splits) {
    // taken along when it is gate_up's own unfinished sum and lies clear of the terms written here
    if (total && pending->y == gate_up && pending->m == rows && pending->n == 2 * hidden && !pending->resid &&
        (uintptr_t)pending->partial >= (uintptr_t)(xl + total))
      pend = *pending;
    else
      FC_TRY(k_flush_deferred(dev, *pending));
  }
  if (!total) return FC_OK;
  FC_LAUNCH(dev, "swiglu_split", swiglu_split_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(
                                     gate_up, rows, mp, hidden, group, xh, xl, pend));
  return FC_OK;
}

int k_embed(FcDevice* dev, const float* tok, const float* pos_table, const int32_t* ids, const int32_t* positions,
            uint32_t rows, uint32_t d, float* x) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "embed", embed_kernel<<<rows, 256, 0, dev->stream>>>(tok, pos_table, ids, positions, d, x));
  return FC_OK;
}

int k_rmsnorm(FcDevice* dev, const float* x, const float* g, uint32_t rows, uint32_t d, float eps, float* y) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "rmsnorm", rmsnorm_kernel<<<rows, 256, 0, dev->stream>>>(x, g, d, eps, y));
  return FC_OK;
}

int k_layernorm(FcDevice* dev, const float* x, const float* g, const float* b, uint32_t rows, uint32_t d, float* y) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "layernorm", layernorm_kernel<<<rows, 256, 0, dev->stream>>>(x, g, b, d, y));
  return FC_OK;
}

int k_swiglu(FcDevice* dev, const float* gate_up, uint32_t rows, uint32_t hidden, uint32_t group, float* act) {
  const size_t total = (size_t)rows * hidden;
  if (!total) return FC_OK;
  FC_LAUNCH(dev, "swiglu", swiglu_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(gate_up, rows, hidden, group, act));
  return FC_OK;
}

int k_rope_kv(FcDevice* dev, float* qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
              const RopeParams& rope, const int32_t* positions, const int32_t* streams, const KvLayer* kv, uint32_t ctx,
              const DeferredReduce* pending) {
  DeferredReduce pend;
  if (pending && pending->splits) {
    // taken along when it is the qkv buffer's own unfinished sum (no residual: the kernel adds none)
    const uint32_t w = (heads + 2 * kv_heads) * hd;
    if (rows && (rope.cos || kv) && pending->y == qkv && pending->m == rows && pending->n == w && w % 4 == 0 &&
        !pending->resid)
      pend = *pending;
    else
      FC_TRY(k_flush_deferred(dev, *pending));
  }
  if (!rows || (!rope.cos && !kv)) return FC_OK;
  KvLayer l = kv ? *kv : KvLayer();
  FC_LAUNCH(dev, "rope_kv",
            rope_kv_kernel<<<rows, 128, 0, dev->stream>>>(qkv, heads, kv_heads, hd, rope, positions, streams, l,
                                                          kv != nullptr, ctx, pend));
  return FC_OK;
}

// The same rule with a row spread over `parts` CTAs (a 150K-entry row is 600 KB: one CTA per row leaves
// most SMs idle). A candidate is the 64-bit key (value as an order-preserving integer, then the
// complement of its index): the largest key is the largest value at its lowest index, whatever order the
// CTAs arrive in. keys[row] and done[row] start at zero and are left at zero by the CTA that finishes the row.
__global__ void __launch_bounds__(512)
    argmax_parts_kernel(const float* __restrict__ logits, uint32_t vocab, uint32_t parts, unsigned long long* keys,
                        uint32_t* done, int32_t* __restrict__ out) {
  __shared__ unsigned long long bk[16];
  const uint32_t r = blockIdx.y, per = ((vocab + parts - 1) / parts + 3) & ~3u; // (whole float4s per CTA)
  const uint32_t i0 = blockIdx.x * per, i1 = min(vocab, i0 + per);
  const float* row = logits + (size_t)r * vocab;
  // The thread's candidate as (value, index): a later entry replaces it only when strictly greater, so the
  // lowest index of the largest value stays; NaN and -inf never win. Four float4 loads are in flight per pass
  // (a pass per load was a chain of trips to L2: 37 us for 64 rows of 152K entries).
  float bv = -INFINITY;
  uint32_t bi = 0;
  auto take = [&](float v, uint32_t i) {
    if (v > bv) bv = v, bi = i;
  };
  if ((vocab & 3u) == 0 && i0 < i1) { // rows start on 16 bytes
    const uint32_t n4 = (i1 - i0) / 4; // (i1 - i0 is a multiple of 4: vocab and per are)
    const float4* row4 = reinterpret_cast<const float4*>(row + i0);
    for (uint32_t j0 = threadIdx.x; j0 < n4; j0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const uint32_t j = j0 + u * blockDim.x;
        v[u] = j < n4 ? row4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const uint32_t i = i0 + 4 * (j0 + u * blockDim.x);
        take(v[u].x, i), take(v[u].y, i + 1), take(v[u].z, i + 2), take(v[u].w, i + 3);
      }
    }
  } else {
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) take(row[i], i);
  }
  unsigned long long best = 0; // "nothing above -inf yet"
  if (bv > -INFINITY) {
    uint32_t u = __float_as_uint(bv + 0.0f); // (-0 and +0 compare equal: one key)
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    best = ((unsigned long long)u << 32) | (uint32_t)~bi;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
    best = ok > best ? ok : best;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) bk[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (uint32_t w = 1; w < blockDim.x / 32; w++) best = bk[w] > best ? bk[w] : best;
    if (best) atomicMax(&keys[r], best);
    __threadfence();
    if (atomicAdd(&done[r], 1u) == parts - 1) { // every CTA of the row has contributed
      __threadfence();
      const unsigned long long k = atomicExch(&keys[r], 0ull);
      done[r] = 0;
      out[r] = k ? (int32_t)~(uint32_t)k : 0; // nothing beat -inf: index 0
    }
  }
}

size_t argmax_scratch_bytes(uint32_t rows) { return (size_t)rows * 16; }

// `scratch` (argmax_scratch_bytes, zeroed once; nullable) lets long rows use several CTAs each.
int k_argmax(FcDevice* dev, const float* logits, uint32_t rows, uint32_t vocab, int32_t* out, void* scratch) {
  if (!rows) return FC_OK;
  const uint32_t sms = (uint32_t)dev->prop.multiProcessorCount;
  uint32_t parts = (2 * sms + rows - 1) / rows;
  const uint32_t max_parts = (vocab + 4095) / 4096; // at least 4096 entries per CTA
  parts = parts > max_parts ? max_parts : parts;
  if (!scratch || parts < 2) {
    FC_LAUNCH(dev, "argmax", argmax_kernel<<<rows, 1024, 0, dev->stream>>>(logits, vocab, out));
    return FC_OK;
  }
  unsigned long long* keys = (unsigned long long*)scratch;
  uint32_t* done = (uint32_t*)(keys + rows);
  FC_LAUNCH(dev, "argmax", argmax_parts_kernel<<<dim3(parts, rows), 512, 0, dev->stream>>>(logits, vocab, parts, keys, done, out));
  return FC_OK;
}

int k_score_partial(FcDevice* dev, const float* logits, const int32_t* targets, uint32_t rows, uint32_t vs, uint32_t v0,
                    float* partial) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "score_partial", score_partial_kernel<<<rows, 512, 0, dev->stream>>>(logits, targets, vs, v0, partial));
  return FC_OK;
}

int k_score_combine(FcDevice* dev, const float* partials, uint32_t n_shards, uint32_t rows, const int32_t* targets,
                    float* logprob, uint8_t* greedy) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "score_combine",
            score_combine_kernel<<<(rows + 127) / 128, 128, 0, dev->stream>>>(partials, n_shards, rows, targets, logprob,
                                                                              greedy));
  return FC_OK;
}

int k_nll_sums(FcDevice* dev, const float* logprob, uint32_t n_seqs, uint32_t rows_per_seq, double* nll) {
  if (!n_seqs) return FC_OK;
  FC_LAUNCH(dev, "nll_sums", nll_sums_kernel<<<(n_seqs + 63) / 64, 64, 0, dev->stream>>>(logprob, n_seqs, rows_per_seq, nll));
  return FC_OK;
}
