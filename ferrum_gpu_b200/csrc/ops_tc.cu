// Companions of the tensor-core scoring path: f32 -> f16 conversion, RMSNorm / LayerNorm with a
// f16 result (the next product's A operand), RoPE on the f16 fused qkv rows, the merge of
// per-tile log-sum-exp partials, and the row permutation that interleaves gate and up rows.
#include "gemm_tc.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_sum(lane < nw ? red[lane] : 0.0f);
}

__global__ void f32_to_f16_kernel(const float* __restrict__ x, size_t n, __half* __restrict__ y) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(y + i) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  } else {
    for (size_t j = i; j < n; j++) y[j] = __float2half_rn(x[j]);
  }
}

// One warp per row, the row held in registers (NV float4 per lane, d <= 128 * NV): the row is read
// from HBM exactly once and written once as f16. Same arithmetic as the f32 norms.
template <bool LAYERNORM, int NV>
__global__ void __launch_bounds__(128)
    norm_f16_warp_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ b,
                          uint32_t rows, uint32_t d, float eps, __half* __restrict__ y) {
  const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint32_t d4 = d / 4;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)row * d);
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const uint32_t c = lane + 32 * i;
    v[i] = c < d4 ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float mean = 0.0f, inv;
  if (LAYERNORM) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    mean = warp_sum(s) / (float)d;
    float vs = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      if ((uint32_t)(lane + 32 * i) < d4) {
        const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
        vs += a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3;
      }
    }
    inv = 1.0f / sqrtf(warp_sum(vs) / (float)d + 1e-5f);
  } else {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
  }
  uint2* dst = reinterpret_cast<uint2*>(y + (size_t)row * d);
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const uint32_t c = lane + 32 * i;
    if (c < d4) {
      const float4 gg = reinterpret_cast<const float4*>(g)[c];
      float o0, o1, o2, o3;
      if (LAYERNORM) {
        const float4 bb = reinterpret_cast<const float4*>(b)[c];
        o0 = (v[i].x - mean) * inv * gg.x + bb.x, o1 = (v[i].y - mean) * inv * gg.y + bb.y;
        o2 = (v[i].z - mean) * inv * gg.z + bb.z, o3 = (v[i].w - mean) * inv * gg.w + bb.w;
      } else {
        o0 = v[i].x * inv * gg.x, o1 = v[i].y * inv * gg.y, o2 = v[i].z * inv * gg.z, o3 = v[i].w * inv * gg.w;
      }
      __half2 p0 = __floats2half2_rn(o0, o1), p1 = __floats2half2_rn(o2, o3);
      dst[c] = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
    }
  }
}

// Fallback for wide or oddly sized rows: one CTA per row, the row re-read from cache.
template <bool LAYERNORM>
__global__ void norm_f16_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ b,
                                 uint32_t d, float eps, __half* __restrict__ y) {
  __shared__ float red[32];
  const float* row = x + (size_t)blockIdx.x * d;
  float mean = 0.0f, inv;
  if (LAYERNORM) {
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s += row[i];
    mean = block_sum(s, red) / (float)d;
    float vs = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
      const float dl = row[i] - mean;
      vs = fmaf(dl, dl, vs);
    }
    inv = 1.0f / sqrtf(block_sum(vs, red) / (float)d + 1e-5f);
  } else {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  }
  for (uint32_t i = threadIdx.x * 2; i < d; i += blockDim.x * 2) { // d is even on this path
    float v0, v1;
    if (LAYERNORM) {
      v0 = (row[i] - mean) * inv * g[i] + b[i];
      v1 = (row[i + 1] - mean) * inv * g[i + 1] + b[i + 1];
    } else {
      v0 = row[i] * inv * g[i];
      v1 = row[i + 1] * inv * g[i + 1];
    }
    *reinterpret_cast<__half2*>(y + (size_t)blockIdx.x * d + i) = __floats2half2_rn(v0, v1);
  }
}

// rope.wgsl on f16 rows: rotate q and k heads in place, angles from the host-built f32 tables.
__global__ void rope_f16_kernel(__half* __restrict__ qkv, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                                 const float* __restrict__ cos, const float* __restrict__ sin, uint32_t rope_dim,
                                 uint32_t type, const int32_t* __restrict__ positions) {
  const uint32_t r = blockIdx.x;
  const uint32_t stride = (heads + 2 * kv_heads) * hd;
  __half* row = qkv + (size_t)r * stride;
  const uint32_t half = rope_dim / 2;
  const float* cs = cos + (size_t)positions[r] * half;
  const float* sn = sin + (size_t)positions[r] * half;
  const uint32_t total = (heads + kv_heads) * half;
  for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
    const uint32_t h = i / half, p = i % half;
    __half* base = row + (size_t)h * hd;
    const uint32_t ia = type == FC_ROPE_NORM ? 2 * p : p;
    const uint32_t ib = type == FC_ROPE_NORM ? 2 * p + 1 : p + half;
    const float c = cs[p], s = sn[p], a = __half2float(base[ia]), b = __half2float(base[ib]);
    base[ia] = __float2half_rn(a * c - b * s);
    base[ib] = __float2half_rn(a * s + b * c);
  }
}

// The same with 16-byte accesses: one thread rotates 8 pairs of one head (NORM: 16 consecutive
// values; NEOX: 8 values and the 8 that sit rope_dim / 2 further). rope_dim % 16 == 0.
__global__ void __launch_bounds__(256)
    rope_f16_vec_kernel(__half* __restrict__ qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                        const float* __restrict__ cos, const float* __restrict__ sin, uint32_t rope_dim, uint32_t type,
                        const int32_t* __restrict__ positions) {
  const uint32_t half = rope_dim / 2, groups = half / 8, per_row = (heads + kv_heads) * groups;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)rows * per_row) return;
  const uint32_t r = (uint32_t)(idx / per_row), rem = (uint32_t)(idx % per_row), h = rem / groups, gidx = rem % groups;
  __half* base = qkv + (size_t)r * (heads + 2 * kv_heads) * hd + (size_t)h * hd;
  const float* cs = cos + (size_t)positions[r] * half + 8 * gidx;
  const float* sn = sin + (size_t)positions[r] * half + 8 * gidx;
  const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  __half* pa = type == FC_ROPE_NORM ? base + 16 * gidx : base + 8 * gidx;
  __half* pb = type == FC_ROPE_NORM ? pa + 8 : pa + half;
  uint4 va = *reinterpret_cast<const uint4*>(pa), vb = *reinterpret_cast<const uint4*>(pb);
  __half2* ha = reinterpret_cast<__half2*>(&va);
  __half2* hb = reinterpret_cast<__half2*>(&vb);
  if (type == FC_ROPE_NORM) { // pairs are the half2 lanes themselves: va holds pairs 0..3, vb pairs 4..7
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 x = __half22float2(ha[i]), y = __half22float2(hb[i]);
      ha[i] = __floats2half2_rn(x.x * c[i] - x.y * s[i], x.x * s[i] + x.y * c[i]);
      hb[i] = __floats2half2_rn(y.x * c[4 + i] - y.y * s[4 + i], y.x * s[4 + i] + y.y * c[4 + i]);
    }
  } else { // element i of va pairs with element i of vb
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 x = __half22float2(ha[i]), y = __half22float2(hb[i]);
      ha[i] = __floats2half2_rn(x.x * c[2 * i] - y.x * s[2 * i], x.y * c[2 * i + 1] - y.y * s[2 * i + 1]);
      hb[i] = __floats2half2_rn(x.x * s[2 * i] + y.x * c[2 * i], x.y * s[2 * i + 1] + y.y * c[2 * i + 1]);
    }
  }
  *reinterpret_cast<uint4*>(pa) = va;
  *reinterpret_cast<uint4*>(pb) = vb;
}

// [n_tiles][rows][4] -> [rows][4]: tiles are in ascending vocabulary order
__global__ void partial_merge_kernel(const float* __restrict__ tiles, uint32_t n_tiles, uint32_t rows,
                                     float* __restrict__ out) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float mx = -INFINITY, tl = -INFINITY;
  for (uint32_t s = 0; s < n_tiles; s++) {
    const float4 p = *reinterpret_cast<const float4*>(tiles + ((size_t)s * rows + r) * 4);
    mx = fmaxf(mx, p.x);
    tl = fmaxf(tl, p.z);
  }
  float se = 0.0f, first = 0.0f;
  bool found = false;
  for (uint32_t s = 0; s < n_tiles; s++) {
    const float4 p = *reinterpret_cast<const float4*>(tiles + ((size_t)s * rows + r) * 4);
    se += p.y * expf(p.x - mx);
    if (!found && p.x == mx) {
      first = p.w;
      found = true;
    }
  }
  *reinterpret_cast<float4*>(out + (size_t)r * 4) = make_float4(mx, se, tl, first);
}

// Rows [0, half) are gate rows, [half, 2*half) up rows; destination groups them as `group` gate
// rows followed by the matching `group` up rows. One CTA per destination row.
__global__ void permute_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t row_bytes,
                                    uint32_t half, uint32_t group) {
  const uint32_t dr = blockIdx.x;
  const uint32_t blk = dr / (2 * group), in = dr % (2 * group);
  const uint32_t sr = in < group ? blk * group + in : half + blk * group + (in - group);
  const uint8_t* s = src + (size_t)sr * row_bytes;
  uint8_t* d = dst + (size_t)dr * row_bytes;
  for (uint32_t i = threadIdx.x; i < row_bytes; i += blockDim.x) d[i] = s[i];
}

} // namespace

int k_f32_to_f16(FcDevice* dev, const float* x, size_t n, __half* y) {
  if (!n) return FC_OK;
  const size_t threads = (n + 3) / 4;
  FC_LAUNCH(dev, "f32_to_f16", f32_to_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, dev->stream>>>(x, n, y));
  return FC_OK;
}

int k_norm_f16(FcDevice* dev, bool layernorm, const float* x, const float* g, const float* b, uint32_t rows, uint32_t d,
                float eps, __half* y) {
  if (!rows) return FC_OK;
  if (d % 2) return fc_fail(dev, FC_ERR_UNSUPPORTED, "the f16 norm needs an even width, not %u", d);
  if (d % 4 == 0 && d <= 1024) {
    const unsigned grid = (rows + 3) / 4;
    if (d <= 512) {
      if (layernorm)
        FC_LAUNCH(dev, "layernorm_f16", norm_f16_warp_kernel<true, 4><<<grid, 128, 0, dev->stream>>>(x, g, b, rows, d, eps, y));
      else
        FC_LAUNCH(dev, "rmsnorm_f16", norm_f16_warp_kernel<false, 4><<<grid, 128, 0, dev->stream>>>(x, g, b, rows, d, eps, y));
    } else {
      if (layernorm)
        FC_LAUNCH(dev, "layernorm_f16", norm_f16_warp_kernel<true, 8><<<grid, 128, 0, dev->stream>>>(x, g, b, rows, d, eps, y));
      else
        FC_LAUNCH(dev, "rmsnorm_f16", norm_f16_warp_kernel<false, 8><<<grid, 128, 0, dev->stream>>>(x, g, b, rows, d, eps, y));
    }
    return FC_OK;
  }
  if (layernorm)
    FC_LAUNCH(dev, "layernorm_f16", norm_f16_kernel<true><<<rows, 128, 0, dev->stream>>>(x, g, b, d, eps, y));
  else
    FC_LAUNCH(dev, "rmsnorm_f16", norm_f16_kernel<false><<<rows, 128, 0, dev->stream>>>(x, g, b, d, eps, y));
  return FC_OK;
}

// The k and v columns of `t` fp16 qkv rows (one sequence, positions start..start + t - 1) into one stream's
// f32 cache: what feed's two cache copies do (ferrum_wgpu/src/models/llama/mod.rs:L393-L399), for a prompt
// that went through the tensor-core passes. One CTA per row.
__global__ void kv_store_f16_kernel(const __half* __restrict__ qkv, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                                    uint32_t slot, uint32_t start, uint32_t ctx, float* __restrict__ kc, float* __restrict__ vc) {
  const uint32_t r = blockIdx.x, qd = heads * hd, kvd = kv_heads * hd;
  const __half* row = qkv + (size_t)r * (qd + 2 * kvd);
  for (uint32_t i = threadIdx.x; i < kvd; i += blockDim.x) {
    const uint32_t h = i / hd, e = i % hd;
    const size_t dst = (((size_t)slot * kv_heads + h) * ctx + start + r) * hd + e;
    kc[dst] = __half2float(row[qd + i]);
    vc[dst] = __half2float(row[qd + kvd + i]);
  }
}

int k_kv_store_f16(FcDevice* dev, const __half* qkv, uint32_t t, uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t slot,
                   uint32_t start, uint32_t ctx, float* k_cache, float* v_cache) {
  if (!t) return FC_OK;
  FC_LAUNCH(dev, "kv_store_f16",
            kv_store_f16_kernel<<<t, 128, 0, dev->stream>>>(qkv, heads, kv_heads, hd, slot, start, ctx, k_cache, v_cache));
  return FC_OK;
}

int k_rope_f16(FcDevice* dev, __half* qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                const float* cos, const float* sin, uint32_t rope_dim, uint32_t type, const int32_t* positions) {
  if (!rows || !cos) return FC_OK;
  if (rope_dim % 16 == 0 && hd % 8 == 0) {
    const size_t total = (size_t)rows * (heads + kv_heads) * (rope_dim / 16);
    FC_LAUNCH(dev, "rope_f16",
              rope_f16_vec_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(qkv, rows, heads, kv_heads, hd, cos,
                                                                                             sin, rope_dim, type, positions));
    return FC_OK;
  }
  FC_LAUNCH(dev, "rope_f16",
            rope_f16_kernel<<<rows, 128, 0, dev->stream>>>(qkv, heads, kv_heads, hd, cos, sin, rope_dim, type, positions));
  return FC_OK;
}

int k_partial_merge(FcDevice* dev, const float* tiles, uint32_t n_tiles, uint32_t rows, float* out) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "partial_merge", partial_merge_kernel<<<(rows + 127) / 128, 128, 0, dev->stream>>>(tiles, n_tiles, rows, out));
  return FC_OK;
}

int k_permute_rows(FcDevice* dev, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t row_bytes, uint32_t half,
                   uint32_t group) {
  if (!rows) return FC_OK;
  FC_LAUNCH(dev, "permute_rows", permute_rows_kernel<<<rows, 128, 0, dev->stream>>>(src, dst, row_bytes, half, group));
  return FC_OK;
}
