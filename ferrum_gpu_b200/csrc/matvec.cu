// Memory-bound quantised matvec for decode: y[m, n] = x[m, k] . W[n, k]^T (+ bias, activation,
// residual) for m = 1..8 rows of x. Replaces qgemv.wgsl / qlinear.wgsl for single rows
// (ferrum_wgpu/src/shaders/quant, chosen by ops/quant.rs:L314-L323).
//
// Shape of the kernel: the weight planes are streamed once with 16-byte loads; a group of LPR
// lanes owns R output rows at a time and walks their K axis in 16-byte chunks, so each lane has R
// independent 16-byte loads in flight while the x chunk it needs (staged once per CTA in shared
// memory) is read once and reused for the R rows. Integer quants are turned into floats with
// bit tricks (no I2F), the per-block f16 scale multiplies the block's partial sum, accumulation
// is f32, and the LPR partial sums are combined with warp shuffles.
#include "common.cuh"
#include "ops.cuh"

namespace {

template <int KIND>
struct Chunk; // one 16-byte load of a weight row
template <>
struct Chunk<FC_Q8_0> {
  static constexpr int ELEMS = 16;
};
template <>
struct Chunk<FC_Q4_0> {
  static constexpr int ELEMS = 32;
};
template <>
struct Chunk<FC_F32> {
  static constexpr int ELEMS = 4;
};
template <>
struct Chunk<FC_F16> {
  static constexpr int ELEMS = 8;
};
template <>
struct Chunk<FC_Q2_K> {
  static constexpr int ELEMS = 64; // four 16-element sub-blocks, each with its own scale and min
};
template <>
struct Chunk<FC_MXFP4> {
  static constexpr int ELEMS = 32;
};
template <>
struct Chunk<FC_FP8_E4M3> {
  static constexpr int ELEMS = 16;
};
template <>
struct Chunk<FC_FP8_E5M2> {
  static constexpr int ELEMS = 16;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// sum over the chunk of x[e] * q[e] (scale not applied)
template <int KIND>
__device__ __forceinline__ float chunk_dot(const uint4& wq, const float* __restrict__ xs) {
  float acc = 0.0f;
  const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
  if (KIND == FC_Q8_0) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      float4 xv = *reinterpret_cast<const float4*>(xs + 4 * w);
      uint32_t u = words[w] ^ 0x80808080u; // int8 -> biased uint8
      // 0x4B000000 | byte is the float 2^23 + byte; subtracting 2^23 + 128 gives the int8 exactly
      float q0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
      float q1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
      float q2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
      float q3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
      acc = fmaf(xv.x, q0, acc);
      acc = fmaf(xv.y, q1, acc);
      acc = fmaf(xv.z, q2, acc);
      acc = fmaf(xv.w, q3, acc);
    }
  } else if (KIND == FC_Q4_0) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      float4 xa = *reinterpret_cast<const float4*>(xs + 8 * w);
      float4 xb = *reinterpret_cast<const float4*>(xs + 8 * w + 4);
      const float xe[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int pos = (j >> 1) + 4 * (j & 1); // nibble position of element j
        uint32_t nib = (words[w] >> (4 * pos)) & 0xfu;
        float q = __uint_as_float(0x4B000000u | nib) - 8388616.0f; // (2^23 + nib) - (2^23 + 8)
        acc = fmaf(xe[j], q, acc);
      }
    }
  } else if (KIND == FC_MXFP4) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float4 xa = *reinterpret_cast<const float4*>(xs + 8 * w);
      const float4 xb = *reinterpret_cast<const float4*>(xs + 8 * w + 4);
      uint32_t h[4];
      e2m1x8_to_f16x2(words[w], h); // element order, exact
      const float2 q0 = __half22float2(*reinterpret_cast<const __half2*>(&h[0]));
      const float2 q1 = __half22float2(*reinterpret_cast<const __half2*>(&h[1]));
      const float2 q2 = __half22float2(*reinterpret_cast<const __half2*>(&h[2]));
      const float2 q3 = __half22float2(*reinterpret_cast<const __half2*>(&h[3]));
      acc = fmaf(xa.x, q0.x, acc);
      acc = fmaf(xa.y, q0.y, acc);
      acc = fmaf(xa.z, q1.x, acc);
      acc = fmaf(xa.w, q1.y, acc);
      acc = fmaf(xb.x, q2.x, acc);
      acc = fmaf(xb.y, q2.y, acc);
      acc = fmaf(xb.z, q3.x, acc);
      acc = fmaf(xb.w, q3.y, acc);
    }
  } else if (kind_is_fp8(KIND)) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + 4 * w);
      const uint32_t lo = fp8x2_to_f16x2<KIND>(words[w]), hi = fp8x2_to_f16x2<KIND>(words[w] >> 16); // exact
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
      acc = fmaf(xv.x, a.x, acc);
      acc = fmaf(xv.y, a.y, acc);
      acc = fmaf(xv.z, b.x, acc);
      acc = fmaf(xv.w, b.y, acc);
    }
  } else if (KIND == FC_F16) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float2 xv = *reinterpret_cast<const float2*>(xs + 2 * w);
      const float2 wv = __half22float2(*reinterpret_cast<const __half2*>(&words[w])); // exact
      acc = fmaf(xv.x, wv.x, acc);
      acc = fmaf(xv.y, wv.y, acc);
    }
  } else {
    float4 xv = *reinterpret_cast<const float4*>(xs);
    acc = fmaf(xv.x, __uint_as_float(wq.x), acc);
    acc = fmaf(xv.y, __uint_as_float(wq.y), acc);
    acc = fmaf(xv.z, __uint_as_float(wq.z), acc);
    acc = fmaf(xv.w, __uint_as_float(wq.w), acc);
  }
  return acc;
}

// Q2_K: the contribution of one 64-element chunk, sum over its sub-blocks j of
// (d * sc_j) * sum(x q) - (dmin * m_j) * sum(x). `sx` holds the four sums of x (shared by the rows).
__device__ __forceinline__ float q2k_chunk(const uint4& wq, const float* __restrict__ xs, const float (&sx)[4], uint32_t scales,
                                           uint32_t d_dmin) {
  const float d = __half2float(__ushort_as_half((unsigned short)(d_dmin & 0xffffu)));
  const float dmin = __half2float(__ushort_as_half((unsigned short)(d_dmin >> 16)));
  const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
  float acc = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + 16 * j + i);
      const uint32_t b = words[j] >> (2 * i);
      sq = fmaf(xv.x, (float)(b & 3u), sq);
      sq = fmaf(xv.y, (float)((b >> 2) & 3u), sq);
      sq = fmaf(xv.z, (float)((b >> 4) & 3u), sq);
      sq = fmaf(xv.w, (float)((b >> 6) & 3u), sq);
    }
    const uint32_t sc = (scales >> (8 * j)) & 0xffu;
    acc = fmaf(d * (float)(sc & 15u), sq, acc);
    acc = fmaf(-(dmin * (float)(sc >> 4)), sx[j], acc);
  }
  return acc;
}

__device__ __forceinline__ float gelu_f(float x) {
  const float K = 0.7978846f; // ferrum_ref/src/kernels/nn.rs:L12-L15
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

// Sum over the CTA, the same order as the stand-alone norm kernels use (elementwise.cu), so the fused
// prologue below reproduces them bit for bit.
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

template <int KIND, int M, int LPR, int R>
__global__ void __launch_bounds__(256)
    qmatvec_kernel(QMat w, const float* __restrict__ x, float* __restrict__ y, Epilogue ep) {
  extern __shared__ __align__(16) float xs[]; // [M][k]
  __shared__ float red[32];
  const uint32_t k = w.k, n = w.n;
  for (uint32_t i = threadIdx.x * 4; i < M * k; i += blockDim.x * 4)
    *reinterpret_cast<float4*>(xs + i) = *reinterpret_cast<const float4*>(x + i);
  __syncthreads();
  if (ep.norm != NORM_NONE) {
    // RMSNorm / LayerNorm of the staged rows, in place (every CTA repeats it: k is a few hundred to a
    // few thousand floats, against a launch and a round trip through global memory saved)
#pragma unroll 1
    for (int m = 0; m < M; m++) {
      float* row = xs + (size_t)m * k;
      if (ep.norm == NORM_RMS) {
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
        ss = block_sum_256(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)k + ep.norm_eps);
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) row[i] = row[i] * inv * ep.norm_g[i];
      } else {
        float s = 0.0f;
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) s += row[i];
        const float mean = block_sum_256(s, red) / (float)k;
        float vs = 0.0f;
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
          const float dl = row[i] - mean;
          vs = fmaf(dl, dl, vs);
        }
        const float var = block_sum_256(vs, red) / (float)k;
        const float is = 1.0f / sqrtf(var + 1e-5f);
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) row[i] = (row[i] - mean) * is * ep.norm_g[i] + ep.norm_b[i];
      }
    }
    __syncthreads();
  }

  constexpr int ELEMS = Chunk<KIND>::ELEMS;
  constexpr int GROUPS_PER_WARP = 32 / LPR;
  const uint32_t chunks = k / ELEMS;
  const size_t row_bytes = (size_t)chunks * 16;
  const uint32_t nb = k / QK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % LPR, g = lane / LPR;
  const uint32_t groups_per_block = (blockDim.x >> 5) * GROUPS_PER_WARP;
  const uint32_t n_groups = (n + R - 1) / R;

  // the loop bound is uniform across the warp (the shuffles below name every lane); a group past
  // the end works on clamped rows and stores nothing
  for (uint32_t base = blockIdx.x * groups_per_block + warp * GROUPS_PER_WARP; base < n_groups;
       base += gridDim.x * groups_per_block) {
    const uint32_t n0 = (base + g) * R;
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[r][m] = 0.0f;
    uint32_t rows[R];
#pragma unroll
    for (int r = 0; r < R; r++) rows[r] = min(n0 + r, n - 1); // clamped rows are computed and dropped

    for (uint32_t c = gl; c < chunks; c += LPR) {
      uint4 wq[R];
      float d[R];
#pragma unroll
      for (int r = 0; r < R; r++) wq[r] = ldg_stream(w.qs + rows[r] * row_bytes + (size_t)c * 16);
      if (kind_has_scales(KIND)) {
#pragma unroll
        for (int r = 0; r < R; r++)
          d[r] = block_scale_f32<KIND>(w.sc[(size_t)rows[r] * nb + (kind_byte_blocks(KIND) ? (c >> 1) : c)]);
      }
      uint32_t q2_sc[R], q2_d[R]; // Q2_K: the chunk's four scale/min bytes and the super-block's d, dmin
      if (KIND == FC_Q2_K) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          const uint32_t* rec =
              reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(w.sc) + ((size_t)rows[r] * (k / QK_K) + (c >> 2)) * 20);
          q2_sc[r] = rec[c & 3];
          q2_d[r] = rec[4];
        }
      }
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float* xp = xs + (size_t)m * k + (size_t)c * ELEMS;
        if (KIND == FC_Q2_K) {
          float sx[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float t = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              const float4 xv = *reinterpret_cast<const float4*>(xp + 16 * j + i);
              t += (xv.x + xv.y) + (xv.z + xv.w);
            }
            sx[j] = t;
          }
#pragma unroll
          for (int r = 0; r < R; r++) acc[r][m] += q2k_chunk(wq[r], xp, sx, q2_sc[r], q2_d[r]);
          continue;
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
          float s = chunk_dot<KIND>(wq[r], xp);
          acc[r][m] = (KIND == FC_F32 || KIND == FC_F16) ? acc[r][m] + s : fmaf(d[r], s, acc[r][m]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        float v = acc[r][m];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[r][m] = v;
      }
    if (gl == 0) {
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint32_t row = n0 + r;
        if (row < n) {
#pragma unroll
          for (int m = 0; m < M; m++) {
            float v = acc[r][m];
            if (ep.bias) v += ep.bias[row];
            if (ep.act == ACT_GELU) v = gelu_f(v);
            if (ep.resid) v = ep.resid[(size_t)m * n + row] + v;
            y[(size_t)m * n + row] = v;
          }
        }
      }
    }
  }
}

template <int KIND, int M, int LPR>
int launch(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep) {
  constexpr int R = M <= 2 ? 4 : 2;
  const size_t smem = (size_t)M * w.k * sizeof(float);
  auto kern = qmatvec_kernel<KIND, M, LPR, R>;
  static OncePerDevice attr; // once per instantiation: the largest staging buffer the host entry admits
  if (attr.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  }
  const uint32_t groups_per_block = 8 * (32 / LPR);
  const uint32_t n_groups = (w.n + R - 1) / R;
  uint32_t blocks = (n_groups + groups_per_block - 1) / groups_per_block;
  // persistent when there is more work than a few waves: x is staged once per CTA
  const uint32_t max_blocks = (uint32_t)dev->prop.multiProcessorCount * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  FC_LAUNCH(dev, "qmatvec", kern<<<blocks, 256, smem, dev->stream>>>(w, x, y, ep));
  return FC_OK;
}

template <int KIND, int M>
int pick_lpr(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep) {
  const uint32_t chunks = w.k / Chunk<KIND>::ELEMS;
  if (chunks % 32 == 0 || chunks > 256) return launch<KIND, M, 32>(dev, w, x, y, ep);
  if (chunks % 16 == 0) return launch<KIND, M, 16>(dev, w, x, y, ep);
  if (chunks % 8 == 0 || chunks > 16) return launch<KIND, M, 8>(dev, w, x, y, ep);
  return launch<KIND, M, 4>(dev, w, x, y, ep);
}

template <int KIND>
int pick_m(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep) {
  switch (m) {
    case 1: return pick_lpr<KIND, 1>(dev, w, x, y, ep);
    case 2: return pick_lpr<KIND, 2>(dev, w, x, y, ep);
    case 3: return pick_lpr<KIND, 3>(dev, w, x, y, ep);
    case 4: return pick_lpr<KIND, 4>(dev, w, x, y, ep);
    case 5: return pick_lpr<KIND, 5>(dev, w, x, y, ep);
    case 6: return pick_lpr<KIND, 6>(dev, w, x, y, ep);
    case 7: return pick_lpr<KIND, 7>(dev, w, x, y, ep);
    case 8: return pick_lpr<KIND, 8>(dev, w, x, y, ep);
  }
  return fc_fail(dev, FC_ERR_UNSUPPORTED, "the matvec kernel takes 1..8 rows, not %u", m);
}

} // namespace

int k_qmatvec(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep) {
  if ((size_t)m * w.k * 4 > 200 * 1024 || w.k % 4)
    return fc_fail(dev, FC_ERR_UNSUPPORTED, "matvec: %u rows of %u inputs do not fit the staging buffer", m, w.k);
  if (w.kind == FC_Q8_0) return pick_m<FC_Q8_0>(dev, w, x, m, y, ep);
  if (w.kind == FC_Q4_0) return pick_m<FC_Q4_0>(dev, w, x, m, y, ep);
  if (w.kind == FC_F16) return pick_m<FC_F16>(dev, w, x, m, y, ep);
  if (w.kind == FC_FP8_E4M3) return pick_m<FC_FP8_E4M3>(dev, w, x, m, y, ep);
  if (w.kind == FC_FP8_E5M2) return pick_m<FC_FP8_E5M2>(dev, w, x, m, y, ep);
  if (w.kind == FC_MXFP4) return pick_m<FC_MXFP4>(dev, w, x, m, y, ep);
  if (w.kind == FC_Q2_K) return pick_m<FC_Q2_K>(dev, w, x, m, y, ep);
  return pick_m<FC_F32>(dev, w, x, m, y, ep);
}

// Which kernel multiplies m rows by a packed matrix in exact-f32 mode:
//   - 2..64 rows of a Q8_0 / Q4_0 matrix whose scratch is at hand: the tensor-core decode product
//     (x as two fp16 terms, integer quants exact in fp16, scales applied in f32) - its cost does not
//     grow with the rows, the FMA kernel's does (8 rows of K = 4096, N = 32000 Q4_0: 74 us against 540);
//   - one row: the f32 FMA matvec (49 us against 71 on that matrix); 1..8 rows without scratch or of
//     another kind likewise; everything else: the tiled f32 product.
//   - one row of a block format whose width the streamed kernel takes (matvec1.cu): that kernel.
// fc_debug_matvec_kernel overrides the choice for 1..8 rows (measurement aid).
bool qlinear_takes_wide_mma(const QMat& w, uint32_t m, const void* scratch) {
  return scratch && m > 8 && qmatvec_mma_supports(w, m); // (x lives in the library's own aligned buffers there)
}

int k_qlinear_f32(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep_in) {
  if (m == 0) return FC_OK;
  const int forced = dev->matvec_choice; // 0: the rule above; 1: FMA kernel; 2: small-batch mma.sync kernel
  Epilogue ep = ep_in;
  if (m == 1 && forced == 0 && qmatvec1_supports(dev, w)) {
    if (ep.pending && ep.pending->splits) FC_TRY(k_flush_deferred(dev, *ep.pending));
    ep.pending = nullptr;
    ep.defer_out = nullptr;
    if (ep.presplit) return fc_fail(dev, FC_ERR_ARG, "a pre-split x needs the 9..64-row tensor-core product");
    return k_qmatvec1(dev, w, x, y, ep);
  }
  const bool fma_ok = m <= 8 && (size_t)m * w.k * 4 <= 200 * 1024 && w.k % 4 == 0;
  // (the tensor-core kernels stage x with 16-byte asynchronous copies)
  const bool mma_ok = ep.scratch && qmatvec_mma_supports(w, m) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0 || ep.presplit);
  if (ep.presplit && !(mma_ok && m > 8)) return fc_fail(dev, FC_ERR_ARG, "a pre-split x needs the 9..64-row tensor-core product");
  const bool use_fma = fma_ok && (!mma_ok || forced == 1 || (forced == 0 && m < 2));
  const bool use_mma_wide = !use_fma && mma_ok && m > 8; // its x split takes the norm along
  if (ep.pending && ep.pending->splits && !use_mma_wide) { // only that split can finish a producer's split-K sum
    FC_TRY(k_flush_deferred(dev, *ep.pending));
    ep.pending = nullptr;
  }
  if (!use_mma_wide) ep.defer_out = nullptr;
  if (ep.norm != NORM_NONE && !use_fma && !use_mma_wide) { // the FMA matvec normalises while it stages x
    if (!ep.norm_tmp) return fc_fail(dev, FC_ERR_ARG, "a fused norm needs a temporary for the kernels that cannot fuse it");
    if (ep.norm == NORM_RMS)
      FC_TRY(k_rmsnorm(dev, x, ep.norm_g, m, w.k, ep.norm_eps, ep.norm_tmp));
    else
      FC_TRY(k_layernorm(dev, x, ep.norm_g, ep.norm_b, m, w.k, ep.norm_tmp));
    x = ep.norm_tmp;
    ep.norm = NORM_NONE;
  }
  if (use_fma) return k_qmatvec(dev, w, x, m, y, ep);
  if (mma_ok) return k_qmatvec_mma(dev, w, x, m, y, ep, ep.scratch);
  return k_qgemm_f32(dev, w, x, m, y, ep);
}
