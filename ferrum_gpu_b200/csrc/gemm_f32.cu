// Exact-f32 batched product y[m, n] = x[m, k] . W[n, k]^T for any m: the f32-accumulated path
// behind forward_all / scoring when FC_EXACT_F32 is asked for, and behind decode batches wider
// than the matvec kernel takes. Replaces qlinear_tiled.wgsl and matmul_blocked4.wgsl
// (ferrum_wgpu/src/shaders/quant/qlinear_tiled.wgsl:L93-L128, shaders/matmul).
//
// 64 x 64 output tile per CTA of 256 threads (4 x 4 outputs per thread), K walked in slices of 32
// (one quantisation block): the x slice and the dequantised weight slice are staged k-major in
// shared memory, values are formed as d * f32(q) exactly as the CPU decoder does, then FMA'd.
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 32, PAD = 4;

__device__ __forceinline__ float gelu_f(float x) {
  const float K = 0.7978846f;
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

template <int KIND>
__global__ void __launch_bounds__(256)
    qgemm_f32_kernel(QMat w, const float* __restrict__ x, uint32_t m, float* __restrict__ y, Epilogue ep) {
  __shared__ __align__(16) float xs[TK][TM + PAD];
  __shared__ __align__(16) float ws[TK][TN + PAD];
  const uint32_t k = w.k, n = w.n;
  const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

  for (uint32_t k0 = 0; k0 < k; k0 += TK) {
    // x slice: 64 rows x 32 k; thread reads 8 consecutive k of one row
    {
      const int r = tid >> 2, c = (tid & 3) * 8;
      const uint32_t row = m0 + r;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const uint32_t kk = k0 + c + j;
        xs[c + j][r] = (row < m && kk < k) ? x[(size_t)row * k + kk] : 0.0f;
      }
    }
    // weight slice: 64 rows x 32 k; thread dequantises 8 consecutive k of one row
    {
      const int r = tid >> 2, part = tid & 3;
      const uint32_t row = n0 + r;
      float v[8];
      if (row < n) {
        if (KIND == FC_Q8_0) {
          const uint2 q = *reinterpret_cast<const uint2*>(w.qs + (size_t)row * k + k0 + part * 8);
          const float d = __half2float(w.sc[(size_t)row * (k / QK) + k0 / QK]);
          const uint32_t qw[2] = {q.x, q.y};
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] = __fmul_rn(d, (float)(int8_t)((qw[j >> 2] >> (8 * (j & 3))) & 0xff));
        } else if (KIND == FC_Q2_K) { // (d * sc) * q - dmin * m, as the decoder rounds it
          const uint32_t kk = k0 + part * 8, sub = kk / 16;
          const uint8_t* rec = reinterpret_cast<const uint8_t*>(w.sc) + ((size_t)row * (k / QK_K) + kk / QK_K) * 20;
          const uint32_t word = reinterpret_cast<const uint32_t*>(w.qs)[(size_t)row * (k / 16) + sub] >> (2 * (kk % 16));
          const uint8_t sc = rec[sub % 16];
          const float dl = __fmul_rn(__half2float(*reinterpret_cast<const __half*>(rec + 16)), (float)(sc & 15));
          const float ml = __fmul_rn(__half2float(*reinterpret_cast<const __half*>(rec + 18)), (float)(sc >> 4));
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] = __fsub_rn(__fmul_rn(dl, (float)((word >> (2 * j)) & 3)), ml);
        } else if (KIND == FC_MXFP4) {
          const uint32_t q = *reinterpret_cast<const uint32_t*>(w.qs + (size_t)row * (k / 2) + (k0 / QK) * 16 + part * 4);
          const float d = block_scale_f32<KIND>(w.sc[(size_t)row * (k / QK) + k0 / QK]);
          uint32_t h[4];
          e2m1x8_to_f16x2(q, h);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[j]));
            v[2 * j] = __fmul_rn(d, f.x);
            v[2 * j + 1] = __fmul_rn(d, f.y);
          }
        } else if (kind_is_fp8(KIND)) {
          const uint2 q = *reinterpret_cast<const uint2*>(w.qs + (size_t)row * k + k0 + part * 8);
          const float d = __half2float(w.sc[(size_t)row * (k / QK) + k0 / QK]);
          const uint32_t qw[2] = {q.x, q.y};
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] = __fmul_rn(d, fp8_to_f32<KIND>(qw[j >> 2] >> (8 * (j & 3))));
        } else if (KIND == FC_Q4_0) {
          const uint32_t q = *reinterpret_cast<const uint32_t*>(w.qs + (size_t)row * (k / 2) + (k0 / QK) * 16 + part * 4);
          const float d = __half2float(w.sc[(size_t)row * (k / QK) + k0 / QK]);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int pos = (j >> 1) + 4 * (j & 1);
            v[j] = __fmul_rn(d, (float)((q >> (4 * pos)) & 0xf) - 8.0f);
          }
        } else if (KIND == FC_F16) {
          const uint4 q = *reinterpret_cast<const uint4*>(w.qs + ((size_t)row * k + k0 + part * 8) * 2);
          const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&qw[j]));
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
          }
        } else {
          const float* src = reinterpret_cast<const float*>(w.qs) + (size_t)row * k;
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint32_t kk = k0 + part * 8 + j;
            v[j] = kk < k ? src[kk] : 0.0f;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < 8; j++) ws[part * 8 + j][r] = v[j];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t row = m0 + ty * 4 + i;
    if (row >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t col = n0 + tx * 4 + j;
      if (col >= n) continue;
      float v = acc[i][j];
      if (ep.bias) v += ep.bias[col];
      if (ep.act == ACT_GELU) v = gelu_f(v);
      if (ep.resid) v = ep.resid[(size_t)row * n + col] + v;
      y[(size_t)row * n + col] = v;
    }
  }
}

} // namespace

int k_qgemm_f32(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep) {
  if (m == 0) return FC_OK;
  dim3 grid((w.n + TN - 1) / TN, (m + TM - 1) / TM);
  if (grid.y > 65535) return fc_fail(dev, FC_ERR_UNSUPPORTED, "qgemm_f32: %u rows exceed one launch", m);
  if (w.kind == FC_Q8_0)
    FC_LAUNCH(dev, "qgemm_f32_q8_0", qgemm_f32_kernel<FC_Q8_0><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_Q4_0)
    FC_LAUNCH(dev, "qgemm_f32_q4_0", qgemm_f32_kernel<FC_Q4_0><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_F16)
    FC_LAUNCH(dev, "qgemm_f32_f16", qgemm_f32_kernel<FC_F16><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_FP8_E4M3)
    FC_LAUNCH(dev, "qgemm_f32_fp8", qgemm_f32_kernel<FC_FP8_E4M3><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_FP8_E5M2)
    FC_LAUNCH(dev, "qgemm_f32_fp8", qgemm_f32_kernel<FC_FP8_E5M2><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_MXFP4)
    FC_LAUNCH(dev, "qgemm_f32_mxfp4", qgemm_f32_kernel<FC_MXFP4><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else if (w.kind == FC_Q2_K)
    FC_LAUNCH(dev, "qgemm_f32_q2_k", qgemm_f32_kernel<FC_Q2_K><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  else
    FC_LAUNCH(dev, "qgemm_f32_f32", qgemm_f32_kernel<FC_F32><<<grid, 256, 0, dev->stream>>>(w, x, m, y, ep));
  return FC_OK;
}
