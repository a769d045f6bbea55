// Block codec on the device: the upload-time quantiser (bit-identical to
// ferrum_gguf::quant::encode, ferrum_gguf/src/codec/quant.rs:L111-L133), the repack of GGUF
// block bytes into split quant / scale planes, its inverse, and the bit-exact dequantiser
// (codec/quant.rs:L50-L88).
//
// All kernels here are one-time or test-time work; they are written for exactness, with
// explicit __fmul_rn / __fadd_rn / __fdiv_rn so the compiler can neither contract nor
// approximate the encoder's arithmetic.
#include "common.cuh"

namespace {

// Device position of element `e` (0..31) of a Q4_0 block: byte offset within the 16-byte block
// and the shift of its nibble.
__host__ __device__ inline void q4_dev_pos(int e, int& byte, int& shift) {
  int w = e >> 3, j = e & 7;
  int pos = (j >> 1) + 4 * (j & 1);
  byte = w * 4 + (pos >> 1);
  shift = (pos & 1) * 4;
}

// Fp8::encode (ferrum_gguf/src/codec/fp8.rs:L75-L109): the nearest code by bisection over the positive
// codes (their values grow with the code), ties to the even code, saturation at the largest finite value.
template <int KIND>
__device__ __forceinline__ uint32_t fp8_encode_dev(float x) {
  if (x != x) return KIND == FC_FP8_E4M3 ? 0x7f : 0x7e;
  const uint32_t sign = (__float_as_uint(x) >> 24) & 0x80u;
  const float a = fminf(fabsf(x), KIND == FC_FP8_E4M3 ? 448.0f : 57344.0f);
  uint32_t lo = 0, hi = KIND == FC_FP8_E4M3 ? 0x7e : 0x7b;
  while (lo < hi) {
    const uint32_t mid = lo + (hi - lo) / 2;
    if (fp8_to_f32<KIND>(mid) < a)
      lo = mid + 1;
    else
      hi = mid;
  }
  const uint32_t up = lo, down = lo ? lo - 1 : 0;
  const float du = fabsf(__fsub_rn(fp8_to_f32<KIND>(up), a)), dd = fabsf(__fsub_rn(a, fp8_to_f32<KIND>(down)));
  return sign | ((du < dd || (du == dd && up % 2 == 0)) ? up : down);
}

// ---- MXFP4 (ferrum_gguf/src/codec/mxfp4.rs) ---------------------------------------------------
// The device keeps the scale byte e as the bf16 bits of 2^(e - 127): e << 7, and 0x0040 for e = 0.
__host__ __device__ inline uint16_t mx_scale_bits(uint32_t e) { return (uint16_t)(e ? e << 7 : 0x0040u); }
__host__ __device__ inline uint8_t mx_scale_byte(uint16_t bits) { return (uint8_t)(bits >= 0x80 ? bits >> 7 : 0); }
// 2^(e - 128), mxfp4.rs:L22-L28
__device__ __forceinline__ float mx_half_scale(uint32_t e) {
  return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1) << 23));
}
// mxfp4.rs:L49-L54. floor(log2(amax)) of the f32 logarithm: taken in f64 and rounded to f32, which gives
// the f32 library's answer on the floats next to every power of two (the only place the floor can differ
// from the exponent field).
__device__ __forceinline__ uint32_t mx_scale_of(float amax) {
  if (!(amax > 0.0f) || isinf(amax)) return 0;
  const int v = (int)floorf((float)log2((double)amax)) - 2 + 127;
  return (uint32_t)min(max(v, 0), 254);
}
// mxfp4.rs:L57-L68: nearest of the sixteen values (twice E2M1, the nibble's top bit the sign), a tie keeps
// the lower index.
__device__ __forceinline__ uint32_t mx_nearest(float x, float d) {
  const float vals[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};
  uint32_t best = 0;
  float best_err = fabsf(__fsub_rn(__fmul_rn(vals[0], d), x));
#pragma unroll
  for (int i = 1; i < 16; i++) {
    const float err = fabsf(__fsub_rn(__fmul_rn(vals[i], d), x));
    if (err < best_err) {
      best = i;
      best_err = err;
    }
  }
  return best;
}

// One thread per (block b, output column col); threads of a warp take consecutive columns so the
// reads of the `[k, n]` matrix coalesce.
template <int KIND>
__global__ void quantise_kn_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, uint8_t* __restrict__ qs,
                                   __half* __restrict__ sc) {
  uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t b = blockIdx.y;
  if (col >= n) return;
  float v[QK];
#pragma unroll
  for (int j = 0; j < QK; j++) v[j] = w[(size_t)(b * QK + j) * n + col];
  uint32_t nb = k / QK;
  if (KIND == FC_MXFP4) { // mxfp4.rs:L71-L82
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < QK; j++) amax = fmaxf(amax, fabsf(v[j]));
    const uint32_t e = mx_scale_of(amax);
    const float d = mx_half_scale(e);
    sc[(size_t)col * nb + b] = __ushort_as_half(mx_scale_bits(e));
    uint32_t words[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < QK; j++) words[j >> 3] |= mx_nearest(v[j], d) << (4 * (j & 7)); // element order
    *reinterpret_cast<uint4*>(qs + (size_t)col * (k / 2) + (size_t)b * 16) =
        make_uint4(words[0], words[1], words[2], words[3]);
  } else if (kind_is_fp8(KIND)) { // fp8.rs:L112-L124: the inverse is taken of the rounded scale
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < QK; j++) amax = fmaxf(amax, fabsf(v[j]));
    const __half d = __float2half_rn(__fdiv_rn(amax, KIND == FC_FP8_E4M3 ? 448.0f : 57344.0f));
    const float df = __half2float(d);
    const float id = df != 0.0f ? __fdiv_rn(1.0f, df) : 0.0f;
    sc[(size_t)col * nb + b] = d;
    uint32_t words[QK / 4];
#pragma unroll
    for (int j = 0; j < QK; j++) { // (unrolled like the other branches: v and words stay in registers)
      const uint32_t c = fp8_encode_dev<KIND>(__fmul_rn(v[j], id));
      if ((j & 3) == 0) words[j >> 2] = 0;
      words[j >> 2] |= c << (8 * (j & 3));
    }
    uint4* dst = reinterpret_cast<uint4*>(qs + (size_t)col * k + (size_t)b * QK);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
  } else if (KIND == FC_Q8_0) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < QK; j++) amax = fmaxf(amax, fabsf(v[j]));
    float d = __fdiv_rn(amax, 127.0f);
    float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    sc[(size_t)col * nb + b] = __float2half_rn(d);
    uint32_t words[QK / 4];
#pragma unroll
    for (int j = 0; j < QK; j++) {
      float r = roundf(__fmul_rn(v[j], id)); // half away from zero
      int q = (r != r) ? 0 : (int)fminf(fmaxf(r, -128.0f), 127.0f); // `as i8`: saturates, NaN -> 0
      if ((j & 3) == 0) words[j >> 2] = 0;
      words[j >> 2] |= (uint32_t)(q & 0xff) << (8 * (j & 3));
    }
    uint4* dst = reinterpret_cast<uint4*>(qs + (size_t)col * k + (size_t)b * QK);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
  } else {
    float mx = 0.0f; // first element of largest magnitude, sign kept
#pragma unroll
    for (int j = 0; j < QK; j++)
      if (fabsf(v[j]) > fabsf(mx)) mx = v[j];
    float d = __fdiv_rn(mx, -8.0f);
    float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    sc[(size_t)col * nb + b] = __float2half_rn(d);
    uint32_t words[4] = {0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < QK; e++) {
      float t = __fadd_rn(__fmul_rn(v[e], id), 8.5f);
      // `as i32` truncates toward zero, saturates, NaN -> 0; then clamp(0, 15)
      int q = (t != t) ? 0 : (t >= 15.0f ? 15 : (t <= 0.0f ? 0 : (int)t));
      int byte, shift;
      q4_dev_pos(e, byte, shift);
      words[byte >> 2] |= (uint32_t)q << (8 * (byte & 3) + shift);
    }
    *reinterpret_cast<uint4*>(qs + (size_t)col * (k / 2) + (size_t)b * 16) =
        make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// `[k, n]` -> `[n, k]` (for matrices kept in f32).
__global__ void transpose_kn_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, float* __restrict__ out) {
  __shared__ float tile[32][33];
  uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    uint32_t r = r0 + i, c = c0 + threadIdx.x;
    if (r < k && c < n) tile[i][threadIdx.x] = w[(size_t)r * n + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    uint32_t c = c0 + i, r = r0 + threadIdx.x;
    if (r < k && c < n) out[(size_t)c * k + r] = tile[threadIdx.x][i];
  }
}

// GGUF block bytes (`n` rows of k/32 blocks of 34 or 18 bytes) -> planes. One thread per block.
template <int KIND>
__global__ void repack_blocks_kernel(const uint8_t* __restrict__ blocks, uint32_t k, uint32_t n,
                                     uint8_t* __restrict__ qs, __half* __restrict__ sc) {
  size_t nb = k / QK;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; // row * nb + b
  if (idx >= nb * n) return;
  if (KIND == FC_MXFP4) { // 17 bytes: the scale byte, then element j | element j + 16 << 4 (mxfp4.rs:L1-L3)
    const uint8_t* p = blocks + idx * 17;
    sc[idx] = __ushort_as_half(mx_scale_bits(p[0]));
    uint32_t words[4] = {0, 0, 0, 0};
    for (int e = 0; e < QK; e++) {
      const uint32_t q = e < 16 ? (p[1 + e] & 0x0f) : (p[1 + e - 16] >> 4);
      words[e >> 3] |= q << (4 * (e & 7));
    }
    *reinterpret_cast<uint4*>(qs + idx * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    return;
  }
  constexpr int FB = KIND == FC_Q8_0 ? 34 : 18; // (the FP8 formats come through as Q8_0: the same bytes)
  const uint8_t* p = blocks + idx * FB;
  uint16_t h = (uint16_t)(p[0] | (p[1] << 8));
  sc[idx] = __ushort_as_half(h);
  if (KIND == FC_Q8_0) {
    uint8_t* dst = qs + idx * QK;
    for (int j = 0; j < QK; j++) dst[j] = p[2 + j];
  } else {
    uint32_t words[4] = {0, 0, 0, 0};
    for (int e = 0; e < QK; e++) {
      int q = e < 16 ? (p[2 + e] & 0x0f) : (p[2 + e - 16] >> 4);
      int byte, shift;
      q4_dev_pos(e, byte, shift);
      words[byte >> 2] |= (uint32_t)q << (8 * (byte & 3) + shift);
    }
    *reinterpret_cast<uint4*>(qs + idx * 16) = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// Planes -> GGUF block bytes.
template <int KIND>
__global__ void export_blocks_kernel(const uint8_t* __restrict__ qs, const __half* __restrict__ sc, uint32_t k,
                                     uint32_t n, uint8_t* __restrict__ blocks) {
  size_t nb = k / QK;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nb * n) return;
  if (KIND == FC_MXFP4) {
    uint8_t* p = blocks + idx * 17;
    p[0] = mx_scale_byte(__half_as_ushort(sc[idx]));
    const uint8_t* src = qs + idx * 16;
    for (int j = 0; j < 16; j++) {
      const uint32_t lo = (src[j >> 1] >> (4 * (j & 1))) & 0x0f, hi = (src[(j + 16) >> 1] >> (4 * (j & 1))) & 0x0f;
      p[1 + j] = (uint8_t)(lo | (hi << 4));
    }
    return;
  }
  constexpr int FB = KIND == FC_Q8_0 ? 34 : 18;
  uint8_t* p = blocks + idx * FB;
  uint16_t h = __half_as_ushort(sc[idx]);
  p[0] = (uint8_t)(h & 0xff);
  p[1] = (uint8_t)(h >> 8);
  if (KIND == FC_Q8_0) {
    for (int j = 0; j < QK; j++) p[2 + j] = qs[idx * QK + j];
  } else {
    const uint8_t* src = qs + idx * 16;
    for (int j = 0; j < 16; j++) {
      int b0, s0, b1, s1;
      q4_dev_pos(j, b0, s0);
      q4_dev_pos(j + 16, b1, s1);
      p[2 + j] = (uint8_t)(((src[b0] >> s0) & 0x0f) | (((src[b1] >> s1) & 0x0f) << 4));
    }
  }
}

// Bit-exact decode: d * f32(q) and d * (f32(nibble) - 8), one rounding each, as the CPU decoder.
template <int KIND>
__global__ void dequant_kernel(const uint8_t* __restrict__ qs, const __half* __restrict__ sc, uint32_t k, uint32_t n,
                               float* __restrict__ out) {
  size_t nb = k / QK;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nb * n) return;
  float d = block_scale_f32<KIND>(sc[idx]);
  float* o = out + idx * QK;
  if (KIND == FC_MXFP4) { // mxfp4.rs:L31-L46: (twice the E2M1 value) x (half the scale), here value x scale
    const uint32_t* src = reinterpret_cast<const uint32_t*>(qs + idx * 16);
    for (int w = 0; w < 4; w++) {
      uint32_t h[4];
      e2m1x8_to_f16x2(src[w], h);
      for (int p = 0; p < 4; p++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[p]));
        o[8 * w + 2 * p] = __fmul_rn(d, f.x);
        o[8 * w + 2 * p + 1] = __fmul_rn(d, f.y);
      }
    }
  } else if (kind_is_fp8(KIND)) { // fp8.rs:L127-L134
    for (int j = 0; j < QK; j++) o[j] = __fmul_rn(d, fp8_to_f32<KIND>(qs[idx * QK + j]));
  } else if (KIND == FC_Q8_0) {
    const int8_t* q = reinterpret_cast<const int8_t*>(qs) + idx * QK;
    for (int j = 0; j < QK; j++) o[j] = __fmul_rn(d, (float)q[j]);
  } else {
    const uint8_t* src = qs + idx * 16;
    for (int e = 0; e < QK; e++) {
      int byte, shift;
      q4_dev_pos(e, byte, shift);
      o[e] = __fmul_rn(d, (float)((src[byte] >> shift) & 0x0f) - 8.0f);
    }
  }
}

// FC_F16: transpose [k, n] -> [n, k] and round to nearest even (f16::f32_to_f16, ferrum_gguf/src/f16.rs:L25-L53)
__global__ void f16_from_kn_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, __half* __restrict__ out) {
  __shared__ float tile[32][33];
  const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32; // columns of w (n), rows of w (k)
  for (uint32_t j = threadIdx.y; j < 32; j += 8) {
    const uint32_t r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < k && c < n) ? w[(size_t)r * n + c] : 0.0f;
  }
  __syncthreads();
  for (uint32_t j = threadIdx.y; j < 32; j += 8) {
    const uint32_t c = c0 + j, r = r0 + threadIdx.x; // out row = column of w
    if (c < n && r < k) {
      const float v = tile[threadIdx.x][j];
      // a NaN becomes the reference's quiet NaN with the input's sign (f16.rs:L25-L53), not the hardware's 0x7fff
      out[(size_t)c * k + r] =
          v != v ? __ushort_as_half((unsigned short)(((__float_as_uint(v) >> 16) & 0x8000u) | 0x7e00u)) : __float2half_rn(v);
    }
  }
}
__global__ void f16_to_f32_kernel(const __half* __restrict__ src, size_t total, float* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = __half2float(src[i]);
}

// ---- Q2_K (ferrum_gguf/src/codec/q2k.rs; decode ferrum_gguf/src/codec/blocks.rs:L199-L220) ----------
// Every f32 operation is spelled with an explicit round-to-nearest intrinsic in the reference's order, so
// the compiler can neither fuse nor reorder it: the encoder's answer depends on exact ties in `mad`.

// q2k.rs:L17-L20
__device__ __forceinline__ int q2k_nearest_int(float x) {
  return (__float_as_int(__fadd_rn(x, 12582912.0f)) & 0x007fffff) - 0x00400000;
}
__device__ __forceinline__ int q2k_level(float iscale, float x, float mn) {
  return min(max(q2k_nearest_int(__fmul_rn(iscale, __fsub_rn(x, mn))), 0), 3);
}

// q2k.rs:L25-L88: scale and min of 16 values on a 0..3 grid; the levels come back packed two bits each.
__device__ void q2k_fit(const float (&x)[16], uint32_t& levels, float& scale_out, float& neg_min_out) {
  float mn = x[0], mx = x[0];
  float sum_w = fabsf(x[0]);
  float sum_x = __fmul_rn(sum_w, x[0]);
#pragma unroll
  for (int i = 1; i < 16; i++) {
    mn = fminf(mn, x[i]);
    mx = fmaxf(mx, x[i]);
    sum_w = __fadd_rn(sum_w, fabsf(x[i]));
    sum_x = __fadd_rn(sum_x, __fmul_rn(fabsf(x[i]), x[i]));
  }
  if (mn > 0.0f) mn = 0.0f;
  levels = 0;
  if (mx == mn) {
    scale_out = 0.0f;
    neg_min_out = -mn;
    return;
  }
  const float range = __fsub_rn(mx, mn);
  float iscale = __fdiv_rn(3.0f, range);
  float scale = __fdiv_rn(1.0f, iscale);
  float best_mad = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const int q = q2k_level(iscale, x[i], mn);
    levels |= (uint32_t)q << (2 * i);
    const float diff = __fsub_rn(__fadd_rn(__fmul_rn(scale, (float)q), mn), x[i]);
    best_mad = __fadd_rn(best_mad, __fmul_rn(fabsf(x[i]), fabsf(diff)));
  }
  float cur_mn = mn; // a winning candidate replaces the min, and later candidates are laid on the new one
#pragma unroll 1
  for (int step = 0; step <= 15; step++) {
    iscale = __fdiv_rn(__fadd_rn(__fadd_rn(-0.5f, __fmul_rn(0.1f, (float)step)), 3.0f), __fsub_rn(mx, cur_mn));
    float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
    uint32_t laux = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const int q = q2k_level(iscale, x[i], cur_mn);
      laux |= (uint32_t)q << (2 * i);
      const float wq = __fmul_rn(fabsf(x[i]), (float)q);
      sum_l = __fadd_rn(sum_l, wq);
      sum_l2 = __fadd_rn(sum_l2, __fmul_rn(wq, (float)q));
      sum_xl = __fadd_rn(sum_xl, __fmul_rn(wq, x[i]));
    }
    const float d = __fsub_rn(__fmul_rn(sum_w, sum_l2), __fmul_rn(sum_l, sum_l));
    if (d > 0.0f) {
      float this_scale = __fdiv_rn(__fsub_rn(__fmul_rn(sum_w, sum_xl), __fmul_rn(sum_x, sum_l)), d);
      float this_min = __fdiv_rn(__fsub_rn(__fmul_rn(sum_l2, sum_x), __fmul_rn(sum_l, sum_xl)), d);
      if (this_min > 0.0f) {
        this_min = 0.0f;
        this_scale = __fdiv_rn(sum_xl, sum_l2);
      }
      float mad = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float q = (float)((laux >> (2 * i)) & 3u);
        const float diff = __fsub_rn(__fadd_rn(__fmul_rn(this_scale, q), this_min), x[i]);
        mad = __fadd_rn(mad, __fmul_rn(fabsf(x[i]), fabsf(diff)));
      }
      if (mad < best_mad) {
        levels = laux;
        best_mad = mad;
        scale = this_scale;
        cur_mn = this_min;
      }
    }
  }
  scale_out = scale;
  neg_min_out = -cur_mn;
}

// q2k.rs:L91-L150. One thread per 16-value sub-block, the 16 lanes of a super-block side by side: grid
// (ceil(n / 8), k / 256), 128 threads = 8 output columns x 16 sub-blocks.
__global__ void __launch_bounds__(128)
    quantise_q2k_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, uint8_t* __restrict__ qs, uint8_t* __restrict__ rec) {
  const uint32_t j = threadIdx.x & 15, col_raw = blockIdx.x * 8 + (threadIdx.x >> 4), b = blockIdx.y;
  const uint32_t col = min(col_raw, n - 1); // lanes past the end work on the last column and store nothing
  float x[16];
#pragma unroll
  for (int i = 0; i < 16; i++) x[i] = w[(size_t)(b * QK_K + 16 * j + i) * n + col];
  uint32_t levels;
  float scale, neg_min;
  q2k_fit(x, levels, scale, neg_min);
  float max_scale = scale, max_min = neg_min;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) { // over the super-block's 16 lanes
    max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, o, 16));
    max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, o, 16));
  }
  max_scale = fmaxf(0.0f, max_scale);
  max_min = fmaxf(0.0f, max_min);
  uint32_t packed = 0;
  __half d = __float2half_rn(0.0f), dmin = __float2half_rn(0.0f);
  if (max_scale > 0.0f) {
    packed = (uint32_t)q2k_nearest_int(__fmul_rn(__fdiv_rn(15.0f, max_scale), scale)) & 0xffu; // `as u8`
    d = __float2half_rn(__fdiv_rn(max_scale, 15.0f));
  }
  if (max_min > 0.0f) {
    packed |= (((uint32_t)q2k_nearest_int(__fmul_rn(__fdiv_rn(15.0f, max_min), neg_min)) & 0xffu) << 4) & 0xffu;
    dmin = __float2half_rn(__fdiv_rn(max_min, 15.0f));
  }
  // the levels again, against the scales as stored
  const float sc = __fmul_rn(__half2float(d), (float)(packed & 15u));
  if (sc != 0.0f) {
    const float dm = __fmul_rn(__half2float(dmin), (float)(packed >> 4));
    levels = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const int q = min(max(q2k_nearest_int(__fdiv_rn(__fadd_rn(x[i], dm), sc)), 0), 3);
      levels |= (uint32_t)q << (2 * i);
    }
  }
  if (col_raw >= n) return;
  const size_t sb = (size_t)col * (k / QK_K) + b;
  reinterpret_cast<uint32_t*>(qs)[sb * 16 + j] = levels;
  rec[sb * 20 + j] = (uint8_t)packed;
  if (j == 0) {
    *reinterpret_cast<__half*>(rec + sb * 20 + 16) = d;
    *reinterpret_cast<__half*>(rec + sb * 20 + 18) = dmin;
  }
}

// 84-byte file blocks <-> planes; one thread per super-block. File element e sits in byte
// 16 + 32 * (e / 128) + e % 32 at shift 2 * ((e % 128) / 32) (blocks.rs:L199-L220).
__global__ void repack_q2k_kernel(const uint8_t* __restrict__ blocks, size_t total, uint8_t* __restrict__ qs, uint8_t* __restrict__ rec) {
  const size_t sb = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (sb >= total) return;
  const uint8_t* p = blocks + sb * 84;
  for (int j = 0; j < 16; j++) {
    uint32_t word = 0;
    for (int i = 0; i < 16; i++) {
      const int e = 16 * j + i;
      word |= (uint32_t)((p[16 + 32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3) << (2 * i);
    }
    reinterpret_cast<uint32_t*>(qs)[sb * 16 + j] = word;
    rec[sb * 20 + j] = p[j];
  }
  for (int i = 0; i < 4; i++) rec[sb * 20 + 16 + i] = p[80 + i];
}
__global__ void export_q2k_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ rec, size_t total, uint8_t* __restrict__ blocks) {
  const size_t sb = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (sb >= total) return;
  uint8_t* p = blocks + sb * 84;
  for (int j = 0; j < 16; j++) p[j] = rec[sb * 20 + j];
  for (int i = 0; i < 64; i++) p[16 + i] = 0;
  for (int e = 0; e < 256; e++) {
    const uint32_t q = (reinterpret_cast<const uint32_t*>(qs)[sb * 16 + e / 16] >> (2 * (e % 16))) & 3;
    p[16 + 32 * (e / 128) + e % 32] |= (uint8_t)(q << (2 * ((e % 128) / 32)));
  }
  for (int i = 0; i < 4; i++) p[80 + i] = rec[sb * 20 + 16 + i];
}
// Bit-exact decode, one thread per sub-block: (d * sc) * q - dmin * m, each product and the difference rounded once.
__global__ void dequant_q2k_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ rec, size_t total_sub, float* __restrict__ out) {
  const size_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= total_sub) return;
  const size_t sb = s / 16;
  const uint8_t sc = rec[sb * 20 + s % 16];
  const float d = __half2float(*reinterpret_cast<const __half*>(rec + sb * 20 + 16));
  const float dmin = __half2float(*reinterpret_cast<const __half*>(rec + sb * 20 + 18));
  const float dl = __fmul_rn(d, (float)(sc & 15)), ml = __fmul_rn(dmin, (float)(sc >> 4));
  const uint32_t word = reinterpret_cast<const uint32_t*>(qs)[s];
  for (int i = 0; i < 16; i++) out[s * 16 + i] = __fsub_rn(__fmul_rn(dl, (float)((word >> (2 * i)) & 3)), ml);
}

} // namespace

int k_quantise_kn(FcDevice* dev, int kind, const float* w, uint32_t k, uint32_t n, uint8_t* qs, __half* sc) {
  if (k == 0 || k % kind_block_elems(kind) || n == 0)
    return fc_fail(dev, FC_ERR_SHAPE, "a %u x %u weight is not whole %u-element blocks", k, n, kind_block_elems(kind));
  if (kind == FC_Q2_K) {
    FC_LAUNCH(dev, "quantise_q2_k",
              quantise_q2k_kernel<<<dim3((n + 7) / 8, k / QK_K), 128, 0, dev->stream>>>(w, k, n, qs, (uint8_t*)sc));
    return FC_OK;
  }
  if (kind == FC_F16) {
    dim3 g16((n + 31) / 32, (k + 31) / 32), b16(32, 8);
    FC_LAUNCH(dev, "quantise_f16", f16_from_kn_kernel<<<g16, b16, 0, dev->stream>>>(w, k, n, (__half*)qs));
    return FC_OK;
  }
  dim3 grid((n + 127) / 128, k / QK);
  if (kind == FC_Q8_0)
    FC_LAUNCH(dev, "quantise_q8_0", quantise_kn_kernel<FC_Q8_0><<<grid, 128, 0, dev->stream>>>(w, k, n, qs, sc));
  else if (kind == FC_Q4_0)
    FC_LAUNCH(dev, "quantise_q4_0", quantise_kn_kernel<FC_Q4_0><<<grid, 128, 0, dev->stream>>>(w, k, n, qs, sc));
  else if (kind == FC_FP8_E4M3)
    FC_LAUNCH(dev, "quantise_fp8", quantise_kn_kernel<FC_FP8_E4M3><<<grid, 128, 0, dev->stream>>>(w, k, n, qs, sc));
  else if (kind == FC_FP8_E5M2)
    FC_LAUNCH(dev, "quantise_fp8", quantise_kn_kernel<FC_FP8_E5M2><<<grid, 128, 0, dev->stream>>>(w, k, n, qs, sc));
  else if (kind == FC_MXFP4)
    FC_LAUNCH(dev, "quantise_mxfp4", quantise_kn_kernel<FC_MXFP4><<<grid, 128, 0, dev->stream>>>(w, k, n, qs, sc));
  else
    return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", kind);
  return FC_OK;
}

int k_transpose_kn(FcDevice* dev, const float* w, uint32_t k, uint32_t n, float* out) {
  dim3 grid((n + 31) / 32, (k + 31) / 32), block(32, 8);
  FC_LAUNCH(dev, "transpose_kn", transpose_kn_kernel<<<grid, block, 0, dev->stream>>>(w, k, n, out));
  return FC_OK;
}

int k_repack_blocks(FcDevice* dev, int kind, const uint8_t* blocks, uint32_t k, uint32_t n, uint8_t* qs, __half* sc) {
  if (kind == FC_F16) { // a GGUF F16 tensor is already [n][k] f16
    FC_CUDA(dev, cudaMemcpyAsync(qs, blocks, (size_t)k * n * 2, cudaMemcpyDeviceToDevice, dev->stream));
    return FC_OK;
  }
  if (kind == FC_Q2_K) {
    const size_t sbs = (size_t)(k / QK_K) * n;
    FC_LAUNCH(dev, "repack_q2_k", repack_q2k_kernel<<<(unsigned)((sbs + 127) / 128), 128, 0, dev->stream>>>(blocks, sbs, qs, (uint8_t*)sc));
    return FC_OK;
  }
  size_t total = (size_t)(k / QK) * n;
  unsigned grid = (unsigned)((total + 127) / 128);
  if (kind_byte_blocks(kind))
    FC_LAUNCH(dev, "repack_q8_0", repack_blocks_kernel<FC_Q8_0><<<grid, 128, 0, dev->stream>>>(blocks, k, n, qs, sc));
  else if (kind == FC_Q4_0)
    FC_LAUNCH(dev, "repack_q4_0", repack_blocks_kernel<FC_Q4_0><<<grid, 128, 0, dev->stream>>>(blocks, k, n, qs, sc));
  else if (kind == FC_MXFP4)
    FC_LAUNCH(dev, "repack_mxfp4", repack_blocks_kernel<FC_MXFP4><<<grid, 128, 0, dev->stream>>>(blocks, k, n, qs, sc));
  else
    return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", kind);
  return FC_OK;
}

int k_export_blocks(FcDevice* dev, const QMat& m, uint8_t* blocks) {
  if (m.kind == FC_F16) {
    FC_CUDA(dev, cudaMemcpyAsync(blocks, m.qs, (size_t)m.k * m.n * 2, cudaMemcpyDeviceToDevice, dev->stream));
    return FC_OK;
  }
  if (m.kind == FC_Q2_K) {
    const size_t sbs = (size_t)(m.k / QK_K) * m.n;
    FC_LAUNCH(dev, "export_q2_k",
              export_q2k_kernel<<<(unsigned)((sbs + 127) / 128), 128, 0, dev->stream>>>(m.qs, (const uint8_t*)m.sc, sbs, blocks));
    return FC_OK;
  }
  size_t total = (size_t)(m.k / QK) * m.n;
  unsigned grid = (unsigned)((total + 127) / 128);
  if (kind_byte_blocks(m.kind))
    FC_LAUNCH(dev, "export_q8_0", export_blocks_kernel<FC_Q8_0><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, blocks));
  else if (m.kind == FC_Q4_0)
    FC_LAUNCH(dev, "export_q4_0", export_blocks_kernel<FC_Q4_0><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, blocks));
  else if (m.kind == FC_MXFP4)
    FC_LAUNCH(dev, "export_mxfp4", export_blocks_kernel<FC_MXFP4><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, blocks));
  else
    return fc_fail(dev, FC_ERR_ARG, "an f32 weight has no block form");
  return FC_OK;
}

int k_dequant(FcDevice* dev, const QMat& m, float* out) {
  if (m.kind == FC_F32) {
    FC_CUDA(dev, cudaMemcpyAsync(out, m.qs, (size_t)m.k * m.n * 4, cudaMemcpyDeviceToDevice, dev->stream));
    return FC_OK;
  }
  if (m.kind == FC_F16) {
    const size_t tot = (size_t)m.k * m.n;
    FC_LAUNCH(dev, "dequant_f16", f16_to_f32_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, dev->stream>>>((const __half*)m.qs, tot, out));
    return FC_OK;
  }
  if (m.kind == FC_Q2_K) {
    const size_t subs = (size_t)(m.k / 16) * m.n;
    FC_LAUNCH(dev, "dequant_q2_k",
              dequant_q2k_kernel<<<(unsigned)((subs + 127) / 128), 128, 0, dev->stream>>>(m.qs, (const uint8_t*)m.sc, subs, out));
    return FC_OK;
  }
  size_t total = (size_t)(m.k / QK) * m.n;
  unsigned grid = (unsigned)((total + 127) / 128);
  if (m.kind == FC_Q8_0)
    FC_LAUNCH(dev, "dequant_q8_0", dequant_kernel<FC_Q8_0><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, out));
  else if (m.kind == FC_FP8_E4M3)
    FC_LAUNCH(dev, "dequant_fp8", dequant_kernel<FC_FP8_E4M3><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, out));
  else if (m.kind == FC_FP8_E5M2)
    FC_LAUNCH(dev, "dequant_fp8", dequant_kernel<FC_FP8_E5M2><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, out));
  else if (m.kind == FC_MXFP4)
    FC_LAUNCH(dev, "dequant_mxfp4", dequant_kernel<FC_MXFP4><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, out));
  else
    FC_LAUNCH(dev, "dequant_q4_0", dequant_kernel<FC_Q4_0><<<grid, 128, 0, dev->stream>>>(m.qs, m.sc, m.k, m.n, out));
  return FC_OK;
}
