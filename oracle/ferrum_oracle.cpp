// TEST INFRASTRUCTURE - NOT PRODUCT CODE.
//
// CPU restatement of the reference's algorithm for the quantised-inference hot path: the GGUF
// block codec (ferrum_gguf) and the f32 CPU models (ferrum_ref, what `--device cpu` runs).
// Only tests, the smoke check and the CPU-baseline leg of the benchmark may load this library;
// the CUDA library never links, loads or calls it.
//
// Parity pin: the reference is Rust and no Rust toolchain exists in the build environment, so
// the reference itself cannot be run. This restatement is pinned against every known-answer
// test the reference holds for the path (tests/test_oracle_kat.py lists them with file:line)
// and cross-checked against an independent numpy float32 implementation. The reference stores
// no golden logits, so model-level parity with the Rust binary is unpinned beyond those tests.
//
// Build with -O2 -ffp-contract=off and without -ffast-math: rustc never contracts a*b+c into
// an FMA and evaluates left to right, and the loops below rely on the same.
//
// Scalar code, written for fidelity, one function per reference function; each cites the
// reference file:line it follows.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

#include "../include/ferrum_cuda.h" // POD config / weight structs only

#define OR_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t QK = 32; // ferrum_gguf/src/lib.rs:L55

// ---- f16 -------------------------------------------------------------------------------------

// ferrum_gguf/src/codec/f16.rs:L4-L22
float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0 && man == 0) {
    bits = sign;
  } else if (exp == 0) {
    uint32_t shift = (uint32_t)__builtin_clz(man) - 21; // man has at most 10 significant bits
    uint32_t m = (man << shift) & 0x3ff;
    uint32_t e = 127 - 15 + 1 - shift;
    bits = sign | (e << 23) | (m << 13);
  } else if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// ferrum_gguf/src/codec/f16.rs:L25-L53 (round to nearest even, overflow -> infinity)
uint16_t f32_to_f16(float x) {
  uint32_t b;
  std::memcpy(&b, &x, 4);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
  int32_t exp = (int32_t)((b >> 23) & 0xff);
  uint32_t man = b & 0x007fffff;
  if (exp == 0xff) return sign | 0x7c00 | (man != 0 ? 0x200 : 0);
  int32_t e = exp - 127 + 15;
  if (e >= 0x1f) return sign | 0x7c00;
  if (e <= 0) {
    if (e < -10) return sign;
    uint32_t m = man | 0x00800000;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t half = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t mid = 1u << (shift - 1);
    uint32_t round = (rem > mid || (rem == mid && (half & 1) == 1)) ? 1 : 0;
    return sign | (uint16_t)(half + round);
  }
  uint32_t half = ((uint32_t)e << 10) | (man >> 13);
  uint32_t rem = man & 0x1fff;
  uint32_t round = (rem > 0x1000 || (rem == 0x1000 && (half & 1) == 1)) ? 1 : 0;
  return sign | (uint16_t)(half + round);
}

// Rust `f32 as i32`: truncates toward zero, saturates, NaN -> 0.
int32_t rust_f32_as_i32(float v) {
  if (v != v) return 0;
  if (v >= 2147483648.0f) return std::numeric_limits<int32_t>::max();
  if (v <= -2147483648.0f) return std::numeric_limits<int32_t>::min();
  return (int32_t)v;
}

// Rust `f32 as i8`: truncates toward zero, saturates, NaN -> 0.
int8_t rust_f32_as_i8(float v) {
  if (v != v) return 0;
  if (v >= 127.0f) return 127;
  if (v <= -128.0f) return -128;
  return (int8_t)v;
}

// ---- block codec -----------------------------------------------------------------------------

// F16 (codec/quant.rs:L30,L70,L108): two bytes per element, little endian, no scale; counted here in
// 32-element groups like the block formats it shares the kernels with (ops/quant.rs:L86)
// The FP8 formats use Q8_0's block: an f16 scale and 32 one-byte codes (ferrum_gguf/src/codec/fp8.rs:L18).
bool is_fp8(int kind) { return kind == FC_FP8_E4M3 || kind == FC_FP8_E5M2; }
size_t block_bytes(int kind) {
  if (kind == FC_MXFP4) return 1 + QK / 2; // ferrum_gguf/src/codec/mxfp4.rs:L12
  return (kind == FC_Q8_0 || is_fp8(kind)) ? 2 + QK : kind == FC_F16 ? 2 * QK : 2 + QK / 2;
}

// ---- MXFP4 (ferrum_gguf/src/codec/mxfp4.rs) ----------------------------------------------------
// The sixteen codes as twice their E2M1 value; the top bit of the nibble is the sign (mxfp4.rs:L15).
const int8_t MXFP4_VALUES[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// 2^(e - 128): half of the E8M0 scale, the two smallest being subnormal f32s (mxfp4.rs:L22-L28).
float mxfp4_half_scale(uint8_t e) {
  const uint32_t bits = e < 2 ? (0x00200000u << e) : (((uint32_t)e - 1) << 23);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// mxfp4.rs:L49-L54: the scale that puts the block's largest magnitude in [4, 8) half-steps; no NaN byte.
uint8_t mxfp4_scale_byte(float amax) {
  if (amax <= 0.0f || !std::isfinite(amax)) return 0;
  const int v = (int)std::floor(std::log2(amax)) - 2 + 127; // f32 log2, as `f32::log2`
  return (uint8_t)std::min(std::max(v, 0), 254);
}

// mxfp4.rs:L57-L68: the code whose value is nearest; a tie keeps the lower index.
uint8_t mxfp4_nearest(float x, float d) {
  size_t best = 0;
  float best_err = std::fabs((float)MXFP4_VALUES[0] * d - x);
  for (size_t i = 1; i < 16; i++) {
    const float err = std::fabs((float)MXFP4_VALUES[i] * d - x);
    if (err < best_err) {
      best = i;
      best_err = err;
    }
  }
  return (uint8_t)best;
}

// ---- FP8 (ferrum_gguf/src/codec/fp8.rs) --------------------------------------------------------
// Largest finite magnitude (fp8.rs:L33-L38).
float fp8_max(int kind) { return kind == FC_FP8_E4M3 ? 448.0f : 57344.0f; }

// fp8.rs:L41-L70. E4M3 has no infinity and one NaN per sign (all ones); E5M2 follows IEEE.
float fp8_decode(int kind, uint8_t code) {
  const float sign = (code & 0x80) ? -1.0f : 1.0f;
  const int ebits = kind == FC_FP8_E4M3 ? 4 : 5, mbits = kind == FC_FP8_E4M3 ? 3 : 2, bias = kind == FC_FP8_E4M3 ? 7 : 15;
  const uint32_t e = ((uint32_t)code >> mbits) & ((1u << ebits) - 1), m = (uint32_t)code & ((1u << mbits) - 1);
  const uint32_t top = (1u << ebits) - 1;
  if (e == top) {
    if (kind == FC_FP8_E4M3) {
      if (m == (1u << mbits) - 1) return std::nanf("");
    } else {
      return m == 0 ? sign * INFINITY : std::nanf("");
    }
  }
  const float frac = (float)m / (float)(1u << mbits);
  if (e == 0) return sign * frac * std::ldexp(1.0f, 1 - bias);
  return sign * (1.0f + frac) * std::ldexp(1.0f, (int)e - bias);
}

// fp8.rs:L75-L109: the nearest code by bisection over the (monotonic) positive codes, ties to the
// even code, magnitudes past the largest finite value saturate to it, NaN has its own code.
uint8_t fp8_encode(int kind, float x) {
  if (x != x) return kind == FC_FP8_E4M3 ? 0x7f : 0x7e;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  const float a = std::fmin(std::fabs(x), fp8_max(kind));
  const uint8_t limit = kind == FC_FP8_E4M3 ? 0x7e : 0x7b;
  uint8_t lo = 0, hi = limit;
  while (lo < hi) {
    const uint8_t mid = (uint8_t)(lo + (hi - lo) / 2);
    if (fp8_decode(kind, mid) < a)
      lo = (uint8_t)(mid + 1);
    else
      hi = mid;
  }
  const uint8_t up = lo, down = lo ? (uint8_t)(lo - 1) : 0;
  const float du = std::fabs(fp8_decode(kind, up) - a), dd = std::fabs(a - fp8_decode(kind, down));
  const uint8_t pick = (du < dd || (du == dd && up % 2 == 0)) ? up : down;
  return sign | pick;
}


// ---- Q2_K (ferrum_gguf/src/codec/q2k.rs, decode ferrum_gguf/src/codec/blocks.rs:L199-L220) -----
constexpr size_t QK_K = 256;                       // ferrum_gguf/src/lib.rs
constexpr size_t Q2K_BLOCK = 16 + QK_K / 4 + 4;    // scales, 2-bit quants, d, dmin (q2k.rs:L13)

// q2k.rs:L17-L20: round half to even through the float's own rounding
int32_t q2k_nearest_int(float x) {
  const float y = x + 12582912.0f;
  int32_t bits;
  std::memcpy(&bits, &y, 4);
  return (bits & 0x007fffff) - 0x00400000;
}

// q2k.rs:L25-L88: scale and min of 16 values on a 0..3 grid, searched over 16 candidate scales for
// the smallest |x|-weighted absolute error. Returns (scale, -min); fills the levels.
void q2k_fit(const float* x, uint8_t* l, float* scale_out, float* neg_min_out) {
  const int NMAX = 3;
  float weights[16];
  for (int i = 0; i < 16; i++) weights[i] = std::fabs(x[i]);
  float mn = x[0], mx = x[0];
  float sum_w = weights[0];
  float sum_x = sum_w * x[0];
  for (int i = 1; i < 16; i++) {
    mn = std::fmin(mn, x[i]);
    mx = std::fmax(mx, x[i]);
    sum_w += weights[i];
    sum_x += weights[i] * x[i];
  }
  if (mn > 0.0f) mn = 0.0f;
  if (mx == mn) {
    for (int i = 0; i < 16; i++) l[i] = 0;
    *scale_out = 0.0f;
    *neg_min_out = -mn;
    return;
  }
  float iscale = (float)NMAX / (mx - mn);
  float scale = 1.0f / iscale;
  float best_mad = 0.0f;
  for (int i = 0; i < 16; i++) {
    const int q = std::min(std::max(q2k_nearest_int(iscale * (x[i] - mn)), 0), NMAX);
    l[i] = (uint8_t)q;
    const float diff = scale * (float)q + mn - x[i];
    best_mad += weights[i] * std::fabs(diff);
  }
  for (int step = 0; step <= 15; step++) {
    iscale = (-0.5f + 0.1f * (float)step + (float)NMAX) / (mx - mn);
    float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
    uint8_t laux[16];
    for (int i = 0; i < 16; i++) {
      const int q = std::min(std::max(q2k_nearest_int(iscale * (x[i] - mn)), 0), NMAX);
      laux[i] = (uint8_t)q;
      const float w = weights[i], qf = (float)q;
      sum_l += w * qf;
      sum_l2 += w * qf * qf;
      sum_xl += w * qf * x[i];
    }
    const float d = sum_w * sum_l2 - sum_l * sum_l;
    if (d > 0.0f) {
      float this_scale = (sum_w * sum_xl - sum_x * sum_l) / d;
      float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / d;
      if (this_min > 0.0f) {
        this_min = 0.0f;
        this_scale = sum_xl / sum_l2;
      }
      float mad = 0.0f;
      for (int i = 0; i < 16; i++) {
        const float diff = this_scale * (float)laux[i] + this_min - x[i];
        mad += weights[i] * std::fabs(diff);
      }
      if (mad < best_mad) {
        for (int i = 0; i < 16; i++) l[i] = laux[i];
        best_mad = mad;
        scale = this_scale;
        mn = this_min;
      }
    }
  }
  *scale_out = scale;
  *neg_min_out = -mn;
}

// q2k.rs:L91-L150: one 84-byte super-block per 256 values.
void q2k_encode(const float* data, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / QK_K; b++) {
    const float* blk = data + b * QK_K;
    uint8_t* o = out + b * Q2K_BLOCK;
    float scales[16], mins[16];
    uint8_t levels[QK_K];
    for (int j = 0; j < 16; j++) q2k_fit(blk + 16 * j, levels + 16 * j, &scales[j], &mins[j]);
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 16; j++) {
      max_scale = std::fmax(max_scale, scales[j]);
      max_min = std::fmax(max_min, mins[j]);
    }
    uint8_t packed[16] = {0};
    uint16_t d = 0, dmin = 0;
    if (max_scale > 0.0f) {
      const float iscale = 15.0f / max_scale;
      for (int j = 0; j < 16; j++) packed[j] = (uint8_t)q2k_nearest_int(iscale * scales[j]);
      d = f32_to_f16(max_scale / 15.0f);
    }
    if (max_min > 0.0f) {
      const float iscale = 15.0f / max_min;
      for (int j = 0; j < 16; j++) packed[j] |= (uint8_t)((uint8_t)q2k_nearest_int(iscale * mins[j]) << 4);
      dmin = f32_to_f16(max_min / 15.0f);
    }
    const float d32 = f16_to_f32(d), dmin32 = f16_to_f32(dmin);
    for (int j = 0; j < 16; j++) { // the levels again, against the scales as stored
      const float sc = d32 * (float)(packed[j] & 15);
      if (sc == 0.0f) continue;
      const float dm = dmin32 * (float)(packed[j] >> 4);
      for (int ii = 0; ii < 16; ii++) {
        const int q = q2k_nearest_int((blk[16 * j + ii] + dm) / sc);
        levels[16 * j + ii] = (uint8_t)std::min(std::max(q, 0), 3);
      }
    }
    std::memcpy(o, packed, 16);
    size_t at = 16;
    for (size_t half = 0; half < QK_K; half += 128)
      for (size_t l = 0; l < 32; l++)
        o[at++] = (uint8_t)(levels[half + l] | (levels[half + l + 32] << 2) | (levels[half + l + 64] << 4) |
                            (levels[half + l + 96] << 6));
    o[80] = (uint8_t)(d & 0xff), o[81] = (uint8_t)(d >> 8);
    o[82] = (uint8_t)(dmin & 0xff), o[83] = (uint8_t)(dmin >> 8);
  }
}

// blocks.rs:L199-L220: y = d * sc * q - dmin * m over two 128-element halves, shifts 0, 2, 4, 6, two
// 16-element runs per shift.
void q2k_decode(const uint8_t* bytes, size_t n, float* out) {
  for (size_t b = 0; b < n / QK_K; b++) {
    const uint8_t* p = bytes + b * Q2K_BLOCK;
    const uint8_t *scales = p, *qs = p + 16;
    const float d = f16_to_f32((uint16_t)(p[80] | (p[81] << 8))), dmin = f16_to_f32((uint16_t)(p[82] | (p[83] << 8)));
    float* o = out + b * QK_K;
    size_t is = 0, at = 0;
    for (size_t half = 0; half < 2; half++) {
      const uint8_t* q = qs + 32 * half;
      for (int shift = 0; shift < 8; shift += 2)
        for (size_t run = 0; run < 2; run++) {
          const uint8_t sc = scales[is++];
          const float dl = d * (float)(sc & 0x0f), ml = dmin * (float)(sc >> 4);
          for (size_t i = 0; i < 16; i++) o[at++] = dl * (float)((q[16 * run + i] >> shift) & 3) - ml;
        }
    }
  }
}

// ferrum_gguf/src/codec/quant.rs:L111-L119 (Q8_0) and L120-L133 (Q4_0)
void encode(int kind, const float* data, size_t n, uint8_t* out) {
  if (kind == FC_Q2_K) return q2k_encode(data, n, out);
  for (size_t b = 0; b < n / QK; b++) {
    const float* blk = data + b * QK;
    uint8_t* o = out + b * block_bytes(kind);
    if (kind == FC_F16) {
      for (size_t j = 0; j < QK; j++) {
        const uint16_t h = f32_to_f16(blk[j]);
        o[2 * j] = (uint8_t)(h & 0xff);
        o[2 * j + 1] = (uint8_t)(h >> 8);
      }
      continue;
    }
    if (kind == FC_MXFP4) { // mxfp4.rs:L71-L82: low nibbles are elements 0..16, high nibbles 16..32
      float amax = 0.0f;
      for (size_t j = 0; j < QK; j++) amax = std::fmax(amax, std::fabs(blk[j]));
      const uint8_t e = mxfp4_scale_byte(amax);
      const float d = mxfp4_half_scale(e);
      o[0] = e;
      for (size_t j = 0; j < QK / 2; j++) o[1 + j] = mxfp4_nearest(blk[j], d) | (uint8_t)(mxfp4_nearest(blk[j + QK / 2], d) << 4);
      continue;
    }
    if (is_fp8(kind)) { // fp8.rs:L112-L124: the scale maps the block's largest magnitude onto the format's
      float amax = 0.0f;
      for (size_t j = 0; j < QK; j++) amax = std::fmax(amax, std::fabs(blk[j]));
      const uint16_t h = f32_to_f16(amax / fp8_max(kind));
      const float df = f16_to_f32(h);
      const float id = df != 0.0f ? 1.0f / df : 0.0f; // (of the rounded scale, unlike Q8_0)
      o[0] = (uint8_t)(h & 0xff);
      o[1] = (uint8_t)(h >> 8);
      for (size_t j = 0; j < QK; j++) o[2 + j] = fp8_encode(kind, blk[j] * id);
      continue;
    }
    if (kind == FC_Q8_0) {
      float amax = 0.0f;
      for (size_t j = 0; j < QK; j++) amax = std::fmax(amax, std::fabs(blk[j])); // f32::max ignores NaN
      float d = amax / 127.0f;
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t h = f32_to_f16(d);
      o[0] = (uint8_t)(h & 0xff);
      o[1] = (uint8_t)(h >> 8);
      for (size_t j = 0; j < QK; j++) o[2 + j] = (uint8_t)rust_f32_as_i8(std::round(blk[j] * id));
    } else {
      // the first element of largest magnitude, sign kept, maps to -8
      float mx = 0.0f;
      for (size_t j = 0; j < QK; j++)
        if (std::fabs(blk[j]) > std::fabs(mx)) mx = blk[j];
      float d = mx / -8.0f;
      float id = d != 0.0f ? 1.0f / d : 0.0f;
      uint16_t h = f32_to_f16(d);
      o[0] = (uint8_t)(h & 0xff);
      o[1] = (uint8_t)(h >> 8);
      auto q = [&](float v) -> uint8_t {
        float t = v * id;
        t = t + 8.5f;
        int32_t i = rust_f32_as_i32(t);
        return (uint8_t)std::min(std::max(i, 0), 15);
      };
      for (size_t j = 0; j < QK / 2; j++) o[2 + j] = q(blk[j]) | (uint8_t)(q(blk[j + QK / 2]) << 4);
    }
  }
}

// ferrum_gguf/src/codec/quant.rs:L50-L88
void decode(int kind, const uint8_t* bytes, size_t n, float* out) {
  if (kind == FC_Q2_K) return q2k_decode(bytes, n, out);
  for (size_t b = 0; b < n / QK; b++) {
    const uint8_t* p = bytes + b * block_bytes(kind);
    float* o = out + b * QK;
    if (kind == FC_F16) {
      for (size_t j = 0; j < QK; j++) o[j] = f16_to_f32((uint16_t)(p[2 * j] | (p[2 * j + 1] << 8)));
      continue;
    }
    if (kind == FC_MXFP4) { // mxfp4.rs:L31-L46
      const float hs = mxfp4_half_scale(p[0]);
      for (size_t j = 0; j < QK / 2; j++) {
        o[j] = (float)MXFP4_VALUES[p[1 + j] & 15] * hs;
        o[j + QK / 2] = (float)MXFP4_VALUES[p[1 + j] >> 4] * hs;
      }
      continue;
    }
    float d = f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
    if (is_fp8(kind)) { // fp8.rs:L127-L134
      for (size_t j = 0; j < QK; j++) o[j] = d * fp8_decode(kind, p[2 + j]);
    } else if (kind == FC_Q8_0) {
      for (size_t j = 0; j < QK; j++) o[j] = d * (float)(int8_t)p[2 + j];
    } else {
      for (size_t j = 0; j < QK / 2; j++) {
        o[j] = d * ((float)(p[2 + j] & 0x0f) - 8.0f);
        o[j + QK / 2] = d * ((float)(p[2 + j] >> 4) - 8.0f);
      }
    }
  }
}

// ferrum_ref/src/models/llama/params.rs:L24-L32
void transpose(const float* data, size_t rows, size_t cols, float* out) {
  for (size_t r = 0; r < rows; r++)
    for (size_t c = 0; c < cols; c++) out[c * rows + r] = data[r * cols + c];
}

// ---- matmul ----------------------------------------------------------------------------------

// ferrum_ref/src/kernels/matmul.rs:L49-L59: i-k-j, ascending p, separate multiply and add
void matmul_rows(const float* a, const float* b, size_t rows, size_t k, size_t n, float* out) {
  for (size_t i = 0; i < rows; i++) {
    float* row = out + i * n;
    for (size_t p = 0; p < k; p++) {
      float av = a[i * k + p];
      const float* brow = b + p * n;
      for (size_t j = 0; j < n; j++) row[j] += av * brow[j];
    }
  }
}

// ferrum_ref/src/kernels/tuned.rs:L10-L134 (`matmul_tuned`): the reference's speed baseline. Output columns in
// panels of NC, the contraction in panels of KC, a 4 x 8 register tile inside, plain loops on the edges; every
// output element still sums k in ascending order, so the result is bit-identical to the simple kernel.
constexpr size_t T_KC = 256, T_NC = 256, T_MR = 4, T_NR = 8;

// tuned.rs:L75-L97 (`edge`): rows ia..ib, columns ja..jb, p in pp..p1
void tuned_edge(const float* a, const float* b, size_t k, size_t n, size_t ia, size_t ib, size_t r0, size_t ja, size_t jb,
                size_t pp, size_t p1, float* out) {
  for (size_t i = ia; i < ib; i++)
    for (size_t p = pp; p < p1; p++) {
      const float av = a[i * k + p];
      float* o = out + (i - r0) * n;
      const float* brow = b + p * n;
      for (size_t j = ja; j < jb; j++) o[j] += av * brow[j];
    }
}

// tuned.rs:L44-L72 (`micro`): the register tile, loaded from and stored back to `out`
void tuned_micro(const float* a, const float* b, size_t k, size_t n, size_t i, size_t r0, size_t j, size_t pp, size_t p1,
                 float* out) {
  float acc[T_MR][T_NR];
  for (size_t r = 0; r < T_MR; r++) std::memcpy(acc[r], out + (i + r - r0) * n + j, sizeof acc[r]);
  for (size_t p = pp; p < p1; p++) {
    const float* bs = b + p * n + j;
    for (size_t r = 0; r < T_MR; r++) {
      const float av = a[(i + r) * k + p];
      for (size_t c = 0; c < T_NR; c++) acc[r][c] += av * bs[c];
    }
  }
  for (size_t r = 0; r < T_MR; r++) std::memcpy(out + (i + r - r0) * n + j, acc[r], sizeof acc[r]);
}

// tuned.rs:L16-L42 (`block`): rows r0..r1 into `out` (those rows, indexed locally, pre-zeroed)
void tuned_block(const float* a, const float* b, size_t k, size_t n, size_t r0, size_t r1, float* out) {
  for (size_t jj = 0; jj < n; jj += T_NC) {
    const size_t j1 = std::min(jj + T_NC, n);
    for (size_t pp = 0; pp < k; pp += T_KC) {
      const size_t p1 = std::min(pp + T_KC, k);
      size_t i = r0;
      for (; i + T_MR <= r1; i += T_MR) {
        size_t j = jj;
        for (; j + T_NR <= j1; j += T_NR) tuned_micro(a, b, k, n, i, r0, j, pp, p1, out);
        if (j < j1) tuned_edge(a, b, k, n, i, i + T_MR, r0, j, j1, pp, p1, out);
      }
      if (i < r1) tuned_edge(a, b, k, n, i, r1, r0, jj, j1, pp, p1, out);
    }
  }
}

// tuned.rs:L99-L134: rows split over scoped threads
void matmul_tuned(const float* a, const float* b, size_t m, size_t k, size_t n, float* out, int threads) {
  std::fill(out, out + m * n, 0.0f);
  if (m == 0 || n == 0) return;
  const size_t per = (m + (size_t)std::max(threads, 1) - 1) / (size_t)std::max(threads, 1);
  std::vector<std::thread> pool;
  for (size_t r0 = 0; r0 < m; r0 += per) {
    const size_t r1 = std::min(r0 + per, m);
    pool.emplace_back(tuned_block, a, b, k, n, r0, r1, out + r0 * n);
  }
  for (auto& t : pool) t.join();
}

// Which kernel the model passes multiply with: the simple one (what `--device cpu` runs,
// ferrum_ref/src/models/llama/mod.rs:L177-L184) unless the all-cores baseline asks for the tuned one.
bool g_use_tuned = false;

// ferrum_ref/src/kernels/matmul.rs:L62-L69 (threads == 1) and L73-L94 (rows split over scoped
// threads; bit-identical for any thread count because rows are independent)
void matmul(const float* a, const float* b, size_t m, size_t k, size_t n, float* out, int threads) {
  if (g_use_tuned) return matmul_tuned(a, b, m, k, n, out, threads);
  std::fill(out, out + m * n, 0.0f);
  if (m == 0 || n == 0) return;
  if (threads <= 1 || m == 1) {
    matmul_rows(a, b, m, k, n, out);
    return;
  }
  size_t per = (m + (size_t)threads - 1) / (size_t)threads;
  std::vector<std::thread> pool;
  for (size_t start = 0; start < m; start += per) {
    size_t cnt = std::min(per, m - start);
    pool.emplace_back(matmul_rows, a + start * k, b, cnt, k, n, out + start * n);
  }
  for (auto& t : pool) t.join();
}

// ferrum_ref/src/kernels/matmul.rs:L97-L107
void rand_vec(size_t len, uint64_t seed, float* out) {
  uint64_t s = seed > 1 ? seed : 1;
  for (size_t i = 0; i < len; i++) {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    out[i] = ((float)(s >> 40) / (float)(1ull << 24)) * 2.0f - 1.0f;
  }
}

// ---- nn ops ----------------------------------------------------------------------------------

constexpr float LN_EPS = 1e-5f; // ferrum_ref/src/kernels/nn.rs:L7
constexpr float MASK = -1e9f;   // nn.rs:L9

// nn.rs:L12-L15
float gelu(float x) {
  const float K = 0.7978846f;
  return 0.5f * x * (1.0f + std::tanh(K * (x + 0.044715f * x * x * x)));
}

// nn.rs:L18-L23
void add_bias(float* x, const float* bias, size_t rows, size_t n) {
  for (size_t i = 0; i < rows * n; i++) x[i] = x[i] + bias[i % n];
}

// nn.rs:L31-L43 (two-pass variance, eps fixed)
void layernorm(const float* x, const float* g, const float* b, size_t rows, size_t cols, float* y) {
  for (size_t r = 0; r < rows; r++) {
    const float* row = x + r * cols;
    float sum = 0.0f;
    for (size_t c = 0; c < cols; c++) sum += row[c];
    float mean = sum / (float)cols;
    float vs = 0.0f;
    for (size_t c = 0; c < cols; c++) {
      float dlt = row[c] - mean;
      vs += dlt * dlt; // powi(2)
    }
    float var = vs / (float)cols;
    float is = 1.0f / std::sqrt(var + LN_EPS);
    for (size_t c = 0; c < cols; c++) y[r * cols + c] = (row[c] - mean) * is * g[c] + b[c];
  }
}

// nn.rs:L47-L90: causal MHA; probabilities divided one by one, then the weighted sum over all t
// columns (masked columns hold exp(-1e9 - max) == 0)
void attention(const float* q, const float* k, const float* v, size_t batch, size_t t, size_t heads,
               size_t hd, float* out) {
  size_t c = heads * hd;
  float scale = 1.0f / std::sqrt((float)hd);
  std::vector<float> s(t), p(t);
  for (size_t b = 0; b < batch; b++)
    for (size_t h = 0; h < heads; h++)
      for (size_t i = 0; i < t; i++) {
        for (size_t j = 0; j < t; j++) s[j] = MASK;
        for (size_t j = 0; j <= i; j++) {
          float dot = 0.0f;
          for (size_t d = 0; d < hd; d++) dot += q[(b * t + i) * c + h * hd + d] * k[(b * t + j) * c + h * hd + d];
          s[j] = dot * scale;
        }
        float mx = -std::numeric_limits<float>::infinity();
        for (size_t j = 0; j < t; j++) mx = std::fmax(mx, s[j]);
        float sum = 0.0f;
        for (size_t j = 0; j < t; j++) {
          s[j] = std::exp(s[j] - mx);
          sum += s[j];
        }
        for (size_t j = 0; j < t; j++) p[j] = s[j] / sum;
        for (size_t d = 0; d < hd; d++) {
          float acc = 0.0f;
          for (size_t j = 0; j < t; j++) acc += p[j] * v[(b * t + j) * c + h * hd + d];
          out[(b * t + i) * c + h * hd + d] = acc;
        }
      }
}

// nn.rs:L117-L129: log-probability of the target and "target is the first argmax"
void score(const float* logits, const int32_t* targets, size_t rows, size_t vocab, float* logprob,
           uint8_t* greedy) {
  for (size_t i = 0; i < rows; i++) {
    const float* row = logits + i * vocab;
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t j = 0; j < vocab; j++) mx = std::fmax(mx, row[j]);
    float se = 0.0f;
    for (size_t j = 0; j < vocab; j++) se += std::exp(row[j] - mx);
    float lse = std::log(se);
    size_t first = 0;
    for (size_t j = 0; j < vocab; j++)
      if (row[j] == mx) {
        first = j;
        break;
      }
    logprob[i] = row[targets[i]] - mx - lse;
    greedy[i] = first == (size_t)targets[i];
  }
}

// ferrum_gpu_core/src/serving/decoder.rs:L69-L83: f64 log-sum-exp; greedy = target reaches the
// maximum (any tie)
void logprobs_f64(const float* logits, const int32_t* targets, size_t rows, size_t vocab, double* lp,
                  uint8_t* greedy) {
  for (size_t i = 0; i < rows; i++) {
    const float* row = logits + i * vocab;
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t j = 0; j < vocab; j++) mx = std::fmax(mx, row[j]);
    double se = 0.0;
    for (size_t j = 0; j < vocab; j++) se += std::exp((double)(row[j] - mx));
    lp[i] = (double)(row[targets[i]] - mx) - std::log(se);
    greedy[i] = row[targets[i]] >= mx;
  }
}

// ferrum_model/src/sampling.rs:L32-L40: strictly greater wins, so the first maximum; NaN never
// wins
int32_t argmax(const float* v, size_t n) {
  int32_t best = 0;
  float bv = -std::numeric_limits<float>::infinity();
  for (size_t i = 0; i < n; i++)
    if (v[i] > bv) {
      bv = v[i];
      best = (int32_t)i;
    }
  return best;
}

// ---- Llama ops -------------------------------------------------------------------------------

// ferrum_ref/src/models/llama/ops.rs:L55-L66
void rmsnorm(const float* x, const float* g, size_t rows, size_t cols, float eps, float* y) {
  for (size_t r = 0; r < rows; r++) {
    const float* row = x + r * cols;
    float ss = 0.0f;
    for (size_t c = 0; c < cols; c++) ss += row[c] * row[c];
    float ms = ss / (float)cols;
    float inv = 1.0f / std::sqrt(ms + eps);
    for (size_t c = 0; c < cols; c++) y[r * cols + c] = row[c] * inv * g[c];
  }
}

// ops.rs:L69-L71
float silu(float x) { return x / (1.0f + std::exp(-x)); }

// ops.rs:L80-L101: powf in f64, everything after in f32, left to right
void rope_tables(size_t start, size_t n, size_t rope_dim, float base, const float* freq_factors,
                 size_t n_ff, float linear_factor, float* cos_out, float* sin_out) {
  size_t half = rope_dim / 2;
  for (size_t p = start; p < start + n; p++)
    for (size_t i = 0; i < half; i++) {
      float freq = (float)std::pow((double)base, -2.0 * (double)i / (double)rope_dim);
      float ff = i < n_ff ? freq_factors[i] : 1.0f;
      float theta = (float)p * freq / ff * (1.0f / linear_factor);
      cos_out[(p - start) * half + i] = std::cos(theta);
      sin_out[(p - start) * half + i] = std::sin(theta);
    }
}

// ops.rs:L105-L127
void apply_rope(float* x, size_t rows, size_t heads, size_t hd, size_t rope_dim, const float* cosv,
                const float* sinv, int type) {
  size_t half = rope_dim / 2;
  for (size_t r = 0; r < rows; r++)
    for (size_t h = 0; h < heads; h++) {
      size_t off = (r * heads + h) * hd;
      for (size_t i = 0; i < half; i++) {
        size_t ia = type == FC_ROPE_NORM ? off + 2 * i : off + i;
        size_t ib = type == FC_ROPE_NORM ? off + 2 * i + 1 : off + i + half;
        float c = cosv[r * half + i], s = sinv[r * half + i];
        float a = x[ia], b = x[ib];
        x[ia] = a * c - b * s;
        x[ib] = a * s + b * c;
      }
    }
}

// ops.rs:L131-L162: one query row over `len` cached positions; each probability is divided by
// the sum before it multiplies v
void attend_row(const float* q, const float* k, const float* v, size_t len, size_t heads,
                size_t kv_heads, size_t hd, float* out) {
  size_t kv_dim = kv_heads * hd;
  size_t group = heads / kv_heads;
  float scale = 1.0f / std::sqrt((float)hd);
  std::vector<float> s(len);
  for (size_t h = 0; h < heads; h++) {
    size_t off = (h / group) * hd;
    for (size_t j = 0; j < len; j++) {
      float dot = 0.0f;
      for (size_t d = 0; d < hd; d++) dot += q[h * hd + d] * k[j * kv_dim + off + d];
      s[j] = dot * scale;
    }
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t j = 0; j < len; j++) mx = std::fmax(mx, s[j]);
    float sum = 0.0f;
    for (size_t j = 0; j < len; j++) {
      s[j] = std::exp(s[j] - mx);
      sum += s[j];
    }
    for (size_t d = 0; d < hd; d++) {
      float acc = 0.0f;
      for (size_t j = 0; j < len; j++) acc += s[j] / sum * v[j * kv_dim + off + d];
      out[h * hd + d] = acc;
    }
  }
}

// ---- models ----------------------------------------------------------------------------------

struct LlamaBlockW {
  std::vector<float> attn_norm, wq, bq, wk, bk, wv, bv, wo, ffn_norm, gate, up, down;
};

struct OrLlama {
  FcLlamaConfig cfg;
  std::vector<float> freq_factors;
  std::vector<float> tok, out_norm, head;
  std::vector<LlamaBlockW> blocks;
  // Cache (ferrum_ref/src/models/llama/mod.rs:L149-L174)
  std::vector<std::vector<float>> ck, cv;
  int threads = 1;
};

struct Gpt2BlockW {
  std::vector<float> ln1_g, ln1_b, wq, bq, wk, bk, wv, bv, wo, bo, ln2_g, ln2_b, w1, b1, w2, b2;
};

struct OrGpt2 {
  FcGpt2Config cfg;
  std::vector<float> tok, pos, lnf_g, lnf_b, head;
  std::vector<Gpt2BlockW> blocks;
  std::vector<std::vector<float>> ck, cv;
  int threads = 1;
};

std::vector<float> vec(const float* p, size_t n) {
  return p ? std::vector<float>(p, p + n) : std::vector<float>();
}

// ferrum_ref/src/models/llama/mod.rs:L176-L184
std::vector<float> linear(const std::vector<float>& x, const std::vector<float>& w,
                          const std::vector<float>& bias, size_t rows, size_t k, size_t n, int threads) {
  std::vector<float> y(rows * n);
  matmul(x.data(), w.data(), rows, k, n, y.data(), threads);
  if (!bias.empty()) add_bias(y.data(), bias.data(), rows, n);
  return y;
}

// ferrum_ref/src/models/llama/mod.rs:L209-L259 (`run`): ids through the stack starting at the
// cache length, appending keys and values; logits for every new row
// (`last_only`: the head product for the last new row alone - rows are independent, so its logits are the same)
int llama_run(OrLlama& m, const int32_t* ids, size_t n, float* logits_out, bool last_only = false) {
  const FcLlamaConfig& c = m.cfg;
  size_t d = c.dim, kvd = (size_t)c.kv_heads * c.head_dim, qd = (size_t)c.heads * c.head_dim;
  for (size_t i = 0; i < n; i++)
    if (ids[i] < 0 || (uint32_t)ids[i] >= c.vocab) return FC_ERR_RANGE;
  size_t start = m.ck.empty() ? 0 : m.ck[0].size() / kvd;
  size_t half = c.rope_dim / 2;
  std::vector<float> cosv(n * half), sinv(n * half);
  rope_tables(start, n, c.rope_dim, c.rope_base, m.freq_factors.data(), m.freq_factors.size(),
              c.rope_linear_factor, cosv.data(), sinv.data());
  std::vector<float> x(n * d);
  for (size_t i = 0; i < n; i++) std::copy_n(m.tok.data() + (size_t)ids[i] * d, d, x.data() + i * d);
  std::vector<float> h(n * d);
  for (size_t l = 0; l < c.layers; l++) {
    const LlamaBlockW& b = m.blocks[l];
    rmsnorm(x.data(), b.attn_norm.data(), n, d, c.eps, h.data());
    auto q = linear(h, b.wq, b.bq, n, d, qd, m.threads);
    auto k = linear(h, b.wk, b.bk, n, d, kvd, m.threads);
    auto v = linear(h, b.wv, b.bv, n, d, kvd, m.threads);
    apply_rope(q.data(), n, c.heads, c.head_dim, c.rope_dim, cosv.data(), sinv.data(), (int)c.rope_type);
    apply_rope(k.data(), n, c.kv_heads, c.head_dim, c.rope_dim, cosv.data(), sinv.data(), (int)c.rope_type);
    m.ck[l].insert(m.ck[l].end(), k.begin(), k.end());
    m.cv[l].insert(m.cv[l].end(), v.begin(), v.end());
    std::vector<float> a(n * qd);
    auto rows_fn = [&](size_t r0, size_t r1) {
      for (size_t r = r0; r < r1; r++)
        attend_row(q.data() + r * qd, m.ck[l].data(), m.cv[l].data(), start + r + 1, c.heads, c.kv_heads,
                   c.head_dim, a.data() + r * qd);
    };
    if (m.threads > 1 && n > 1) { // rows are independent: same values for any split
      size_t per = (n + (size_t)m.threads - 1) / (size_t)m.threads;
      std::vector<std::thread> pool;
      for (size_t s0 = 0; s0 < n; s0 += per) pool.emplace_back(rows_fn, s0, std::min(n, s0 + per));
      for (auto& t : pool) t.join();
    } else {
      rows_fn(0, n);
    }
    auto o = linear(a, b.wo, {}, n, qd, d, m.threads);
    for (size_t i = 0; i < n * d; i++) x[i] = x[i] + o[i];
    rmsnorm(x.data(), b.ffn_norm.data(), n, d, c.eps, h.data());
    auto g = linear(h, b.gate, {}, n, d, c.hidden, m.threads);
    auto u = linear(h, b.up, {}, n, d, c.hidden, m.threads);
    for (size_t i = 0; i < g.size(); i++) g[i] = silu(g[i]) * u[i]; // ops.rs:L74-L76
    auto f = linear(g, b.down, {}, n, c.hidden, d, m.threads);
    for (size_t i = 0; i < n * d; i++) x[i] = x[i] + f[i];
  }
  rmsnorm(x.data(), m.out_norm.data(), n, d, c.eps, h.data());
  if (last_only)
    matmul(h.data() + (n - 1) * d, m.head.data(), 1, d, c.vocab, logits_out, 1);
  else
    matmul(h.data(), m.head.data(), n, d, c.vocab, logits_out, m.threads);
  return FC_OK;
}

// ferrum_ref/src/models/gpt2/mod.rs:L203-L230 (`forward_logits`)
int gpt2_forward(OrGpt2& m, const int32_t* ids, size_t t, float* logits_out) {
  const FcGpt2Config& c = m.cfg;
  if (t == 0 || t > c.ctx) return FC_ERR_SHAPE;
  for (size_t i = 0; i < t; i++)
    if (ids[i] < 0 || (uint32_t)ids[i] >= c.vocab) return FC_ERR_RANGE;
  size_t d = c.dim, hd = d / c.heads;
  std::vector<float> x(t * d), h(t * d), a(t * d);
  for (size_t r = 0; r < t; r++) // nn.rs:L132-L140 (`embed`)
    for (size_t i = 0; i < d; i++) x[r * d + i] = m.tok[(size_t)ids[r] * d + i] + m.pos[(r % t) * d + i];
  for (size_t l = 0; l < c.layers; l++) {
    const Gpt2BlockW& b = m.blocks[l];
    layernorm(x.data(), b.ln1_g.data(), b.ln1_b.data(), t, d, h.data());
    auto q = linear(h, b.wq, b.bq, t, d, d, m.threads);
    auto k = linear(h, b.wk, b.bk, t, d, d, m.threads);
    auto v = linear(h, b.wv, b.bv, t, d, d, m.threads);
    attention(q.data(), k.data(), v.data(), 1, t, c.heads, hd, a.data());
    auto o = linear(a, b.wo, b.bo, t, d, d, m.threads);
    for (size_t i = 0; i < t * d; i++) x[i] = x[i] + o[i];
    layernorm(x.data(), b.ln2_g.data(), b.ln2_b.data(), t, d, h.data());
    auto f = linear(h, b.w1, b.b1, t, d, c.hidden, m.threads);
    for (auto& e : f) e = gelu(e);
    auto f2 = linear(f, b.w2, b.b2, t, c.hidden, d, m.threads);
    for (size_t i = 0; i < t * d; i++) x[i] = x[i] + f2[i];
  }
  layernorm(x.data(), m.lnf_g.data(), m.lnf_b.data(), t, d, h.data());
  matmul(h.data(), m.head.data(), t, d, c.vocab, logits_out, m.threads);
  return FC_OK;
}

// ferrum_ref/src/models/gpt2/decode.rs:L42-L55 (`gemv`): rows of w accumulated in ascending k,
// bias added after
std::vector<float> gemv(const std::vector<float>& x, const std::vector<float>& w, const std::vector<float>* bias,
                        size_t n) {
  std::vector<float> y(n, 0.0f);
  for (size_t p = 0; p < x.size(); p++) {
    float xv = x[p];
    const float* wr = w.data() + p * n;
    for (size_t j = 0; j < n; j++) y[j] += xv * wr[j];
  }
  if (bias)
    for (size_t j = 0; j < n; j++) y[j] += (*bias)[j];
  return y;
}

// ferrum_ref/src/models/gpt2/decode.rs:L57-L116 (`feed`)
int gpt2_feed(OrGpt2& m, int32_t token, float* logits_out) {
  const FcGpt2Config& c = m.cfg;
  size_t d = c.dim, pos = m.ck[0].size() / d;
  if (pos >= c.ctx) return FC_ERR_CONTEXT_FULL;
  if (token < 0 || (uint32_t)token >= c.vocab) return FC_ERR_RANGE;
  size_t hd = d / c.heads;
  std::vector<float> x(d), h(d);
  for (size_t i = 0; i < d; i++) x[i] = m.tok[(size_t)token * d + i] + m.pos[pos * d + i];
  for (size_t l = 0; l < c.layers; l++) {
    const Gpt2BlockW& b = m.blocks[l];
    layernorm(x.data(), b.ln1_g.data(), b.ln1_b.data(), 1, d, h.data());
    auto q = gemv(h, b.wq, &b.bq, d);
    auto kk = gemv(h, b.wk, &b.bk, d);
    auto vv = gemv(h, b.wv, &b.bv, d);
    m.ck[l].insert(m.ck[l].end(), kk.begin(), kk.end());
    m.cv[l].insert(m.cv[l].end(), vv.begin(), vv.end());
    const std::vector<float>&kc = m.ck[l], &vc = m.cv[l];
    float scale = 1.0f / std::sqrt((float)hd);
    std::vector<float> a(d, 0.0f), s(pos + 1);
    for (size_t hh = 0; hh < c.heads; hh++) {
      for (size_t j = 0; j <= pos; j++) {
        float dot = 0.0f;
        for (size_t i = 0; i < hd; i++) dot += q[hh * hd + i] * kc[j * d + hh * hd + i];
        s[j] = dot * scale;
      }
      float mx = -std::numeric_limits<float>::infinity();
      for (size_t j = 0; j <= pos; j++) mx = std::fmax(mx, s[j]);
      float sum = 0.0f;
      for (size_t j = 0; j <= pos; j++) {
        s[j] = std::exp(s[j] - mx);
        sum += s[j];
      }
      for (size_t i = 0; i < hd; i++) {
        float acc = 0.0f;
        for (size_t j = 0; j <= pos; j++) acc += s[j] / sum * vc[j * d + hh * hd + i];
        a[hh * hd + i] = acc;
      }
    }
    auto o = gemv(a, b.wo, &b.bo, d);
    for (size_t i = 0; i < d; i++) x[i] = x[i] + o[i];
    layernorm(x.data(), b.ln2_g.data(), b.ln2_b.data(), 1, d, h.data());
    auto f = gemv(h, b.w1, &b.b1, c.hidden);
    for (auto& e : f) e = gelu(e);
    auto f2 = gemv(f, b.w2, &b.b2, d);
    for (size_t i = 0; i < d; i++) x[i] = x[i] + f2[i];
  }
  layernorm(x.data(), m.lnf_g.data(), m.lnf_b.data(), 1, d, h.data());
  auto lg = gemv(h, m.head, nullptr, c.vocab);
  std::copy(lg.begin(), lg.end(), logits_out);
  return FC_OK;
}

} // namespace

// ================================ exported C interface ========================================

OR_API float or_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
OR_API uint16_t or_f32_to_f16(float x) { return f32_to_f16(x); }

// MXFP4 pieces (ferrum_gguf/src/codec/mxfp4.rs:L22-L28, L49-L54)
OR_API float or_mxfp4_half_scale(uint8_t e) { return mxfp4_half_scale(e); }
OR_API uint8_t or_mxfp4_scale_byte(float amax) { return mxfp4_scale_byte(amax); }

// One FP8 code <-> f32 (ferrum_gguf/src/codec/fp8.rs:L41-L109)
OR_API float or_fp8_decode(int kind, uint8_t code) { return fp8_decode(kind, code); }
OR_API uint8_t or_fp8_encode(int kind, float x) { return fp8_encode(kind, x); }

OR_API size_t or_block_bytes(int kind, size_t n) {
  if (kind == FC_F32) return n * 4;
  if (kind == FC_Q2_K) return n % QK_K ? 0 : n / QK_K * Q2K_BLOCK;
  if (n % QK) return 0;
  return n / QK * block_bytes(kind);
}

// `effective` (ferrum_wgpu/src/ops/quant.rs:L134-L144): Q2_K needs 256-wide blocks; a width that is whole
// 32s only is stored as Q4_0 instead.
OR_API int or_effective_kind(int kind, size_t k) {
  return (kind == FC_Q2_K && k % QK_K != 0 && k > 0 && k % QK == 0) ? FC_Q4_0 : kind;
}
OR_API int32_t or_q2k_nearest_int(float x) { return q2k_nearest_int(x); }

// ferrum_gguf::quant::encode / decode over whole-block data; returns FC_ERR_SHAPE for a length
// that is not whole blocks (quant.rs:L19-L23)
OR_API int or_encode(int kind, const float* data, size_t n, uint8_t* out) {
  if (n % (kind == FC_Q2_K ? QK_K : QK)) return FC_ERR_SHAPE;
  encode(kind, data, n, out);
  return FC_OK;
}
OR_API int or_decode(int kind, const uint8_t* bytes, size_t n, float* out) {
  if (n % (kind == FC_Q2_K ? QK_K : QK)) return FC_ERR_SHAPE;
  decode(kind, bytes, n, out);
  return FC_OK;
}

// ferrum_wgpu/src/ops/quant.rs:L238-L252: `[k, n]` f32 -> transpose -> encode rows
OR_API int or_quantise_matrix(int kind, const float* w, size_t k, size_t n, uint8_t* out) {
  if (k == 0 || k % (kind == FC_Q2_K ? QK_K : QK)) return FC_ERR_SHAPE;
  std::vector<float> rows(k * n);
  transpose(w, k, n, rows.data());
  encode(kind, rows.data(), k * n, out);
  return FC_OK;
}

// The `snap` closure of ferrum_wgpu/src/models/llama/mod.rs:L188-L199: quantise, decode,
// transpose back to `[k, n]`; an ineligible width is returned unchanged
OR_API int or_snap_matrix(int kind, const float* w, size_t k, size_t n, float* out) {
  kind = or_effective_kind(kind, k);
  if (kind == FC_F32 || k == 0 || k % QK) {
    std::copy(w, w + k * n, out);
    return FC_OK;
  }
  std::vector<uint8_t> bytes(or_block_bytes(kind, k * n));
  or_quantise_matrix(kind, w, k, n, bytes.data());
  std::vector<float> rows(k * n);
  decode(kind, bytes.data(), k * n, rows.data());
  transpose(rows.data(), n, k, out);
  return FC_OK;
}

// Encode then decode a tensor along its own rows (what a GGUF round trip does to the token
// embedding: ferrum_model/src/gguf/llama/mod.rs:L297-L316, gguf/gpt2.rs:L205-L231)
OR_API int or_snap_rows(int kind, const float* data, size_t n, float* out) {
  if (kind == FC_F32) {
    std::copy(data, data + n, out);
    return FC_OK;
  }
  if (n % (kind == FC_Q2_K ? QK_K : QK)) return FC_ERR_SHAPE;
  std::vector<uint8_t> bytes(or_block_bytes(kind, n));
  encode(kind, data, n, bytes.data());
  decode(kind, bytes.data(), n, out);
  return FC_OK;
}

// ferrum_wgpu/src/ops/quant.rs:L186-L234 (`pack`) for Q8_0 / Q4_0: the reference's own device
// layout (block-major records, scale widened to f32 bits). Restated only so its layout
// known-answer test can pin the block order this repository's repack starts from.
OR_API int or_pack_reference_layout(int kind, const uint8_t* bytes, size_t k, size_t n, uint32_t* out) {
  if (k == 0 || k % QK) return FC_ERR_SHAPE;
  size_t nb = k / QK, fb = block_bytes(kind), w = kind == FC_Q8_0 ? 1 + QK / 4 : 1 + QK / 8;
  for (size_t col = 0; col < n; col++)
    for (size_t b = 0; b < nb; b++) {
      const uint8_t* blk = bytes + (col * nb + b) * fb;
      uint32_t* rec = out + (b * n + col) * w;
      float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
      std::memcpy(&rec[0], &d, 4);
      for (size_t i = 0; i + 1 < w; i++)
        rec[1 + i] = (uint32_t)blk[2 + 4 * i] | ((uint32_t)blk[3 + 4 * i] << 8) | ((uint32_t)blk[4 + 4 * i] << 16) |
                     ((uint32_t)blk[5 + 4 * i] << 24);
    }
  return FC_OK;
}

OR_API void or_transpose(const float* data, size_t rows, size_t cols, float* out) { transpose(data, rows, cols, out); }
OR_API void or_matmul(const float* a, const float* b, size_t m, size_t k, size_t n, float* out, int threads) {
  matmul(a, b, m, k, n, out, threads);
}
OR_API void or_matmul_tuned(const float* a, const float* b, size_t m, size_t k, size_t n, float* out, int threads) {
  matmul_tuned(a, b, m, k, n, out, threads);
}
// Every later product of the model passes on the tuned kernel (1) or the simple one (0); results are bit-identical.
OR_API void or_set_tuned(int on) { g_use_tuned = on != 0; }
OR_API void or_rand_vec(size_t len, uint64_t seed, float* out) { rand_vec(len, seed, out); }
OR_API float or_gelu(float x) { return gelu(x); }
OR_API float or_silu(float x) { return silu(x); }
OR_API void or_layernorm(const float* x, const float* g, const float* b, size_t rows, size_t cols, float* y) {
  layernorm(x, g, b, rows, cols, y);
}
OR_API void or_rmsnorm(const float* x, const float* g, size_t rows, size_t cols, float eps, float* y) {
  rmsnorm(x, g, rows, cols, eps, y);
}
OR_API void or_rope_tables(size_t start, size_t n, size_t rope_dim, float base, const float* ff, size_t n_ff,
                           float linear, float* cos_out, float* sin_out) {
  rope_tables(start, n, rope_dim, base, ff, n_ff, linear, cos_out, sin_out);
}
OR_API void or_apply_rope(float* x, size_t rows, size_t heads, size_t hd, size_t rope_dim, const float* c,
                          const float* s, int type) {
  apply_rope(x, rows, heads, hd, rope_dim, c, s, type);
}
OR_API void or_attend_row(const float* q, const float* k, const float* v, size_t len, size_t heads, size_t kv_heads,
                          size_t hd, float* out) {
  attend_row(q, k, v, len, heads, kv_heads, hd, out);
}
OR_API void or_attention(const float* q, const float* k, const float* v, size_t batch, size_t t, size_t heads,
                         size_t hd, float* out) {
  attention(q, k, v, batch, t, heads, hd, out);
}
OR_API void or_score(const float* logits, const int32_t* targets, size_t rows, size_t vocab, float* lp, uint8_t* g) {
  score(logits, targets, rows, vocab, lp, g);
}
OR_API void or_logprobs_f64(const float* logits, const int32_t* targets, size_t rows, size_t vocab, double* lp,
                            uint8_t* g) {
  logprobs_f64(logits, targets, rows, vocab, lp, g);
}
OR_API int32_t or_argmax(const float* v, size_t n) { return argmax(v, n); }

static float or_rng_next_f32_fwd(uint64_t* state);
// ferrum_model/src/sampling.rs:L42-L100 `sample`: repetition penalty over `recent` in order (a token
// listed twice is penalised twice), temperature <= 0 -> argmax, else candidates = non-NaN logits in
// descending `total_cmp` order (stable: ties keep the lower index first), truncated to top_k, softmax
// of (l - max) / temperature with sequential f32 sums, nucleus cut at top_p with renormalisation, one
// `next_f32` draw, the last candidate as the fallback. `rng_state` advances only when a draw is made.
static inline uint32_t total_order_key(float v) {  // ascending key order == f32::total_cmp order
  uint32_t b;
  memcpy(&b, &v, 4);
  return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}
OR_API int32_t or_sample(const float* logits, size_t n, float temperature, size_t top_k, float top_p, float rep_penalty,
                         const int64_t* recent, size_t n_recent, uint64_t* rng_state) {
  std::vector<float> l(logits, logits + n);
  if (rep_penalty != 1.0f) {
    for (size_t i = 0; i < n_recent; i++) {
      if (recent[i] >= 0 && (size_t)recent[i] < n) {
        float& v = l[(size_t)recent[i]];
        v = v > 0.0f ? v / rep_penalty : v * rep_penalty;
      }
    }
  }
  if (temperature <= 0.0f) return argmax(l.data(), n);
  std::vector<size_t> idx;
  for (size_t i = 0; i < n; i++)
    if (!std::isnan(l[i])) idx.push_back(i);
  if (idx.empty()) return 0;
  std::stable_sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return total_order_key(l[a]) > total_order_key(l[b]); });
  if (top_k > 0 && idx.size() > top_k) idx.resize(top_k);
  const float mx = l[idx[0]];
  std::vector<float> probs(idx.size());
  for (size_t i = 0; i < idx.size(); i++) probs[i] = expf((l[idx[i]] - mx) / temperature);
  float sum = 0.0f;
  for (float x : probs) sum += x;
  for (float& x : probs) x /= sum;
  if (top_p < 1.0f) {
    float acc = 0.0f;
    size_t keep = probs.size();
    for (size_t i = 0; i < probs.size(); i++) {
      acc += probs[i];
      if (acc >= top_p) {
        keep = i + 1;
        break;
      }
    }
    idx.resize(keep);
    probs.resize(keep);
    float s2 = 0.0f;
    for (float x : probs) s2 += x;
    for (float& x : probs) x /= s2;
  }
  const float r = or_rng_next_f32_fwd(rng_state);
  float acc = 0.0f;
  for (size_t i = 0; i < idx.size(); i++) {
    acc += probs[i];
    if (r < acc) return (int32_t)idx[i];
  }
  return (int32_t)idx.back();
}

// ferrum_ref/src/kernels/rng.rs:L7-L41 (xorshift64*): `state` is the caller's generator
OR_API uint64_t or_rng_new(uint64_t seed) { return seed == 0 ? 0x9e3779b97f4a7c15ull : seed; }
OR_API uint64_t or_rng_next_u64(uint64_t* state) {
  uint64_t s = *state;
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  *state = s;
  return s * 0x2545f4914f6cdd1dull;
}
OR_API float or_rng_next_f32(uint64_t* state) { return (float)(or_rng_next_u64(state) >> 40) / (float)(1ull << 24); }
static float or_rng_next_f32_fwd(uint64_t* state) { return or_rng_next_f32(state); }
OR_API uint64_t or_rng_below(uint64_t* state, uint64_t n) {
  uint64_t zone = UINT64_MAX - (UINT64_MAX % n);
  for (;;) {
    uint64_t r = or_rng_next_u64(state);
    if (r < zone) return r % n;
  }
}

// ---- model handles ---------------------------------------------------------------------------

OR_API void* or_llama_create(const FcLlamaConfig* cfg, const FcLlamaWeights* w, int threads) {
  auto* m = new OrLlama();
  m->cfg = *cfg;
  m->freq_factors = vec(cfg->freq_factors, cfg->n_freq_factors);
  m->cfg.freq_factors = nullptr;
  size_t d = cfg->dim, qd = (size_t)cfg->heads * cfg->head_dim, kvd = (size_t)cfg->kv_heads * cfg->head_dim,
         hid = cfg->hidden;
  m->tok = vec(w->tok, (size_t)cfg->vocab * d);
  m->out_norm = vec(w->out_norm, d);
  m->head = vec(w->head, d * cfg->vocab);
  for (uint32_t l = 0; l < cfg->layers; l++) {
    const FcLlamaBlock& b = w->blocks[l];
    LlamaBlockW o;
    o.attn_norm = vec(b.attn_norm, d);
    o.wq = vec(b.wq, d * qd);
    o.bq = vec(b.bq, qd);
    o.wk = vec(b.wk, d * kvd);
    o.bk = vec(b.bk, kvd);
    o.wv = vec(b.wv, d * kvd);
    o.bv = vec(b.bv, kvd);
    o.wo = vec(b.wo, qd * d);
    o.ffn_norm = vec(b.ffn_norm, d);
    o.gate = vec(b.gate, d * hid);
    o.up = vec(b.up, d * hid);
    o.down = vec(b.down, hid * d);
    m->blocks.push_back(std::move(o));
  }
  m->ck.assign(cfg->layers, {});
  m->cv.assign(cfg->layers, {});
  m->threads = threads < 1 ? 1 : threads;
  return m;
}
OR_API void or_llama_destroy(void* h) { delete (OrLlama*)h; }
OR_API void or_llama_reset(void* h) {
  auto* m = (OrLlama*)h;
  for (auto& v : m->ck) v.clear();
  for (auto& v : m->cv) v.clear();
}
OR_API uint32_t or_llama_pos(void* h) {
  auto* m = (OrLlama*)h;
  return (uint32_t)(m->ck[0].size() / ((size_t)m->cfg.kv_heads * m->cfg.head_dim));
}
// Llama::feed (models/llama/mod.rs:L198-L204)
OR_API int or_llama_feed(void* h, int32_t token, float* logits_out) {
  auto* m = (OrLlama*)h;
  if (or_llama_pos(h) >= m->cfg.ctx) return FC_ERR_CONTEXT_FULL;
  return llama_run(*m, &token, 1, logits_out);
}
// Llama::forward_logits (models/llama/mod.rs:L186-L196): a fresh cache, so stateless
OR_API int or_llama_forward_logits(void* h, const int32_t* ids, uint32_t n, float* logits_out) {
  auto* m = (OrLlama*)h;
  if (n == 0 || n > m->cfg.ctx) return FC_ERR_SHAPE;
  auto sk = std::move(m->ck), sv = std::move(m->cv);
  m->ck.assign(m->cfg.layers, {});
  m->cv.assign(m->cfg.layers, {});
  int rc = llama_run(*m, ids, n, logits_out);
  m->ck = std::move(sk);
  m->cv = std::move(sv);
  return rc;
}
// Continue the cached context with several tokens at once (`run` with n > 1 on a live cache)
OR_API int or_llama_extend(void* h, const int32_t* ids, uint32_t n, float* logits_out) {
  auto* m = (OrLlama*)h;
  if (or_llama_pos(h) + n > m->cfg.ctx) return FC_ERR_CONTEXT_FULL;
  return llama_run(*m, ids, n, logits_out);
}

// The same, returning the logits of the last new position only (a long prompt of a large-vocabulary model)
OR_API int or_llama_extend_last(void* h, const int32_t* ids, uint32_t n, float* logits_last) {
  auto* m = (OrLlama*)h;
  if (n == 0) return FC_ERR_SHAPE;
  if (or_llama_pos(h) + n > m->cfg.ctx) return FC_ERR_CONTEXT_FULL;
  return llama_run(*m, ids, n, logits_last, true);
}

OR_API void* or_gpt2_create(const FcGpt2Config* cfg, const FcGpt2Weights* w, int threads) {
  auto* m = new OrGpt2();
  m->cfg = *cfg;
  size_t d = cfg->dim, hid = cfg->hidden;
  m->tok = vec(w->tok, (size_t)cfg->vocab * d);
  m->pos = vec(w->pos, (size_t)cfg->ctx * d);
  m->lnf_g = vec(w->lnf_g, d);
  m->lnf_b = vec(w->lnf_b, d);
  m->head = vec(w->head, d * cfg->vocab);
  for (uint32_t l = 0; l < cfg->layers; l++) {
    const FcGpt2Block& b = w->blocks[l];
    Gpt2BlockW o;
    o.ln1_g = vec(b.ln1_g, d);
    o.ln1_b = vec(b.ln1_b, d);
    o.wq = vec(b.wq, d * d);
    o.bq = vec(b.bq, d);
    o.wk = vec(b.wk, d * d);
    o.bk = vec(b.bk, d);
    o.wv = vec(b.wv, d * d);
    o.bv = vec(b.bv, d);
    o.wo = vec(b.wo, d * d);
    o.bo = vec(b.bo, d);
    o.ln2_g = vec(b.ln2_g, d);
    o.ln2_b = vec(b.ln2_b, d);
    o.w1 = vec(b.w1, d * hid);
    o.b1 = vec(b.b1, hid);
    o.w2 = vec(b.w2, hid * d);
    o.b2 = vec(b.b2, d);
    m->blocks.push_back(std::move(o));
  }
  m->ck.assign(cfg->layers, {});
  m->cv.assign(cfg->layers, {});
  m->threads = threads < 1 ? 1 : threads;
  return m;
}
OR_API void or_gpt2_destroy(void* h) { delete (OrGpt2*)h; }
OR_API void or_gpt2_reset(void* h) {
  auto* m = (OrGpt2*)h;
  for (auto& v : m->ck) v.clear();
  for (auto& v : m->cv) v.clear();
}
OR_API uint32_t or_gpt2_pos(void* h) {
  auto* m = (OrGpt2*)h;
  return (uint32_t)(m->ck[0].size() / m->cfg.dim);
}
OR_API int or_gpt2_feed(void* h, int32_t token, float* logits_out) { return gpt2_feed(*(OrGpt2*)h, token, logits_out); }
OR_API int or_gpt2_forward_logits(void* h, const int32_t* ids, uint32_t n, float* logits_out) {
  return gpt2_forward(*(OrGpt2*)h, ids, n, logits_out);
}
