// Single-row decode product for the block formats: y[n] = x[k] . W[n, k]^T (+ bias, activation,
// residual), one row of x, streamed at the speed of the weight planes. Replaces qgemv.wgsl
// (ferrum_wgpu/src/shaders/quant/qgemv.wgsl:L88-L115, chosen by ops/quant.rs:L314-L323) for Q8_0, Q4_0
// and the formats that share their planes (FP8, MXFP4).
//
// Why not the f32 FMA kernel of matvec.cu: turning a packed weight into a float and multiplying it
// costs 3.5 (Q8_0) to 5 (Q4_0) issue slots per weight, which caps the stream at a third to a half of
// the HBM rate. Here the multiply-adds run on the tensor cores and the only per-weight work left is
// the unpack to fp16 (about 1.2 slots per weight):
//
//   * one persistent CTA per SM owns a contiguous range of 16-row tiles. Its work is counted in units
//     (one tile x one stage of K) laid out tile after tile, and every warp takes an equal, contiguous
//     share of the units, whatever the number of tiles: a share may end in the middle of a tile and the
//     next warp carries on from there. Each warp is a pipeline of its own: lane 0 keeps a ring of TMA
//     box loads in flight (16 rows x 256 bytes of packed quants, 128B-swizzled, plus the rows' f16
//     scales of the same K range; completion on the stage's mbarrier), so the bytes in flight per SM are
//     set by the rings (about 130 KB), not by registers, and no warp waits for another. The pieces of a
//     tile that was cut are added up by whichever warp brings the last one, in K order (no atomics on
//     the values: repeated runs are bit-identical);
//   * lane (g, t) reads 16 bytes of two rows and unpacks them into A fragments of
//     mma.sync.m16n8k16 (fp16 in, f32 accumulate). The quants are small integers, exact in fp16;
//   * x is split once per CTA into two fp16 terms, hi = fp16(x), lo = fp16(x - hi) (22 significant
//     bits together, the products are exact, sums are f32), and the eight B columns of the MMA are
//     used as (block, term) pairs: the four lanes t that share an A row hold different 32-blocks, so
//     column pair c only carries the x values of block c and zeros elsewhere. One accumulator tile
//     then holds the separate partial sums of four blocks, which the lane that owns the column pair
//     multiplies by its block's f16 scale in f32 - the per-block scale is applied to an f32 partial
//     sum exactly as the reference applies it.
//
// Every wait is bounded; a wait that gives up raises the device status flag and its warp returns.
#include <cuda.h>

#include "common.cuh"
#include "ops.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int MAX_STAGES = 8;
constexpr int TILE_ROWS = 16;
constexpr int XR = 32;                           // elements of x one thread stages, at most
constexpr uint32_t HDR_BYTES = 2304;             // norm scratch, zero region, slice counters, barriers
constexpr uint32_t CNT_OFF = 640;                // uint32 [MAX_WARPS]: pieces of a cut tile that have arrived
constexpr int MAX_WARPS = 16;
constexpr uint32_t NORM_RED_OFF = 128;           // float [32]
constexpr uint32_t ZERO_OFF = 512;               // 128 zero bytes (the B operand of lanes whose column belongs to another block)
constexpr uint32_t BAR_OFF = 1024;               // uint64 [MAX_WARPS][MAX_STAGES]
constexpr uint32_t SMEM_LIMIT = 227 * 1024;

struct Plan {
  uint32_t grid, tile_base, tile_rem, n_stage_iters, n_stages, kpad, x_off_lo, xs_off, part_off, ring_off, sc_off, sc_stage;
  size_t smem;
};

// D = A B (+ C): m16n8k16, fp16 operands, f32 accumulate. Not volatile: the compiler may interleave the chains.
__device__ __forceinline__ void mma_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float gelu_f(float x) {
  const float K = 0.7978846f; // ferrum_ref/src/kernels/nn.rs:L12-L15
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int j) { return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w; }

// The integer formats go to the tensor cores without a subtraction. A code c in the low bits of an fp16 half is
// the subnormal c * 2^-24, exactly, and the MMA takes subnormals as they are, so a mask or a byte permute is the
// whole conversion. What that leaves out is the code's offset (Q8_0: the byte is biased to q + 128; Q4_0: the
// nibble is q + 8), and sum((c - o) x) = sum(c x) - o sum(x): the block's sum of x is the same for every
// row, is computed once while x is staged, and is taken off in f32 where the block's scale is applied.
//
// Four bytes of a byte-per-weight format as two fp16 pairs (exact): elements (0, 1) and (2, 3).
// Q8_0: (q + 128) * 2^-24 each; FP8: the value itself.
template <int KIND>
__device__ __forceinline__ void bytes4_to_h2(uint32_t w, uint32_t& p01, uint32_t& p23) {
  if (KIND == FC_Q8_0) {
    const uint32_t u = w ^ 0x80808080u; // int8 -> biased uint8
    p01 = __byte_perm(u, 0u, 0x4140);   // halves 0x00b0, 0x00b1
    p23 = __byte_perm(u, 0u, 0x4342);
  } else {
    p01 = fp8x2_to_f16x2<KIND>(w);
    p23 = fp8x2_to_f16x2<KIND>(w >> 16);
  }
}
// One word (eight weights) of a nibble format as four fp16 pairs in element order (exact).
// Q4_0: nibble position p holds element 2p in the low half-word and 2p + 1 in the high one (the upload's
// order); pairs (0,1) and (4,5) come out as n * 2^-24, pairs (2,3) and (6,7) as n * 2^-20 (the nibble one place
// up) - x is staged 16 times larger at the k slots of the former, so every product carries 2^-20.
// MXFP4: the values themselves.
template <int KIND>
__device__ __forceinline__ void nibbles8_to_h2(uint32_t w, uint32_t (&p)[4]) {
  if (KIND == FC_Q4_0) {
    const uint32_t w8 = w >> 8;
    p[0] = w & 0x000f000fu;
    p[1] = w & 0x00f000f0u;
    p[2] = w8 & 0x000f000fu;
    p[3] = w8 & 0x00f000f0u;
  } else {
    e2m1x8_to_f16x2(w, p);
  }
}

// Sum over the first 256 threads of the CTA, in the order the stand-alone norm kernels use (elementwise.cu: CTAs
// of 256 threads), so the fused prologue reproduces them bit for bit. Named barrier 1: only those threads call it.
__device__ __forceinline__ float norm_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  asm volatile("bar.sync 1, 256;" ::: "memory");
  if (lane == 0) red[warp] = v;
  asm volatile("bar.sync 1, 256;" ::: "memory");
  float t = lane < 8 ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// One element of x, already scaled into the fp16 range, as its two fp16 terms; `mul` is the slot's extra factor
// (16 or 1). Returns the value the two terms stand for, without that factor.
__device__ __forceinline__ float store_split(__half* xh, __half* xl, uint32_t i, float v, float mul) {
  v = fminf(fmaxf(v * mul, -65504.0f), 65504.0f); // (a non-finite x: saturate instead of spreading infinities)
  const __half h = __float2half_rn(v);
  const __half l = __float2half_rn(v - __half2float(h));
  xh[i] = h;
  xl[i] = l;
  return (__half2float(h) + __half2float(l)) * (1.0f / mul);
}

// NW warps per CTA; a stage is one TMA box of 16 rows x LINES 128-byte lines of packed quants.
template <int KIND, int NW, int LINES>
__global__ void __launch_bounds__(NW * 32, 1)
    qmatvec1_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s, const uint32_t k,
                    const uint32_t n, const float* __restrict__ x, float* y, const Epilogue ep, const Plan pl, int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle is a function of the absolute shared-memory address
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  constexpr bool BYTES = kind_byte_blocks(KIND);      // one byte per weight (else half a byte)
  constexpr int WARPS = NW, THREADS = NW * 32;
  static_assert(NW <= MAX_WARPS, "the piece counters are one per warp");
  constexpr uint32_t W_STAGE = TILE_ROWS * LINES * 128;
  constexpr uint32_t SC_PER_STAGE = (BYTES ? 4u : 8u) * LINES; // blocks of one row in a stage
  constexpr uint32_t SC_STAGE = TILE_ROWS * SC_PER_STAGE * 2;
  float* norm_red = reinterpret_cast<float*>(smem + NORM_RED_OFF);
  __half* xh = reinterpret_cast<__half*>(smem + HDR_BYTES);
  __half* xl = reinterpret_cast<__half*>(smem + pl.x_off_lo);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t S = pl.n_stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFF) + warp * MAX_STAGES;
  uint8_t* ring = smem + pl.ring_off + warp * S * W_STAGE;
  uint8_t* sc_ring = smem + pl.sc_off + warp * S * SC_STAGE;
  const uint32_t row_bytes = BYTES ? k : k / 2;
  // this CTA's tiles: tile_base each, one more for the first tile_rem CTAs
  const uint32_t t0 = blockIdx.x * pl.tile_base + min(blockIdx.x, pl.tile_rem);
  const uint32_t n_tiles = pl.tile_base + (blockIdx.x < pl.tile_rem ? 1u : 0u);
  // work units: unit u is stage iteration u % iters of tile t0 + u / iters. Warp w of the `weff` warps that work
  // takes units [U w / weff, U (w + 1) / weff): never empty, since weff <= U
  const uint32_t iters = pl.n_stage_iters;
  const uint32_t U = n_tiles * iters, weff = min((uint32_t)NW, U);
  auto begin_of = [&](uint32_t w) { return (uint32_t)((uint64_t)U * w / weff); };
  auto warp_of = [&](uint32_t u) { return (uint32_t)((((uint64_t)u + 1) * weff - 1) / U); }; // whose share holds unit u
  uint32_t* cnt = reinterpret_cast<uint32_t*>(smem + CNT_OFF);
  float* part = reinterpret_cast<float*>(smem + pl.part_off); // [2 * warps][16]: a warp's first and last piece

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmap_w);
    tc::prefetch_tmap(&tmap_s);
    for (int i = 0; i < MAX_WARPS; i++) cnt[i] = 0u;
  }
  if (lane == 0) {
    for (uint32_t s = 0; s < S; s++) tc::mbar_init(&full[s], 1);
    tc::fence_barrier_init();
  }
  if (threadIdx.x >= 32 && threadIdx.x < 64) reinterpret_cast<uint32_t*>(smem + ZERO_OFF)[lane] = 0u;
  __syncwarp();

  // Loads of (tile, stage iteration) pairs, in the order this warp will consume them.
  const uint32_t ring_u32 = tc::smem_u32(ring), sc_u32 = tc::smem_u32(sc_ring), full_u32 = tc::smem_u32(full);
  auto issue = [&](uint32_t tile, uint32_t si, uint32_t it) { // lane 0 only
    const uint32_t s = it % S;
    const uint32_t bar = full_u32 + s * 8;
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(bar), "r"(W_STAGE + SC_STAGE)
                 : "memory");
    // packed quants: 128-byte lines si * LINES .. of rows tile * 16 ..; a line past the row's end is zero-filled
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            ring_u32 + s * W_STAGE),
        "l"(&tmap_w), "r"(bar), "r"(0), "r"((int32_t)(si * LINES)), "r"((int32_t)(tile * TILE_ROWS))
        : "memory");
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     sc_u32 + s * SC_STAGE),
                 "l"(&tmap_s), "r"(bar), "r"((int32_t)(si * SC_PER_STAGE)), "r"((int32_t)(tile * TILE_ROWS))
                 : "memory");
  };

  // The prologue of the warp's ring goes out before x is staged: the weight stream starts at once.
  // (ahead_tl, ahead_si) is the next load to issue, ahead_it its running number, ahead_left the loads still to issue.
  const bool dead = *err_flag != 0; // an earlier launch gave up: do not wait again
  const bool works = (uint32_t)warp < weff;
  const uint32_t u_begin = works ? begin_of(warp) : 0u, u_end = works ? begin_of(warp + 1) : 0u;
  const uint32_t tl_first = u_begin / iters;
  uint32_t ahead_tl = tl_first, ahead_si = u_begin - tl_first * iters, ahead_it = 0, ahead_left = u_end - u_begin;
  auto run_ahead = [&](uint32_t it) { // lane 0: fill every slot whose previous use (iteration < it) is over
    while (ahead_it < it + S && ahead_left) {
      issue(t0 + ahead_tl, ahead_si, ahead_it);
      ahead_it++, ahead_left--;
      if (++ahead_si == iters) ahead_si = 0, ahead_tl++;
    }
  };
  if (lane == 0 && !dead) run_ahead(0);
  // The launch may overlap the end of the kernel before it in the stream (programmatic dependent launch): the
  // weights are never written by a kernel, so their stream could start above; x, y and the residual may be that
  // kernel's results and are touched only below this wait. The kernel after this one may begin its own prologue.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // x -> hi / lo fp16 terms in shared memory: the RMSNorm / LayerNorm of x first when the product is fed the raw
  // residual stream, then a power-of-two scale that brings max |x| into [1024, 2048) (both terms keep their
  // full precision however small x is, and 16 x still fits fp16), undone on the results.
  constexpr bool BIASED = KIND == FC_Q8_0 || KIND == FC_Q4_0;
  float* stat = norm_red + 32; // [0] 1/rms or 1/std, [1] mean, [2..] per-warp maxima
  float* xsum = reinterpret_cast<float*>(smem + pl.xs_off); // per block: -offset * sum of the staged x
  float* xf = reinterpret_cast<float*>(xh); // x as it is, over the place of the two terms, until they are written
  for (uint32_t i = threadIdx.x; i < k; i += THREADS) xf[i] = x[i];
  __syncthreads();
  if (ep.norm != NORM_NONE && threadIdx.x < 256) {
    // statistics by the first 256 threads, which sum in the order of the stand-alone norm kernels (256-thread CTAs)
    constexpr uint32_t NT = 256;
    if (ep.norm == NORM_RMS) {
      float ss = 0.0f;
      for (uint32_t i = threadIdx.x; i < k; i += NT) ss = fmaf(xf[i], xf[i], ss);
      ss = norm_sum(ss, norm_red);
      if (threadIdx.x == 0) stat[0] = 1.0f / sqrtf(ss / (float)k + ep.norm_eps), stat[1] = 0.0f;
    } else {
      float sm = 0.0f;
      for (uint32_t i = threadIdx.x; i < k; i += NT) sm += xf[i];
      const float mean = norm_sum(sm, norm_red) / (float)k;
      float vs = 0.0f;
      for (uint32_t i = threadIdx.x; i < k; i += NT) {
        const float dl = xf[i] - mean;
        vs = fmaf(dl, dl, vs);
      }
      const float var = norm_sum(vs, norm_red) / (float)k;
      if (threadIdx.x == 0) stat[0] = 1.0f / sqrtf(var + 1e-5f), stat[1] = mean;
    }
  }
  if (ep.norm != NORM_NONE) __syncthreads();
  const float n_inv = ep.norm != NORM_NONE ? stat[0] : 1.0f, n_mean = ep.norm != NORM_NONE ? stat[1] : 0.0f;
  // this thread's elements (threadIdx.x + j * THREADS) into registers, normalised; their largest magnitude
  float xr[XR];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < XR; j++) {
    if ((uint32_t)j * THREADS >= k) break;
    const uint32_t i = threadIdx.x + j * THREADS;
    float v = 0.0f;
    if (i < k)
      v = ep.norm == NORM_NONE  ? xf[i]
          : ep.norm == NORM_RMS ? xf[i] * n_inv * ep.norm_g[i]
                                : (xf[i] - n_mean) * n_inv * ep.norm_g[i] + ep.norm_b[i];
    xr[j] = v;
    amax = fmaxf(amax, fabsf(v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) stat[2 + warp] = amax;
  __syncthreads(); // (every thread holds its elements: the raw copy may be overwritten)
  amax = lane < WARPS ? stat[2 + lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // 2^e with amax * 2^e in [1024, 2048); the exponent field is clamped so that 2^e and 2^-e are normal floats
  uint32_t ex = (__float_as_uint(amax) >> 23) & 0xffu;
  ex = ex < 11u ? 11u : ex > 254u ? 254u : ex;
  const float x_scale = __uint_as_float((264u - ex) << 23), y_scale = __uint_as_float((ex - 10u) << 23);
  for (uint32_t i = k + threadIdx.x; i < pl.kpad; i += THREADS) xh[i] = xl[i] = __float2half_rn(0.0f);
#pragma unroll
  for (int j = 0; j < XR; j++) { // (k is whole 32-blocks: a warp's 32 elements are one block)
    if ((uint32_t)j * THREADS >= k) break;
    const uint32_t i = threadIdx.x + j * THREADS;
    if (i < k) {
      const float mul = (KIND == FC_Q4_0 && !(i & 2u)) ? 16.0f : 1.0f;
      float used = store_split(xh, xl, i, xr[j] * x_scale, mul);
      if (BIASED) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) used += __shfl_xor_sync(0xffffffffu, used, o);
        if (lane == 0) xsum[i >> 5] = used * (KIND == FC_Q8_0 ? -128.0f : -8.0f);
      }
    }
  }
  __syncthreads();
  if (dead) return;

  const int g = lane >> 2, t = lane & 3;
  // Fragment row g is tile row rho(g). A row's 128-byte lines sit at rho * LINES * 128 + c * 128; line
  // L = LINES * rho + c of the box has its 16-byte chunks XORed with L & 7 (the 128B swizzle). rho is chosen so
  // that the two rows a quarter-warp reads carry swizzle terms that differ in bit 2: their four chunks each then
  // fall into different halves of the banks (two lines per row: the low two bits of g swapped; four: g itself).
  const uint32_t rho = LINES == 2 ? ((uint32_t)(g & 4) | (((uint32_t)g & 1u) << 1) | (((uint32_t)g >> 1) & 1u)) : (uint32_t)g;
  constexpr uint32_t ROW8 = 8 * LINES * 128; // row rho + 8
  uint32_t w_off[LINES][2]; // [line c][step h of the line]: byte offset of this lane's 16 bytes of row rho in a stage
#pragma unroll
  for (int c = 0; c < LINES; c++)
#pragma unroll
    for (int h = 0; h < 2; h++)
      w_off[c][h] = rho * (LINES * 128) + c * 128 + ((((uint32_t)h * 4 + (uint32_t)t) ^ ((LINES * rho + c) & 7u)) * 16);
  const uint32_t sc_row = rho * SC_PER_STAGE * 2;
  // B operand: column g of the MMA is (block g >> 1 of the accumulator tile, term g & 1). A lane supplies the x
  // values of its own k slots only to the column pair of its block; for the other columns it reads zeros.
  //   byte formats: a step is 64 weights = two blocks, lanes t = 0, 1 hold the first; the two steps of a line share
  //     one accumulator tile, the first in columns 0..3, the second in columns 4..7
  //   nibble formats: a step is 128 weights = four blocks, lane t holds block t; columns 2t, 2t + 1
  const uint8_t* x_term = reinterpret_cast<const uint8_t*>((g & 1) ? xl : xh);
  const uint8_t* zero = smem + ZERO_OFF;
  const bool act0 = BYTES ? (g < 4 && (g >> 1) == (t >> 1)) : ((g >> 1) == t);
  const bool act1 = BYTES ? (g >= 4 && ((g - 4) >> 1) == (t >> 1)) : act0;
  constexpr uint32_t XSTEP = BYTES ? 128u : 256u; // bytes of one x term per step
  const uint8_t* x_lane = x_term + (BYTES ? t * 32u : t * 64u);
  // (lanes that read zeros read them from banks the x values of their quarter-warp do not use)
  const uint8_t* zero_lane = zero + (BYTES ? ((g & 2) ? 0u : 64u) : 32u);
  const uint8_t* bx_base[2] = {act0 ? x_lane : zero_lane, act1 ? x_lane : zero_lane};
  const uint32_t bx_mul[2] = {act0 ? 1u : 0u, act1 ? 1u : 0u};

  uint32_t it = 0;
  for (uint32_t u = u_begin; u < u_end;) { // one piece per pass: the units of this share that belong to one tile
    const uint32_t tl = u / iters, si_begin = u - tl * iters, tile = t0 + tl;
    const uint32_t si_end = min(iters, si_begin + (u_end - u));
    u += si_end - si_begin;
    float acc_g = 0.0f, acc_g8 = 0.0f;
    for (uint32_t si = si_begin; si < si_end; si++, it++) {
      if (lane == 0) run_ahead(it); // the slot of iteration it - 1 is free: every lane passed the __syncwarp below
      const uint32_t s = it % S;
      if (!tc::mbar_wait(&full[s], (it / S) & 1)) {
        if (lane == 0) *err_flag = 1;
        return;
      }
      const uint8_t* wst = ring + s * W_STAGE;
      const __half* sst = reinterpret_cast<const __half*>(sc_ring + s * SC_STAGE + sc_row);
      const uint32_t lines = min((uint32_t)LINES, (row_bytes - si * (LINES * 128)) / 128); // (a row may end inside the stage)
#pragma unroll
      for (int cp = 0; cp < LINES; cp += 2) { // two lines at a time
      if ((uint32_t)cp >= lines) break;
      if (BYTES) {
        // 16 MMAs in four chains [line][word parity]; the loads first, so that they are all in flight
        uint4 wa[2][2], wb[2][2], bx[2][2][2];
        float d_g[2], d_g8[2];
#pragma unroll
        for (int c = 0; c < 2; c++) {
          d_g[c] = block_scale_f32<KIND>(sst[4 * (cp + c) + t]);
          d_g8[c] = block_scale_f32<KIND>(sst[8 * SC_PER_STAGE + 4 * (cp + c) + t]);
#pragma unroll
          for (int h = 0; h < 2; h++) {
            wa[c][h] = *reinterpret_cast<const uint4*>(wst + w_off[cp + c][h]);
            wb[c][h] = *reinterpret_cast<const uint4*>(wst + ROW8 + w_off[cp + c][h]);
            const uint8_t* xo = bx_base[h] + bx_mul[h] * (((si * LINES + cp + c) * 2 + h) * XSTEP);
            bx[c][h][0] = *reinterpret_cast<const uint4*>(xo);
            bx[c][h][1] = *reinterpret_cast<const uint4*>(xo + 16);
          }
        }
        float cc[2][2][4];
#pragma unroll
        for (int jj = 0; jj < 2; jj++)
#pragma unroll
          for (int h = 0; h < 2; h++)
#pragma unroll
            for (int par = 0; par < 2; par++)
#pragma unroll
              for (int c = 0; c < 2; c++) {
                const int j = 2 * jj + par;
                uint32_t a0, a1, a2, a3;
                bytes4_to_h2<KIND>(word_of(wa[c][h], j), a0, a2);
                bytes4_to_h2<KIND>(word_of(wb[c][h], j), a1, a3);
                const uint4& bb = bx[c][h][j >> 1];
                const uint32_t b0 = (j & 1) ? bb.z : bb.x, b1 = (j & 1) ? bb.w : bb.y;
                if (jj == 0 && h == 0)
                  mma_zero(cc[c][par], a0, a1, a2, a3, b0, b1);
                else
                  mma_acc(cc[c][par], a0, a1, a2, a3, b0, b1);
              }
#pragma unroll
        for (int c = 0; c < 2; c++) {
          float v_g = (cc[c][0][0] + cc[c][1][0]) + (cc[c][0][1] + cc[c][1][1]);
          float v_g8 = (cc[c][0][2] + cc[c][1][2]) + (cc[c][0][3] + cc[c][1][3]);
          if (BIASED) { // products carry 2^-24; minus 128 times the block's sum of x
            const float off = xsum[(si * LINES + cp + c) * 4 + t];
            v_g = fmaf(v_g, 16777216.0f, off);
            v_g8 = fmaf(v_g8, 16777216.0f, off);
          }
          acc_g = fmaf(d_g[c], v_g, acc_g);
          acc_g8 = fmaf(d_g8[c], v_g8, acc_g8);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; c++) {
          if ((uint32_t)(cp + c) >= lines) break;
          // a line: two steps of four blocks, 16 MMAs in four chains [step][pair parity]
          uint4 wa[2], wb[2], bx[2][4];
          float d_g[2], d_g8[2];
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const uint32_t blk = (2 * (cp + c) + h) * 4 + t;
            d_g[h] = block_scale_f32<KIND>(sst[blk]);
            d_g8[h] = block_scale_f32<KIND>(sst[8 * SC_PER_STAGE + blk]);
            wa[h] = *reinterpret_cast<const uint4*>(wst + w_off[cp + c][h]);
            wb[h] = *reinterpret_cast<const uint4*>(wst + ROW8 + w_off[cp + c][h]);
            const uint8_t* xo = bx_base[0] + bx_mul[0] * (((si * LINES + cp + c) * 2 + h) * XSTEP);
#pragma unroll
            for (int j = 0; j < 4; j++) bx[h][j] = *reinterpret_cast<const uint4*>(xo + j * 16);
          }
          float cc[2][2][4];
#pragma unroll
          for (int j = 0; j < 4; j++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
              uint32_t pa[4], pb[4];
              nibbles8_to_h2<KIND>(word_of(wa[h], j), pa);
              nibbles8_to_h2<KIND>(word_of(wb[h], j), pb);
              if (j == 0) {
                mma_zero(cc[h][0], pa[0], pb[0], pa[1], pb[1], bx[h][j].x, bx[h][j].y);
                mma_zero(cc[h][1], pa[2], pb[2], pa[3], pb[3], bx[h][j].z, bx[h][j].w);
              } else {
                mma_acc(cc[h][0], pa[0], pb[0], pa[1], pb[1], bx[h][j].x, bx[h][j].y);
                mma_acc(cc[h][1], pa[2], pb[2], pa[3], pb[3], bx[h][j].z, bx[h][j].w);
              }
            }
#pragma unroll
          for (int h = 0; h < 2; h++) {
            float v_g = (cc[h][0][0] + cc[h][1][0]) + (cc[h][0][1] + cc[h][1][1]);
            float v_g8 = (cc[h][0][2] + cc[h][1][2]) + (cc[h][0][3] + cc[h][1][3]);
            if (BIASED) { // products carry 2^-20; minus 8 times the block's sum of x
              const float off = xsum[((si * LINES + cp + c) * 2 + h) * 4 + t];
              v_g = fmaf(v_g, 1048576.0f, off);
              v_g8 = fmaf(v_g8, 1048576.0f, off);
            }
            acc_g = fmaf(d_g[h], v_g, acc_g);
            acc_g8 = fmaf(d_g8[h], v_g8, acc_g8);
          }
        }
      }
      }
      __syncwarp(); // every lane is done with the stage before lane 0 refills its slot
    }
    // the item's 16 partial results: the four lanes t of a row
    acc_g += __shfl_xor_sync(0xffffffffu, acc_g, 1);
    acc_g += __shfl_xor_sync(0xffffffffu, acc_g, 2);
    acc_g8 += __shfl_xor_sync(0xffffffffu, acc_g8, 1);
    acc_g8 += __shfl_xor_sync(0xffffffffu, acc_g8, 2);
    auto finish = [&](uint32_t row, float v) {
      if (row >= n) return;
      v *= y_scale;
      if (ep.bias) v += ep.bias[row];
      if (ep.act == ACT_GELU) v = gelu_f(v);
      if (ep.resid) v = ep.resid[row] + v;
      y[row] = v;
    };
    if (si_begin == 0 && si_end == iters) { // the whole tile was this warp's
      if (t < 2) finish(tile * TILE_ROWS + rho + (t ? 8u : 0u), t ? acc_g8 : acc_g);
      continue;
    }
    // A cut tile: its pieces belong to the consecutive warps wa..wb. Each leaves its partial sums in a slot of its
    // own (a warp has at most two pieces of cut tiles: its first and its last) and counts itself in at wa's counter,
    // which no other tile uses; the warp that arrives last adds the pieces up in K order.
    const uint32_t wa = warp_of(tl * iters), wb = warp_of(tl * iters + iters - 1);
    float* mine = part + (2 * warp + (tl != tl_first ? 1 : 0)) * TILE_ROWS;
    if (t == 0) {
      mine[rho] = acc_g;
      mine[rho + 8] = acc_g8;
    }
    __syncwarp();
    uint32_t last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(&cnt[wa], 1u) == wb - wa ? 1u : 0u;
    }
    if (__shfl_sync(0xffffffffu, last, 0)) {
      __threadfence_block();
      if (lane < TILE_ROWS) {
        float v = 0.0f;
        for (uint32_t w2 = wa; w2 <= wb; w2++) {
          const uint32_t slot = 2 * w2 + (tl != begin_of(w2) / iters ? 1u : 0u);
          v += const_cast<const volatile float*>(part)[slot * TILE_ROWS + lane];
        }
        finish(tile * TILE_ROWS + lane, v);
      }
    }
  }
}

uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

template <int KIND>
struct Cfg { // warps per CTA and 128-byte lines of a row per stage
  static constexpr int NW = 16;
  static constexpr int LINES = 2;
};

bool make_plan(const FcDevice* dev, const QMat& w, Plan& p) {
  const bool bytes = kind_byte_blocks(w.kind);
  if (!(bytes || kind_nibble_blocks(w.kind))) return false;
  // the scale plane is a TMA tensor: its row pitch (k / 32 halves) must be whole 16 bytes
  if (w.k % 256 || w.n == 0 || w.k == 0) return false;
  if ((reinterpret_cast<uintptr_t>(w.qs) | reinterpret_cast<uintptr_t>(w.sc)) & 15) return false;
  const uint32_t nw = bytes ? Cfg<FC_Q8_0>::NW : Cfg<FC_Q4_0>::NW, lines = 2;
  if (w.k > (uint32_t)XR * nw * 32) return false; // x is staged through registers
  const uint32_t sms = (uint32_t)dev->prop.multiProcessorCount;
  const uint32_t tiles = (w.n + TILE_ROWS - 1) / TILE_ROWS;
  p.grid = tiles < sms ? tiles : sms;
  p.tile_base = tiles / p.grid;
  p.tile_rem = tiles % p.grid;
  const uint32_t row_bytes = bytes ? w.k : w.k / 2;
  const uint32_t w_stage = TILE_ROWS * lines * 128;
  p.sc_stage = TILE_ROWS * (bytes ? 4u : 8u) * lines * 2;
  p.n_stage_iters = (row_bytes + lines * 128 - 1) / (lines * 128);
  // (the kernel counts a CTA's work units, tiles x stage iterations, in 32 bits)
  if ((uint64_t)(p.tile_base + 1) * p.n_stage_iters >= (1ull << 31)) return false;
  p.kpad = p.n_stage_iters * lines * (bytes ? 128u : 256u); // x is zero past k where a stage reaches past the row
  p.x_off_lo = HDR_BYTES + 2 * p.kpad + 16;          // the lo term 16 bytes off the hi term's banks
  p.xs_off = align_up(p.x_off_lo + 2 * p.kpad, 16);  // per-block sums of x (those past k are never read)
  p.part_off = align_up(p.xs_off + p.kpad / 32 * 4, 16);
  p.ring_off = align_up(p.part_off + 2 * nw * TILE_ROWS * 4, 1024);
  const uint32_t per_stage = nw * (w_stage + p.sc_stage);
  if (p.ring_off + 2 * per_stage + 1024 > SMEM_LIMIT) return false;
  p.n_stages = (SMEM_LIMIT - 1024 - p.ring_off) / per_stage;
  if (p.n_stages > MAX_STAGES) p.n_stages = MAX_STAGES;
  p.sc_off = p.ring_off + nw * p.n_stages * w_stage;
  p.smem = (size_t)p.sc_off + (size_t)nw * p.n_stages * p.sc_stage + 1024; // (+ the alignment slack)
  return true;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int KIND, int NW, int LINES>
int launch_cfg(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep, const Plan& p) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const bool bytes = kind_byte_blocks(KIND);
  const uint32_t row_bytes = bytes ? w.k : w.k / 2;
  CUtensorMap tw, ts;
  {
    // [row][128-byte line][byte]: a box is LINES lines of 16 rows
    const cuuint64_t dims[3] = {128, row_bytes / 128, w.n};
    const cuuint64_t strides[2] = {128, row_bytes};
    const cuuint32_t box[3] = {128, LINES, TILE_ROWS};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult cr = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)w.qs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (weights) failed with %d", (int)cr);
  }
  {
    const uint32_t nb = w.k / QK;
    const cuuint64_t dims[2] = {nb, w.n};
    const cuuint64_t strides[1] = {(cuuint64_t)nb * 2};
    const cuuint32_t box[2] = {(bytes ? 4u : 8u) * LINES, TILE_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)w.sc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (scales) failed with %d", (int)cr);
  }
  auto kern = qmatvec1_kernel<KIND, NW, LINES>;
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.grid), cfg.blockDim = dim3(NW * 32), cfg.dynamicSmemBytes = p.smem, cfg.stream = dev->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; // see the kernel's griddepcontrol.wait
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at, cfg.numAttrs = 1;
  FC_LAUNCH(dev, "qmatvec1", cudaLaunchKernelEx(&cfg, kern, tw, ts, w.k, w.n, x, y, ep, p, dev->d_flag));
  return FC_OK;
}

template <int KIND>
int launch(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep, const Plan& p) {
  return launch_cfg<KIND, Cfg<KIND>::NW, Cfg<KIND>::LINES>(dev, w, x, y, ep, p);
}

} // namespace

bool qmatvec1_supports(const FcDevice* dev, const QMat& w) {
  Plan p;
  return make_plan(dev, w, p);
}

int k_qmatvec1(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep) {
  Plan p;
  if (!make_plan(dev, w, p)) return fc_fail(dev, FC_ERR_UNSUPPORTED, "the streamed one-row product does not take this matrix");
  switch (w.kind) {
    case FC_Q8_0: return launch<FC_Q8_0>(dev, w, x, y, ep, p);
    case FC_Q4_0: return launch<FC_Q4_0>(dev, w, x, y, ep, p);
    case FC_FP8_E4M3: return launch<FC_FP8_E4M3>(dev, w, x, y, ep, p);
    case FC_FP8_E5M2: return launch<FC_FP8_E5M2>(dev, w, x, y, ep, p);
    case FC_MXFP4: return launch<FC_MXFP4>(dev, w, x, y, ep, p);
  }
  return fc_fail(dev, FC_ERR_UNSUPPORTED, "the streamed one-row product does not take this format");
}
