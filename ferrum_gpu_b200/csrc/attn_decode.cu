// Decode attention, head_dim 64: one query row per stream against that stream's f32 K/V cache,
// split along the context so that every SM streams cache (flash-decoding).
//
// Grid (split, kv-head, row). A CTA of 4 warps owns a contiguous range of cached positions of one
// (stream, kv-head) and serves all G query heads that share the kv-head from one pass over K and V,
// so the cache - the dominant HBM traffic of batched decode - is read exactly once per step.
// A warp works on 4 positions at a time: 8 lanes per position, each lane holding 8 of the 64
// channels (two 16-byte loads of K, two of V; a position's 256-byte row is one coalesced segment).
// Scores are reduced over the 8 lanes with shuffles; the softmax is online with one rescale per
// block of 4 positions per lane group. Lane groups, warps and finally splits are merged with the
// usual (max, sum, weighted output) rule; with one split the CTA writes the result directly.
//
// The number of splits is fixed per batch width (a captured step can be replayed) and chosen so that
// all CTAs are resident at once: a second, partly filled wave costs more than longer ranges (64 streams
// x 2 kv-heads at 1550 positions: 2 splits 0.60 ms per step of 24 layers, 3 splits 0.70). The range
// of a split is not fixed: each row's current length is cut into equal parts, so the CTAs of a row
// carry the same load whatever the length. The merge launch writes f32 rows or, for a following
// 9..64-row tensor-core product, directly that product's two fp16 terms.
// Replaces attn_gqd_probs.wgsl + attn_gqd_pv.wgsl (ferrum_wgpu/src/ops/llama.rs:L150-L179).
#include "ops.cuh"

namespace {

constexpr int HD = 64;
constexpr int POS_PER_ITER = 64; // positions a CTA consumes per loop iteration (4 warps x 4 groups x 4)
constexpr size_t TILE_BYTES = (size_t)2 * 2 * POS_PER_ITER * HD * 4; // two stages of a K and a V tile

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Where the result goes: f32 rows [rows][heads * 64], or (xh set) the two fp16 terms of the same rows,
// saturated like the product's own split of x, in blocks of `mp` rows.
struct DecodeOut {
  float* out;
  __half *xh, *xl;
  uint32_t mp;
  __device__ __forceinline__ void put(size_t at, float v) const {
    if (xh) {
      v = fminf(fmaxf(v, -65504.0f), 65504.0f);
      const __half h = __float2half_rn(v);
      xh[at] = h;
      xl[at] = __float2half_rn(v - __half2float(h));
    } else {
      out[at] = v;
    }
  }
};

// partial layout per (row, kv-head, split): [G] max (log2 domain), [G] sum, [G][64] weighted output
template <int G>
__global__ void __launch_bounds__(128)
    attn_decode_split_kernel(const float* __restrict__ qkv, uint32_t q_stride, uint32_t heads, uint32_t kv_heads,
                             const int32_t* __restrict__ positions, const int32_t* __restrict__ streams, KvLayer kv,
                             uint32_t ctx, uint32_t n_splits, float* __restrict__ partial, DecodeOut dst, bool append) {
  __shared__ float sm_m[4][G], sm_l[4][G];
  __shared__ __align__(16) float sm_o[4][G][HD];
  const uint32_t split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;
  const uint32_t len = (uint32_t)positions[r] + 1;
  const uint32_t split_len = ((len + n_splits - 1) / n_splits + POS_PER_ITER - 1) / POS_PER_ITER * POS_PER_ITER;
  const uint32_t p0 = min(len, split * split_len), p1 = min(len, p0 + split_len);
  if (dst.xh && split == 0 && r + 1 == gridDim.z) // the padding rows of the product's n-block are zero
    for (uint32_t i = threadIdx.x; i < (dst.mp - gridDim.z) * G * HD; i += blockDim.x) {
      const size_t at = (size_t)(gridDim.z + i / (G * HD)) * heads * HD + (size_t)kvh * G * HD + i % (G * HD);
      dst.xh[at] = dst.xl[at] = __float2half_rn(0.0f);
    }
  const uint32_t slot = streams ? (uint32_t)streams[r] : 0;

  // this lane's 8 channels of each query head, pre-scaled by log2(e) / sqrt(64): scores live in the
  // log2 domain so the exponentials are single ex2 instructions
  float q[G][8];
  const float qs = 0.125f * 1.4426950408889634f;
#pragma unroll
  for (int g = 0; g < G; g++) {
    const float* qp = qkv + (size_t)r * q_stride + (size_t)(kvh * G + g) * HD + sub * 8;
    const float4 a = *reinterpret_cast<const float4*>(qp), b = *reinterpret_cast<const float4*>(qp + 4);
    q[g][0] = a.x * qs, q[g][1] = a.y * qs, q[g][2] = a.z * qs, q[g][3] = a.w * qs;
    q[g][4] = b.x * qs, q[g][5] = b.y * qs, q[g][6] = b.z * qs, q[g][7] = b.w * qs;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; g++) {
    m[g] = -INFINITY, l[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) acc[g][i] = 0.0f;
  }

  // K and V tiles of 64 positions travel through two shared-memory stages by cp.async: the loads of the next
  // tile are in flight while this one is multiplied (with two 242-register CTAs per SM, loads held in
  // registers left the kernel waiting on memory latency). A position's row is 16 chunks of 16 bytes; a lane
  // reads chunks 2 * sub and 2 * sub + 1, the upper four lanes of a group in the opposite order, which keeps
  // the eight lanes of one position on 32 different banks.
  extern __shared__ __align__(16) float tiles[]; // [2 stages][K, V][64 positions][64]
  constexpr uint32_t TILE = POS_PER_ITER * HD;
  const float* krow_new = qkv + (size_t)r * q_stride + (size_t)(heads + kvh) * HD;
  const float* vrow_new = qkv + (size_t)r * q_stride + (size_t)(heads + kv_heads + kvh) * HD;
  const float* kcache = kv.k + ((size_t)slot * kv_heads + kvh) * ctx * HD;
  const float* vcache = kv.v + ((size_t)slot * kv_heads + kvh) * ctx * HD;
  if (append && p0 < len && p1 == len) {
    // the row's own k and v (models without RoPE) are not in the cache yet: this CTA's range ends with them,
    // so it stores them; the tiles below take that position from the qkv row
    float* kc = kv.k + (((size_t)slot * kv_heads + kvh) * ctx + (len - 1)) * HD;
    float* vc = kv.v + (((size_t)slot * kv_heads + kvh) * ctx + (len - 1)) * HD;
    if (threadIdx.x < HD) kc[threadIdx.x] = krow_new[threadIdx.x];
    else vc[threadIdx.x - HD] = vrow_new[threadIdx.x - HD];
  }
  auto stage = [&](uint32_t j0, uint32_t buf) {
#pragma unroll
    for (int c = 0; c < 16; c++) { // 2 tensors x 64 positions x 16 chunks over 128 threads
      const uint32_t id = threadIdx.x + 128 * c, tensor = id >> 10, pos = (id >> 4) & 63, ch = id & 15;
      const uint32_t j = j0 + pos;
      const uint32_t jj = j < p1 ? j : p0; // past the range: any valid row (its scores are masked)
      const bool fresh = append && jj + 1 == len;
      const float* src = tensor ? (fresh ? vrow_new : vcache + (size_t)jj * HD) : (fresh ? krow_new : kcache + (size_t)jj * HD);
      const uint32_t dst_addr = (uint32_t)__cvta_generic_to_shared(tiles + (buf * 2 + tensor) * TILE + pos * HD + ch * 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_addr), "l"(src + ch * 4) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int c_first = 2 * sub + (sub >> 2), c_second = 2 * sub + 1 - (sub >> 2);
  if (p0 < p1) stage(p0, 0);
  uint32_t buf = 0;
  for (uint32_t j0 = p0; j0 < p1; j0 += POS_PER_ITER, buf ^= 1) {
    if (j0 + POS_PER_ITER < p1) {
      stage(j0 + POS_PER_ITER, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* kt = tiles + (buf * 2) * TILE;
    const float* vt = kt + TILE;
    // this lane group's 4 positions of the iteration
    float s[4][G];
    float4 vv[4][2];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t pl = warp * 16 + i * 4 + grp;
      const bool ok = j0 + pl < p1;
      const float4 ka = *reinterpret_cast<const float4*>(kt + pl * HD + c_first * 4);
      const float4 kb = *reinterpret_cast<const float4*>(kt + pl * HD + c_second * 4);
      const float4 va = *reinterpret_cast<const float4*>(vt + pl * HD + c_first * 4);
      const float4 vb = *reinterpret_cast<const float4*>(vt + pl * HD + c_second * 4);
      const bool swap = sub >= 4; // the upper lanes fetched their second chunk first
      const float4 k0 = swap ? kb : ka, k1 = swap ? ka : kb;
      vv[i][0] = swap ? vb : va;
      vv[i][1] = swap ? va : vb;
#pragma unroll
      for (int g = 0; g < G; g++) {
        float d = q[g][0] * k0.x;
        d = fmaf(q[g][1], k0.y, d), d = fmaf(q[g][2], k0.z, d), d = fmaf(q[g][3], k0.w, d);
        d = fmaf(q[g][4], k1.x, d), d = fmaf(q[g][5], k1.y, d), d = fmaf(q[g][6], k1.z, d), d = fmaf(q[g][7], k1.w, d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        s[i][g] = ok ? d : -INFINITY;
      }
    }
    __syncthreads(); // (registers hold what this iteration needs: the stage may be refilled)
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float bm = fmaxf(fmaxf(s[0][g], s[1][g]), fmaxf(s[2][g], s[3][g]));
      const float mn = fmaxf(m[g], bm);
      if (mn == -INFINITY) continue; // nothing valid yet for this group
      const float corr = ex2(m[g] - mn);
      m[g] = mn;
      float p[4];
#pragma unroll
      for (int i = 0; i < 4; i++) p[i] = ex2(s[i][g] - mn);
      l[g] = fmaf(l[g], corr, (p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
      for (int c = 0; c < 8; c++) {
        float a = acc[g][c] * corr;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float v = c < 4 ? (&vv[i][0].x)[c] : (&vv[i][1].x)[c - 4];
          a = fmaf(p[i], v, a);
        }
        acc[g][c] = a;
      }
    }
  }

  // merge the 4 lane groups of the warp (lanes with equal `sub`)
#pragma unroll
  for (int g = 0; g < G; g++) {
    float mm = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], 8));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
    const float sc = m[g] == -INFINITY ? 0.0f : ex2(m[g] - mm);
    float ll = l[g] * sc;
    ll += __shfl_xor_sync(0xffffffffu, ll, 8);
    ll += __shfl_xor_sync(0xffffffffu, ll, 16);
#pragma unroll
    for (int c = 0; c < 8; c++) {
      float a = acc[g][c] * sc;
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      acc[g][c] = a;
    }
    m[g] = mm, l[g] = ll;
    if (grp == 0) {
      if (sub == 0) sm_m[warp][g] = mm, sm_l[warp][g] = ll;
#pragma unroll
      for (int c = 0; c < 8; c++) sm_o[warp][g][sub * 8 + c] = acc[g][c];
    }
  }
  __syncthreads();
  // merge the 4 warps: thread t handles channel t % 64 of heads g = t / 64, t / 64 + 2, ...
  for (int g = threadIdx.x / HD; g < G; g += 2) {
    const int c = threadIdx.x % HD;
    float mm = fmaxf(fmaxf(sm_m[0][g], sm_m[1][g]), fmaxf(sm_m[2][g], sm_m[3][g]));
    float ll = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float sc = sm_m[w][g] == -INFINITY ? 0.0f : ex2(sm_m[w][g] - mm);
      ll = fmaf(sm_l[w][g], sc, ll);
      o = fmaf(sm_o[w][g][c], sc, o);
    }
    if (n_splits == 1) {
      dst.put((size_t)r * heads * HD + (size_t)(kvh * G + g) * HD + c, o / ll);
    } else {
      float* p = partial + (((size_t)r * kv_heads + kvh) * n_splits + split) * (size_t)(G * (2 + HD));
      if (c == 0) p[g] = mm, p[G + g] = ll;
      p[2 * G + g * HD + c] = o;
    }
  }
}

// out[row][head][c] = merge over splits, ascending
template <int G>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial, uint32_t heads, uint32_t kv_heads,
                                         uint32_t n_splits, DecodeOut dst) {
  const uint32_t kvh = blockIdx.x, r = blockIdx.y;
  const float* base = partial + ((size_t)r * kv_heads + kvh) * n_splits * (size_t)(G * (2 + HD));
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, c = idx % HD;
    float mm = -INFINITY;
    for (uint32_t s = 0; s < n_splits; s++) mm = fmaxf(mm, base[(size_t)s * G * (2 + HD) + g]);
    float ll = 0.0f, o = 0.0f;
    for (uint32_t s = 0; s < n_splits; s++) {
      const float* p = base + (size_t)s * G * (2 + HD);
      const float sc = p[g] == -INFINITY ? 0.0f : ex2(p[g] - mm);
      ll = fmaf(p[G + g], sc, ll);
      o = fmaf(p[2 * G + g * HD + c], sc, o);
    }
    dst.put((size_t)r * heads * HD + (size_t)(kvh * G + g) * HD + c, o / ll);
  }
}

template <int G>
int launch(FcDevice* dev, const float* qkv, uint32_t q_stride, uint32_t rows, uint32_t heads, uint32_t kv_heads,
           const int32_t* positions, const int32_t* streams, const KvLayer& kv, uint32_t ctx, uint32_t n_splits,
           float* scratch, const DecodeOut& dst, bool append) {
  dim3 grid(n_splits, kv_heads, rows);
  static OncePerDevice attr;
  if (attr.first(dev->ordinal))
    FC_CUDA(dev, cudaFuncSetAttribute(attn_decode_split_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILE_BYTES));
  FC_LAUNCH(dev, "attn_decode",
            attn_decode_split_kernel<G><<<grid, 128, TILE_BYTES, dev->stream>>>(qkv, q_stride, heads, kv_heads, positions, streams, kv, ctx,
                                                                       n_splits, scratch, dst, append));
  if (n_splits > 1) {
    dim3 mg(kv_heads, rows);
    FC_LAUNCH(dev, "attn_decode_merge",
              attn_decode_merge_kernel<G><<<mg, 128, 0, dev->stream>>>(scratch, heads, kv_heads, n_splits, dst));
  }
  return FC_OK;
}

} // namespace

// CTAs of the split kernel one SM holds (registers bound it: 2 at 8 heads per kv-head, more below).
template <int G>
static int resident_ctas() {
  static int n = 0;
  if (!n && (cudaFuncSetAttribute(attn_decode_split_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILE_BYTES) !=
                 cudaSuccess ||
             cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_split_kernel<G>, 128, TILE_BYTES) != cudaSuccess)) {
    cudaGetLastError();
    n = 2;
  }
  return n < 1 ? 1 : n;
}

// How many ways the context is cut for `rows` streams: the most that keeps every CTA resident at
// once, no range shorter than 64 positions of a full cache. It depends only on (rows, ctx), never on
// the current positions, so a captured decode step can be replayed.
static uint32_t attn_decode_splits(const FcDevice* dev, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t ctx) {
  int per_sm = 2;
  switch (heads / kv_heads) {
    case 1: per_sm = resident_ctas<1>(); break;
    case 2: per_sm = resident_ctas<2>(); break;
    case 3: per_sm = resident_ctas<3>(); break;
    case 4: per_sm = resident_ctas<4>(); break;
    case 6: per_sm = resident_ctas<6>(); break;
    case 8: per_sm = resident_ctas<8>(); break;
  }
  const uint32_t slots = (uint32_t)per_sm * (uint32_t)dev->prop.multiProcessorCount;
  uint32_t s = slots / (rows * kv_heads);
  const uint32_t max_s = (ctx + POS_PER_ITER - 1) / POS_PER_ITER;
  if (s > max_s) s = max_s;
  if (ctx <= 512) s = 1; // a short cache is a microsecond for one CTA: the merge launch would cost more
  return s < 1 ? 1 : s;
}

// Partial results of every split.
size_t attn_decode_scratch_bytes(const FcDevice* dev, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t ctx) {
  const uint32_t ns = attn_decode_splits(dev, rows, heads, kv_heads, ctx);
  return (size_t)rows * kv_heads * ns * (heads / kv_heads) * (2 + HD) * 4 + 256;
}

bool attn_decode_split_supports(uint32_t heads, uint32_t kv_heads, uint32_t hd) {
  const uint32_t G = heads / kv_heads;
  return hd == HD && (G == 1 || G == 2 || G == 3 || G == 4 || G == 6 || G == 8);
}

int k_attn_decode_split(FcDevice* dev, const float* qkv, uint32_t q_stride, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                        const int32_t* positions, const int32_t* streams, const KvLayer& kv, uint32_t ctx, float* scratch,
                        float* out, __half* xh, __half* xl, uint32_t mp, bool append) {
  if (!rows) return FC_OK;
  const uint32_t ns = attn_decode_splits(dev, rows, heads, kv_heads, ctx);
  DecodeOut dst;
  dst.out = out, dst.xh = xh, dst.xl = xl, dst.mp = mp;
  switch (heads / kv_heads) {
    case 1: return launch<1>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
    case 2: return launch<2>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
    case 3: return launch<3>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
    case 4: return launch<4>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
    case 6: return launch<6>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
    case 8: return launch<8>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append);
  }
  return fc_fail(dev, FC_ERR_UNSUPPORTED, "split decode attention: group size %u", heads / kv_heads);
}
