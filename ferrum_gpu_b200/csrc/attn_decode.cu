// Decode attention, head_dim 64: one query row per stream against that stream's f32 K/V cache,
// split along the context so that every SM streams cache (flash-decoding).
//
// Grid (split, kv-head, row). A CTA of 4 warps owns a contiguous range of cached positions of one
// (stream, kv-head) and serves all G query heads that share the kv-head from one pass over K and V,
// so the cache - the dominant HBM traffic of batched decode - is read exactly once per step.
// A warp works on 4 positions at a time: 8 lanes per position, which divide the position's 64 channels and
// the G query heads among them and read the K and V rows from a tile staged in shared memory. The softmax is online with one rescale per
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
// NW warps per CTA (4, or 8 for the one-CTA-per-(row, kv-head) form that needs no merge launch): a CTA consumes
// NW x 16 positions per loop iteration (4 lane groups x 4 positions per warp)
template <int NW>
struct Tile {
  static constexpr int POS = NW * 16;
  static constexpr size_t BYTES = (size_t)2 * 2 * POS * HD * 4; // two stages of a K and a V tile
};
constexpr int POS_PER_ITER = Tile<4>::POS;

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

// What the launch does to the fused qkv row before it attends, when the RoPE / cache launch is folded into it
// (`on`): finish the qkv product's pending split-K sum and bias exactly as its own reduce would (ascending split
// order), rotate q and k, and write the slice back; the row's k and v then reach the cache through the append path.
struct QkvFinish {
  bool on = false;
  DeferredReduce pend; // splits == 0: the row is already summed
  RopeParams rope;
};

// partial layout per (row, kv-head, split): [G] max (log2 domain), [G] sum, [G][64] weighted output
template <int G, int NW>
__global__ void __launch_bounds__(NW * 32)
    attn_decode_split_kernel(const float* qkv, uint32_t q_stride, uint32_t heads, uint32_t kv_heads,
                             const int32_t* __restrict__ positions, const int32_t* __restrict__ streams, KvLayer kv,
                             uint32_t ctx, uint32_t n_splits, float* __restrict__ partial, DecodeOut dst, bool append, QkvFinish fin) {
  constexpr int POS_PER_ITER = Tile<NW>::POS; // (this kernel's own step; the host's split rule keeps the 4-warp one)
  __shared__ float sm_m[NW][G], sm_l[NW][G];
  __shared__ __align__(16) float sm_o[NW][G][HD];
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
  if (fin.on) {
    // This CTA's slice of the row: its G query heads, its k head and its v head (every split of the same
    // (row, kv-head) computes and writes the same values).
    __shared__ float slice[(G + 2) * HD];
    const uint32_t qd = heads * HD, kvd = kv_heads * HD, w = qd + 2 * kvd;
    float* grow = const_cast<float*>(qkv) + (size_t)r * q_stride;
    auto col_of = [&](uint32_t idx) {
      const uint32_t hs = idx / HD, e = idx % HD;
      return hs < (uint32_t)G ? (kvh * G + hs) * HD + e : hs == (uint32_t)G ? qd + kvh * HD + e : qd + kvd + kvh * HD + e;
    };
    for (uint32_t idx = threadIdx.x; idx < (G + 2) * HD; idx += blockDim.x) {
      const uint32_t col = col_of(idx);
      float v;
      if (fin.pend.splits) {
        v = 0.0f;
        const float* p = fin.pend.partial + (size_t)r * w + col;
        for (uint32_t sp = 0; sp < fin.pend.splits; sp++) v += p[(size_t)sp * fin.pend.m * w];
        if (fin.pend.bias) v += fin.pend.bias[col];
      } else {
        v = grow[col]; // (host code folds the launch only with a pending sum: see attn_decode_folds_rope)
      }
      slice[idx] = v;
    }
    __syncthreads();
    if (fin.rope.cos) { // the q heads and the k head: pairs (2p, 2p + 1) or (p, p + half) of the first rope_dim channels
      const uint32_t half = fin.rope.rope_dim / 2, pos = (uint32_t)positions[r];
      const float* cs = fin.rope.cos + (size_t)pos * half;
      const float* sn = fin.rope.sin + (size_t)pos * half;
      for (uint32_t i = threadIdx.x; i < (G + 1) * half; i += blockDim.x) {
        const uint32_t h = i / half, pp = i % half;
        float* base = slice + h * HD;
        const uint32_t ia = fin.rope.type == FC_ROPE_NORM ? 2 * pp : pp, ib = fin.rope.type == FC_ROPE_NORM ? 2 * pp + 1 : pp + half;
        const float c = cs[pp], sv = sn[pp], a = base[ia], b = base[ib];
        base[ia] = a * c - b * sv;
        base[ib] = a * sv + b * c;
      }
      __syncthreads();
    }
    for (uint32_t idx = threadIdx.x; idx < (G + 2) * HD; idx += blockDim.x) grow[col_of(idx)] = slice[idx];
    __threadfence(); // (the tiles below fetch the row's k and v with cp.async, past this SM's L1)
    __syncthreads();
  }

  // The 8 lanes of a lane group share one cached position and divide it two ways: CP lanes split the 64
  // channels (CH each), 8 / CP groups of lanes split the G query heads (HL each). More head groups mean fewer
  // shuffles per score and fewer softmax updates per lane, more channel parts mean fewer shared-memory reads
  // (every lane of a head group reads its CH channels of the K and V row): 8 heads run as 2 head groups x 4
  // channel parts (one lane per head, each reading whole rows, was bound by those reads; one head group, each
  // lane holding 8 channels for all 8 heads, by shuffles and eight softmax updates per lane). q is pre-scaled
  // by log2(e) / sqrt(64): scores live in the log2 domain so the exponentials are single ex2 instructions.
  constexpr int CP = (G == 1 || G == 3) ? 8 : 4;
  constexpr int HGROUPS = 8 / CP, HL = G / HGROUPS, CH = HD / CP;
  static_assert(HL * HGROUPS == G, "the head groups divide the heads");
  const int part = sub % CP, h0 = (sub / CP) * HL;
  // The CP lanes of a head group read their 16-byte chunks of a row at the same time, CH * 4 bytes apart: that
  // is 2 lanes per bank. The upper half of the lanes therefore walks its chunks rotated by one (register slot
  // c4 holds chunk (c4 + rot) % NCH, for q, K, V and the output alike), which spreads the 8 lanes of a
  // position over all 32 banks.
  constexpr int NCH = CH / 4;
  const int rot = part >= CP / 2 ? 1 : 0;
  float q[HL][CH];
  const float qs = 0.125f * 1.4426950408889634f;
#pragma unroll
  for (int h = 0; h < HL; h++) {
    const float* qp = qkv + (size_t)r * q_stride + (size_t)(kvh * G + h0 + h) * HD + part * CH;
#pragma unroll
    for (int c = 0; c < CH; c += 4) {
      const float4 a = *reinterpret_cast<const float4*>(qp + ((c / 4 + rot) & (NCH - 1)) * 4);
      q[h][c] = a.x * qs, q[h][c + 1] = a.y * qs, q[h][c + 2] = a.z * qs, q[h][c + 3] = a.w * qs;
    }
  }
  float m[HL], l[HL], acc[HL][CH];
#pragma unroll
  for (int h = 0; h < HL; h++) {
    m[h] = -INFINITY, l[h] = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; c++) acc[h][c] = 0.0f;
  }

  // K and V tiles of 64 positions travel through two shared-memory stages by cp.async: the loads of the next
  // tile are in flight while this one is multiplied, and the lanes of a group can all read the same row
  // (a shared-memory broadcast) instead of each holding a slice of it in registers.
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
    else if (threadIdx.x < 2 * HD) vc[threadIdx.x - HD] = vrow_new[threadIdx.x - HD];
  }
  auto stage = [&](uint32_t j0, uint32_t buf) {
#pragma unroll
    for (int c = 0; c < 16; c++) { // 2 tensors x POS positions x 16 chunks over NW x 32 threads
      const uint32_t id = threadIdx.x + NW * 32 * c, tensor = id / (POS_PER_ITER * 16), pos = (id >> 4) % POS_PER_ITER, ch = id & 15;
      const uint32_t j = j0 + pos;
      const uint32_t jj = j < p1 ? j : p0; // past the range: any valid row (its scores are masked)
      const bool fresh = append && jj + 1 == len;
      const float* src = tensor ? (fresh ? vrow_new : vcache + (size_t)jj * HD) : (fresh ? krow_new : kcache + (size_t)jj * HD);
      const uint32_t dst_addr = (uint32_t)__cvta_generic_to_shared(tiles + (buf * 2 + tensor) * TILE + pos * HD + ch * 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_addr), "l"(src + ch * 4) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
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
    const float* kt = tiles + (buf * 2) * TILE + part * CH;
    const float* vt = kt + TILE;
    // this lane group's 4 positions of the iteration
    float s[4][HL];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t pl = warp * 16 + i * 4 + grp;
      float k[CH];
#pragma unroll
      for (int c = 0; c < CH; c += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(kt + pl * HD + ((c / 4 + rot) & (NCH - 1)) * 4);
        k[c] = kk.x, k[c + 1] = kk.y, k[c + 2] = kk.z, k[c + 3] = kk.w;
      }
      const bool ok = j0 + pl < p1;
#pragma unroll
      for (int h = 0; h < HL; h++) {
        float d = q[h][0] * k[0];
#pragma unroll
        for (int c = 1; c < CH; c++) d = fmaf(q[h][c], k[c], d);
#pragma unroll
        for (int o = 1; o < CP; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[i][h] = ok ? d : -INFINITY;
      }
    }
    float p[4][HL], corr[HL];
#pragma unroll
    for (int h = 0; h < HL; h++) {
      const float bm = fmaxf(fmaxf(s[0][h], s[1][h]), fmaxf(s[2][h], s[3][h]));
      const float mn = fmaxf(m[h], bm);
      if (mn == -INFINITY) { // nothing valid yet for this group: leave the state as it is
        corr[h] = 1.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) p[i][h] = 0.0f;
        continue;
      }
      corr[h] = ex2(m[h] - mn);
      m[h] = mn;
#pragma unroll
      for (int i = 0; i < 4; i++) p[i][h] = ex2(s[i][h] - mn);
      l[h] = fmaf(l[h], corr[h], (p[0][h] + p[1][h]) + (p[2][h] + p[3][h]));
    }
#pragma unroll
    for (int h = 0; h < HL; h++)
#pragma unroll
      for (int c = 0; c < CH; c++) acc[h][c] *= corr[h];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float* vr = vt + (warp * 16 + i * 4 + grp) * HD;
#pragma unroll
      for (int c = 0; c < CH; c += 4) {
        const float4 v = *reinterpret_cast<const float4*>(vr + ((c / 4 + rot) & (NCH - 1)) * 4);
#pragma unroll
        for (int h = 0; h < HL; h++) {
          acc[h][c] = fmaf(p[i][h], v.x, acc[h][c]);
          acc[h][c + 1] = fmaf(p[i][h], v.y, acc[h][c + 1]);
          acc[h][c + 2] = fmaf(p[i][h], v.z, acc[h][c + 2]);
          acc[h][c + 3] = fmaf(p[i][h], v.w, acc[h][c + 3]);
        }
      }
    }
    __syncthreads(); // the stage may be refilled
  }

  // merge the 4 lane groups of the warp (lanes with equal `sub`)
#pragma unroll
  for (int h = 0; h < HL; h++) {
    float mm = fmaxf(m[h], __shfl_xor_sync(0xffffffffu, m[h], 8));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
    const float sc = m[h] == -INFINITY ? 0.0f : ex2(m[h] - mm);
    float ll = l[h] * sc;
    ll += __shfl_xor_sync(0xffffffffu, ll, 8);
    ll += __shfl_xor_sync(0xffffffffu, ll, 16);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      float a = acc[h][c] * sc;
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      acc[h][c] = a;
    }
    if (grp == 0) {
      if (part == 0) sm_m[warp][h0 + h] = mm, sm_l[warp][h0 + h] = ll;
#pragma unroll
      for (int c = 0; c < CH; c++) sm_o[warp][h0 + h][part * CH + ((c / 4 + rot) & (NCH - 1)) * 4 + (c & 3)] = acc[h][c];
    }
  }
  __syncthreads();
  // merge the warps: thread t handles channel t % 64 of heads g = t / 64, t / 64 + NW / 2, ...
  for (int g = threadIdx.x / HD; g < G; g += NW / 2) {
    const int c = threadIdx.x % HD;
    float mm = sm_m[0][g];
#pragma unroll
    for (int w = 1; w < NW; w++) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; w++) {
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
           float* scratch, const DecodeOut& dst, bool append, const QkvFinish& fin) {
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(attn_decode_split_kernel<G, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile<4>::BYTES));
    FC_CUDA(dev, cudaFuncSetAttribute(attn_decode_split_kernel<G, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile<8>::BYTES));
  }
  // Two splits of four-warp CTAs, two CTAs per SM, and a merge launch - or, where every (row, kv-head) can have
  // an SM of its own, one eight-warp CTA over the whole context: the same eight warps per SM stream the same
  // positions, and the partial results and the merge launch (about 4 us of a 64-row step's layer) fall away.
  if (n_splits == 2 && rows * kv_heads <= (uint32_t)dev->prop.multiProcessorCount) {
    dim3 grid(1, kv_heads, rows);
    FC_LAUNCH(dev, "attn_decode",
              attn_decode_split_kernel<G, 8><<<grid, 256, Tile<8>::BYTES, dev->stream>>>(qkv, q_stride, heads, kv_heads, positions, streams,
                                                                                      kv, ctx, 1, scratch, dst, append, fin));
    return FC_OK;
  }
  dim3 grid(n_splits, kv_heads, rows);
  FC_LAUNCH(dev, "attn_decode",
            attn_decode_split_kernel<G, 4><<<grid, 128, Tile<4>::BYTES, dev->stream>>>(qkv, q_stride, heads, kv_heads, positions, streams, kv,
                                                                                    ctx, n_splits, scratch, dst, append, fin));
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
  if (!n && (cudaFuncSetAttribute(attn_decode_split_kernel<G, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile<4>::BYTES) !=
                 cudaSuccess ||
             cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_split_kernel<G, 4>, 128, Tile<4>::BYTES) != cudaSuccess)) {
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
                        float* out, __half* xh, __half* xl, uint32_t mp, bool append, const DeferredReduce* qkv_pending,
                        const RopeParams* rope) {
  if (!rows) return FC_OK;
  const uint32_t ns = attn_decode_splits(dev, rows, heads, kv_heads, ctx);
  DecodeOut dst;
  dst.out = out, dst.xh = xh, dst.xl = xl, dst.mp = mp;
  QkvFinish fin;
  if (rope) { // the RoPE / cache launch folded into this one (the caller passes append = true with it)
    fin.on = true;
    fin.rope = *rope;
    if (qkv_pending) fin.pend = *qkv_pending;
  }
  switch (heads / kv_heads) {
    case 1: return launch<1>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
    case 2: return launch<2>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
    case 3: return launch<3>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
    case 4: return launch<4>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
    case 6: return launch<6>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
    case 8: return launch<8>(dev, qkv, q_stride, rows, heads, kv_heads, positions, streams, kv, ctx, ns, scratch, dst, append, fin);
  }
  return fc_fail(dev, FC_ERR_UNSUPPORTED, "split decode attention: group size %u", heads / kv_heads);
}
