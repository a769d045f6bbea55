// Single-stream decode of a small GPT-2-style model as ONE kernel per run of tokens: the op order of
// GpuGpt2::feed (ferrum_wgpu/src/models/gpt2.rs:L192-L265: embed+pos -> LN -> q,k,v (+bias) -> cache ->
// attention -> wo (+bias) -> add -> LN -> w1 (+bias) -> gelu -> w2 (+bias) -> add; final LN -> head), with the
// greedy pick and the next token's embedding inside, so that a chain of greedy steps never leaves the device.
//
// Why: such a model's packed weights (11 MB for 6 layers of width 384) live in L2, and a token is 30-odd
// dependent matrix-vector stages of a few hundred kilobytes each. As separate launches every stage pays a
// launch and a drain (about 6 us each, 0.19 ms per token); the reference's own analysis of its per-command cost
// is docs/decode-crossover.md:L35. Here the stages of a token are separated by hardware barriers of one
// thread-block cluster instead:
//
//   * one cluster of 16 (or 8) CTAs; every CTA keeps the whole activation vectors of the token (residual
//     stream, q, FFN activations, attention partials) in its own shared memory;
//   * a stage splits the rows of its matrix over all warps of the cluster; a warp streams its rows from L2
//     (16-byte loads, the f32 dequantisation of the one-row matvec: exact products, f32 sums), and writes each
//     result into the shared memory of every CTA (distributed shared memory), so the next stage reads its
//     whole input locally;
//   * k and v go to the f32 cache in global memory; attention is split into (head, half of the positions) items
//     whose (max, sum, weighted v) partials are exchanged like any other result and merged by the consumer;
//   * barrier.cluster (arrive.release / wait.acquire) between stages: a hardware barrier, not a spin, so there
//     is no wait to bound; every CTA executes the same sequence of barriers whatever the data.
//
// LayerNorm statistics, the merge of the attention partials, the final pick and the next embedding are computed
// redundantly by every CTA (a few hundred flops) instead of being exchanged.
#include <cooperative_groups.h>

#include "model.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int DC_THREADS = 384;
constexpr int DC_WARPS = DC_THREADS / 32;
constexpr int DC_MAX_CLUSTER = 16;

struct DcMat {
  const uint8_t* qs;
  const __half* sc;
  const float* bias;
  uint32_t k, n;
  int kind;
};
struct DcLayer {
  const float *n1g, *n1b, *n2g, *n2b;
  DcMat qkv, wo, ff1, ff2;
  float *kc, *vc; // the layer's caches: [stream][heads][ctx][hd]
};
struct DcArgs {
  const DcLayer* layers;
  uint32_t n_layers, dim, heads, hd, hidden, vocab, ctx;
  const float *tok, *pos_table, *nfg, *nfb;
  DcMat head;
  float* logits;     // [vocab], global: the last step's row
  int32_t* d_ids;    // [1] token of the step (read when !chained; written back)
  int32_t* d_pos;    // [1] position of the step (read; written back)
  int32_t* d_argmax; // [1] pick (read when chained: the token of the first step; written)
  int32_t* log;      // tokens consumed by chained steps
  uint32_t* log_cnt; // [1]
  uint32_t steps;
  int chained;
  size_t kv_off; // the stream's offset into a layer's caches (floats)
  // shared-memory layout (floats): x | h | q | act | part | am | ln | layer descriptors
  uint32_t off_h, off_q, off_act, off_part, off_am, off_ln, off_desc, smem_floats;
};

__device__ __forceinline__ uint4 ldg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// sum over a 16-byte chunk of x[e] * q[e] (scale not applied); the bit tricks of the one-row matvec
template <int KIND>
__device__ __forceinline__ float dc_chunk_dot(const uint4& wq, const float* __restrict__ xs) {
  float acc = 0.0f;
  const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
  if (KIND == FC_Q8_0) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + 4 * w);
      const uint32_t u = words[w] ^ 0x80808080u;
      acc = fmaf(xv.x, __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f, acc);
      acc = fmaf(xv.y, __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f, acc);
      acc = fmaf(xv.z, __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f, acc);
      acc = fmaf(xv.w, __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f, acc);
    }
  } else { // FC_Q4_0: element j of a word at nibble position (j >> 1) + 4 (j & 1)
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float4 xa = *reinterpret_cast<const float4*>(xs + 8 * w);
      const float4 xb = *reinterpret_cast<const float4*>(xs + 8 * w + 4);
      const float xe[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int pos = (j >> 1) + 4 * (j & 1);
        const uint32_t nib = (words[w] >> (4 * pos)) & 0xfu;
        acc = fmaf(xe[j], __uint_as_float(0x4B000000u | nib) - 8388616.0f, acc);
      }
    }
  }
  return acc;
}

constexpr int DC_CH = 6; // 16-byte chunks per lane and batch
// lanes along K of a row: so that a row is one batch where it can be
__device__ __forceinline__ uint32_t dc_lpr(const DcMat& W) {
  const uint32_t per = (W.k / (W.kind == FC_Q8_0 ? 16u : 32u) + DC_CH - 1) / DC_CH;
  return per > 16 ? 32u : per > 8 ? 16u : per > 4 ? 8u : per > 2 ? 4u : 2u;
}
__device__ __forceinline__ void dc_load_batch(const DcMat& W, uint32_t rc, uint32_t c0, uint32_t lpr, uint32_t gl, uint32_t chunks,
                                              uint32_t nb, uint4 (&wq)[DC_CH], float (&d)[DC_CH]) {
#pragma unroll
  for (int j = 0; j < DC_CH; j++) {
    const uint32_t c = c0 + j * lpr;
    const bool in = c < chunks;
    const uint32_t cc = in ? c : gl;
    wq[j] = ldg16(W.qs + ((size_t)rc * chunks + cc) * 16);
    d[j] = in ? __half2float(W.sc[(size_t)rc * nb + (W.kind == FC_Q8_0 ? (cc >> 1) : cc)]) : 0.0f;
  }
}
// y[row] = x . W[row] for the rows of this warp: `lpr` lanes along K, 32 / lpr rows at a time. All 16-byte loads
// of a batch (DC_CH chunks per lane) are issued before the first is used: a stage then costs about one trip to L2,
// not one per chunk. `emit(row, value, i, n)` is called by the n lanes
// of the row's group, i = 0..n-1. One copy of this code serves every stage of the kernel (format and lane split
// are run-time values): the instruction cache, like everything else here, is re-used token after token.
template <typename Emit>
__device__ __forceinline__ void dc_rows(const DcMat& W, const float* __restrict__ xs, uint32_t gwarp, uint32_t n_gwarps,
                                        Emit&& emit) {
  const bool q8 = W.kind == FC_Q8_0;
  const uint32_t elems = q8 ? 16u : 32u, lpr = dc_lpr(W), rpt = 32 / lpr;
  const uint32_t lane = threadIdx.x & 31, gl = lane & (lpr - 1), g = lane / lpr;
  const uint32_t chunks = W.k / elems, nb = W.k / QK;
  const uint32_t tasks = (W.n + rpt - 1) / rpt;
  for (uint32_t task = gwarp; task < tasks; task += n_gwarps) {
    const uint32_t row = task * rpt + g, rc = min(row, W.n - 1);
    const float bias = W.bias ? W.bias[rc] : 0.0f; // (requested with the weights, used after them)
    float acc = 0.0f;
    for (uint32_t c0 = gl; c0 < chunks; c0 += DC_CH * lpr) {
      uint4 wq[DC_CH];
      float d[DC_CH];
      dc_load_batch(W, rc, c0, lpr, gl, chunks, nb, wq, d);
#pragma unroll
      for (int j = 0; j < DC_CH; j++) {
        const uint32_t c = min(c0 + j * lpr, chunks - 1); // (past the end: scale 0 times a finite sum)
        const float* xp = xs + (size_t)c * elems;
        acc = fmaf(d[j], q8 ? dc_chunk_dot<FC_Q8_0>(wq[j], xp) : dc_chunk_dot<FC_Q4_0>(wq[j], xp), acc);
      }
    }
    for (uint32_t o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    // every lane of the row's group holds the sum: they share the stores to the other CTAs
    if (row < W.n) emit(row, acc + bias, gl, lpr);
  }
}

// LayerNorm of x[0..d) into h (ferrum_ref/src/kernels/nn.rs:L31-L43: two-pass variance, eps 1e-5). Every warp
// computes the two statistics for itself with shuffles - d is a few hundred floats in shared memory - so the
// stage has one CTA barrier instead of five.
__device__ __forceinline__ void dc_layernorm(const float* x, const float* g, const float* b, uint32_t d, float* h) {
  const int lane = threadIdx.x & 31;
  float s = 0.0f;
  for (uint32_t i = lane; i < d; i += 32) s += x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s / (float)d;
  float vs = 0.0f;
  for (uint32_t i = lane; i < d; i += 32) {
    const float dl = x[i] - mean;
    vs = fmaf(dl, dl, vs);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) vs += __shfl_xor_sync(0xffffffffu, vs, o);
  const float is = 1.0f / sqrtf(vs / (float)d + 1e-5f);
  for (uint32_t i = threadIdx.x; i < d; i += DC_THREADS) h[i] = (x[i] - mean) * is * g[i] + b[i];
  __syncthreads();
}

__device__ __forceinline__ float dc_gelu(float x) {
  const float K = 0.7978846f; // ferrum_ref/src/kernels/nn.rs:L12-L15
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

__global__ void __launch_bounds__(DC_THREADS, 1) decode_cluster_kernel(const DcArgs a) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float wpart[DC_WARPS][66]; // per-warp attention partials of this CTA's item
  __shared__ float merged[66];          // and their merge, before it goes to every CTA
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t ncta = cluster.num_blocks(), cta = cluster.block_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // warps are numbered across the CTAs first: a stage with few row tasks then spreads them over all SMs
  const uint32_t gwarp = warp * ncta + cta, n_gwarps = ncta * DC_WARPS;
  float* x = sm;                 // residual stream [dim]
  float* h = sm + a.off_h;       // normed x / merged attention output [dim]
  float* q = sm + a.off_q;       // [dim]
  float* act = sm + a.off_act;   // [hidden]
  float* part = sm + a.off_part; // [items][66]: max, sum, weighted v[64]
  float* am = sm + a.off_am;     // [ncta][2]: best value, best index
  // the same arrays in every CTA of the cluster (distributed shared memory): a result goes to all of them
  const uint32_t sm_base = (uint32_t)__cvta_generic_to_shared(sm);
  // (caller i of n writes to CTAs i, i + n, ...: a remote store is slow to issue, so the callers share them)
  auto put_all = [&](uint32_t off, float v, uint32_t i, uint32_t n) {
    const uint32_t local = sm_base + off * 4;
    for (uint32_t r = i; r < ncta; r += n)
      asm volatile("{\n.reg .b32 ra;\nmapa.shared::cluster.u32 ra, %0, %1;\nst.shared::cluster.f32 [ra], %2;\n}" ::"r"(local), "r"(r),
                   "f"(v)
                   : "memory");
  };

  const uint32_t d = a.dim, hd = a.hd, heads = a.heads;
  const uint32_t parts = ncta / heads >= 1 ? ncta / heads : 1; // position parts per head
  const uint32_t items = heads * parts;                         // (items beyond ncta take a second round)
  const float scale = 1.0f / sqrtf((float)hd);

  // The layer descriptors into shared memory once: they are read at every stage, and from global memory each
  // read would be a trip to L2 in the stage's dependency chain (the barriers make the compiler read them again).
  DcLayer* layers = reinterpret_cast<DcLayer*>(sm + a.off_desc);
  for (uint32_t i = threadIdx.x; i < a.n_layers * (uint32_t)(sizeof(DcLayer) / 4); i += DC_THREADS)
    reinterpret_cast<uint32_t*>(layers)[i] = reinterpret_cast<const uint32_t*>(a.layers)[i];
  __syncthreads();
  // LayerNorm gains and shifts of every layer, and of the final norm, into shared memory once
  float* ln = sm + a.off_ln; // [(4 l + {n1g, n1b, n2g, n2b}) * dim], then the final gain and shift
  for (uint32_t l = 0; l < a.n_layers; l++)
    for (uint32_t i = threadIdx.x; i < d; i += DC_THREADS) {
      ln[(4 * l + 0) * d + i] = layers[l].n1g[i];
      ln[(4 * l + 1) * d + i] = layers[l].n1b[i];
      ln[(4 * l + 2) * d + i] = layers[l].n2g[i];
      ln[(4 * l + 3) * d + i] = layers[l].n2b[i];
    }
  for (uint32_t i = threadIdx.x; i < d; i += DC_THREADS) {
    ln[(4 * a.n_layers) * d + i] = a.nfg[i];
    ln[(4 * a.n_layers + 1) * d + i] = a.nfb[i];
  }
  cluster.sync(); // every CTA of the cluster is running before anyone writes into its shared memory
  int32_t token = a.chained ? a.d_argmax[0] : a.d_ids[0];
  uint32_t pos = (uint32_t)a.d_pos[0] + (a.chained ? 1u : 0u);
  const uint32_t log_base = a.chained ? a.log_cnt[0] : 0u;
  int32_t pick = 0;
  // A token is a flat sequence of stages, five per layer and the head, run by ONE copy of the code below (the
  // stage's kind picks its input, its matrix and what happens to a result): qkv | attention | wo | ff1 | ff2.
  enum { ST_QKV = 0, ST_ATTN = 1, ST_WO = 2, ST_FF1 = 3, ST_FF2 = 4, ST_HEAD = 5 };
  const uint32_t n_stages = 5 * a.n_layers + 1;
  auto stage_mat = [&](uint32_t sidx) -> const DcMat& { // the matrix of a stage (attention: the one after it)
    if (sidx >= 5 * a.n_layers) return a.head;
    const DcLayer& L = layers[sidx / 5];
    const uint32_t st = sidx % 5;
    return st == ST_QKV ? L.qkv : st <= ST_WO ? L.wo : st == ST_FF1 ? L.ff1 : L.ff2;
  };

  for (uint32_t step = 0; step < a.steps; step++, pos++) {
    // embedding + position row (ops::embed_at, ferrum_wgpu/src/ops/mod.rs:L189-L211), every CTA for itself
    if (a.chained && cta == 0 && threadIdx.x == 0) a.log[log_base + step] = token;
    for (uint32_t i = threadIdx.x; i < d; i += DC_THREADS)
      x[i] = a.tok[(size_t)token * d + i] + (a.pos_table ? a.pos_table[(size_t)pos * d + i] : 0.0f);
    __syncthreads();
    float best = -INFINITY; // the head stage's pick among this lane's rows: first maximum, NaN never wins
    int bi = 0x7fffffff;
    for (uint32_t sidx = 0; sidx < n_stages; sidx++) {
      const uint32_t l = sidx / 5, st = sidx < 5 * a.n_layers ? sidx % 5 : (uint32_t)ST_HEAD;
      const DcLayer& L = layers[min(l, a.n_layers - 1)];
      // ---- what the stage does before its product ----
      if (st == ST_QKV || st == ST_FF1 || st == ST_HEAD) {
        const uint32_t which = st == ST_HEAD ? 4 * a.n_layers : 4 * l + (st == ST_FF1 ? 2 : 0);
        dc_layernorm(x, ln + which * d, ln + (which + 1) * d, d, h);
      } else if (st == ST_ATTN) {
        // item (head, part) -> (max, sum exp, sum exp * v) over its positions
        const uint32_t len = pos + 1;
        for (uint32_t item = cta; item < items; item += ncta) {
          const uint32_t head = item / parts, pt = item % parts;
          const uint32_t p0 = (uint32_t)(((uint64_t)len * pt) / parts), p1 = (uint32_t)(((uint64_t)len * (pt + 1)) / parts);
          const float* kc = L.kc + a.kv_off + (size_t)head * a.ctx * hd;
          const float* vc = L.vc + a.kv_off + (size_t)head * a.ctx * hd;
          // a lane owns head dims 2 lane, 2 lane + 1 (hd = 64); a warp takes positions p0 + warp, + DC_WARPS, ...
          const float2 qv = *reinterpret_cast<const float2*>(q + head * hd + 2 * lane);
          float m = -INFINITY, s = 0.0f, o0 = 0.0f, o1 = 0.0f;
          for (uint32_t pb = p0 + warp; pb < p1; pb += 4 * DC_WARPS) { // four positions at a time: their loads go out together
            float2 kv[4], vv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t p = min(pb + j * DC_WARPS, p1 - 1);
              kv[j] = __ldcg(reinterpret_cast<const float2*>(kc + (size_t)p * hd + 2 * lane));
              vv[j] = __ldcg(reinterpret_cast<const float2*>(vc + (size_t)p * hd + 2 * lane));
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float dot = fmaf(qv.x, kv[j].x, qv.y * kv[j].y);
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
              if (pb + j * DC_WARPS < p1) { // (uniform across the warp)
                dot *= scale;
                const float mn = fmaxf(m, dot);
                const float corr = expf(m - mn), e = expf(dot - mn); // (m = -inf the first time: corr = 0)
                s = s * corr + e;
                o0 = o0 * corr + e * vv[j].x;
                o1 = o1 * corr + e * vv[j].y;
                m = mn;
              }
            }
          }
          if (lane == 0) wpart[warp][0] = m, wpart[warp][1] = s;
          wpart[warp][2 + 2 * lane] = o0;
          wpart[warp][3 + 2 * lane] = o1;
          __syncthreads();
          if (threadIdx.x < 64 + 2) {
            // merge the warps in order; threads 0..63: a dim of the weighted v, 64: the max, 65: the sum
            float M = -INFINITY;
            for (int w = 0; w < DC_WARPS; w++) M = fmaxf(M, wpart[w][0]);
            float out = 0.0f;
            if (threadIdx.x == 64) {
              out = M;
            } else {
              for (int w = 0; w < DC_WARPS; w++) {
                const float wm = wpart[w][0];
                const float f = wm == -INFINITY ? 0.0f : expf(wm - M);
                out += f * (threadIdx.x == 65 ? wpart[w][1] : wpart[w][2 + threadIdx.x]);
              }
            }
            const uint32_t slot = threadIdx.x == 64 ? 0 : threadIdx.x == 65 ? 1 : 2 + threadIdx.x;
            merged[slot] = out;
          }
          __syncthreads();
          for (uint32_t i = threadIdx.x; i < 66 * ncta; i += DC_THREADS) // 66 values to every CTA, shared by all threads
            put_all(a.off_part + item * 66 + i % 66, merged[i % 66], i / 66, ncta);
          __syncthreads();
        }
      } else if (st == ST_WO) {
        // merge the parts of every head into h (attend_row, ferrum_ref/src/models/llama/ops.rs:L143-L160)
        for (uint32_t i = threadIdx.x; i < d; i += DC_THREADS) {
          const uint32_t head = i / hd, c = i % hd;
          float M = -INFINITY;
          for (uint32_t pt = 0; pt < parts; pt++) M = fmaxf(M, part[(head * parts + pt) * 66]);
          float num = 0.0f, den = 0.0f;
          for (uint32_t pt = 0; pt < parts; pt++) {
            const float* pp = part + (head * parts + pt) * 66;
            const float f = pp[0] == -INFINITY ? 0.0f : expf(pp[0] - M);
            num += f * pp[2 + c];
            den += f * pp[1];
          }
          h[i] = num / den;
        }
        __syncthreads();
      }
      // ---- the stage's product; a result goes where the stage's kind says ----
      if (st != ST_ATTN) {
        const DcMat& W = stage_mat(sidx);
        dc_rows(W, st == ST_FF2 ? act : h, gwarp, n_gwarps, [&](uint32_t row, float v, uint32_t gi, uint32_t gn) {
          if (st == ST_QKV) {
            if (row < d) {
              put_all(a.off_q + row, v, gi, gn);
            } else if (gi == 0) { // k rows then v rows: the cache row of this position, [head][ctx][hd]
              const uint32_t r = row - d, which = r / d, c = r % d;
              float* dst = (which ? L.vc : L.kc) + a.kv_off;
              dst[((size_t)(c / hd) * a.ctx + pos) * hd + (c % hd)] = v;
            }
          } else if (st == ST_FF1) {
            put_all(a.off_act + row, dc_gelu(v), gi, gn);
          } else if (st == ST_HEAD) {
            if (gi == 0) {
              a.logits[row] = v;
              if (v > best || (v == best && (int)row < bi)) best = v, bi = (int)row;
            }
          } else { // wo, ff2: + residual, the new residual stream
            put_all(row, x[row] + v, gi, gn);
          }
        });
      }
      if (st == ST_HEAD) { // this CTA's pick to every CTA
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
        }
        if (lane == 0) wpart[warp][0] = best, wpart[warp][1] = __int_as_float(bi);
        __syncthreads();
        if (threadIdx.x == 0) {
          for (int w = 1; w < DC_WARPS; w++) {
            const float ov = wpart[w][0];
            const int oi = __float_as_int(wpart[w][1]);
            if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
          }
          merged[0] = best, merged[1] = __int_as_float(bi);
        }
        __syncthreads();
        if (threadIdx.x < 2 * ncta) put_all(a.off_am + 2 * cta + (threadIdx.x & 1), merged[threadIdx.x & 1], threadIdx.x >> 1, ncta);
      }
      // ---- the barrier (loading the next product's first weights between its arrive and its wait was measured
      // slower: 143 us per token against 120) ----
      cluster.sync();
    }
    {
      float bv = am[0];
      int bidx = __float_as_int(am[1]);
      for (uint32_t r = 1; r < ncta; r++) {
        const float ov = am[2 * r];
        const int oi = __float_as_int(am[2 * r + 1]);
        if (ov > bv || (ov == bv && oi < bidx)) bv = ov, bidx = oi;
      }
      pick = bidx == 0x7fffffff ? 0 : bidx;
    }
    if (step + 1 < a.steps) token = pick;
    // (`am` is rewritten only after this token's other barriers)
  }
  if (cta == 0 && threadIdx.x == 0) {
    a.d_argmax[0] = pick;
    a.d_ids[0] = token;
    a.d_pos[0] = (int32_t)(pos - 1);
    if (a.chained) a.log_cnt[0] = log_base + a.steps;
  }
}

struct DcState {
  DcLayer* d_layers = nullptr;
  int cluster = 0; // 0: not probed; -1: unavailable
  DcArgs args;
};

} // namespace

void decode_cluster_free(FcModel* m) {
  if (!m->dc) return;
  DcState* st = (DcState*)m->dc;
  if (st->d_layers) cudaFree(st->d_layers);
  delete st;
  m->dc = nullptr;
}

// Whether the single-stream decode of this model can run as the cluster kernel, and the set-up on first use.
bool decode_cluster_ready(FcModel* m) {
  if (m->dc) return ((DcState*)m->dc)->cluster > 0;
  DcState* st = new DcState();
  m->dc = st;
  st->cluster = -1;
  auto mat_ok = [&](const Linear& l) {
    const QMat& q = l.w->m;
    return (q.kind == FC_Q8_0 || q.kind == FC_Q4_0) && q.k % 128 == 0 && ((uintptr_t)q.qs & 15) == 0;
  };
  if (m->arch != ARCH_GPT2 || m->hd != 64 || m->heads != m->kv_heads) return false;
  if (m->dim % 64 || m->hidden % 128 || m->heads > DC_MAX_CLUSTER || !mat_ok(m->head)) return false;
  for (auto& l : m->layers)
    if (!mat_ok(l.qkv) || !mat_ok(l.wo) || !mat_ok(l.ff1) || !mat_ok(l.ff2)) return false;
  // small enough that a token is bound by its chain of stages, not by its bytes (the weights live in L2)
  if (m->weight_bytes > ((uint64_t)48 << 20)) return false;
  DcArgs& a = st->args;
  a = DcArgs();
  const uint32_t items_max = DC_MAX_CLUSTER; // heads * parts <= cluster size by construction
  a.off_h = m->dim;
  a.off_q = a.off_h + m->dim;
  a.off_act = a.off_q + m->dim;
  a.off_part = a.off_act + m->hidden;
  a.off_am = a.off_part + items_max * 66;
  a.off_ln = a.off_am + 2 * DC_MAX_CLUSTER;
  a.off_desc = (a.off_ln + (4 * m->n_layers + 2) * m->dim + 3) & ~3u; // (16-byte aligned: the descriptors hold pointers)
  a.smem_floats = a.off_desc + (uint32_t)((m->n_layers * sizeof(DcLayer) + 3) / 4);
  const size_t smem = (size_t)a.smem_floats * 4;
  if (smem > 200 * 1024) return false;
  if (cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
      cudaFuncSetAttribute(decode_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  for (int size : {16, 8}) {
    if ((int)m->heads > size) continue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size);
    cfg.blockDim = dim3(DC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = size, at.val.clusterDim.y = 1, at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_cluster_kernel, &cfg) == cudaSuccess && n >= 1) {
      st->cluster = size;
      break;
    }
    cudaGetLastError();
  }
  if (st->cluster <= 0) return false;
  std::vector<DcLayer> hl(m->n_layers);
  auto mat = [](const Linear& l) {
    DcMat d;
    d.qs = l.w->m.qs, d.sc = l.w->m.sc, d.bias = l.bias, d.k = l.w->m.k, d.n = l.w->m.n, d.kind = l.w->m.kind;
    return d;
  };
  for (uint32_t i = 0; i < m->n_layers; i++) {
    const Layer& l = m->layers[i];
    hl[i].n1g = l.norm1_g, hl[i].n1b = l.norm1_b, hl[i].n2g = l.norm2_g, hl[i].n2b = l.norm2_b;
    hl[i].qkv = mat(l.qkv), hl[i].wo = mat(l.wo), hl[i].ff1 = mat(l.ff1), hl[i].ff2 = mat(l.ff2);
    hl[i].kc = l.kv.k, hl[i].vc = l.kv.v;
  }
  if (cudaMalloc((void**)&st->d_layers, hl.size() * sizeof(DcLayer)) != cudaSuccess ||
      cudaMemcpy(st->d_layers, hl.data(), hl.size() * sizeof(DcLayer), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    st->cluster = -1;
    return false;
  }
  a.layers = st->d_layers;
  a.n_layers = m->n_layers, a.dim = m->dim, a.heads = m->heads, a.hd = m->hd, a.hidden = m->hidden, a.vocab = m->vocab, a.ctx = m->ctx;
  a.tok = m->tok, a.pos_table = m->pos_table, a.nfg = m->normf_g, a.nfb = m->normf_b;
  a.head = mat(m->head);
  a.head.bias = nullptr;
  a.logits = m->logits, a.d_ids = m->d_ids, a.d_pos = m->d_pos, a.d_argmax = m->d_argmax;
  a.log = m->d_chain_log, a.log_cnt = m->d_chain_cnt;
  return true;
}

// `steps` decode steps of one stream in one launch. !chained: the step's token and position are in d_ids / d_pos
// (one step). chained: the first token is the pick in d_argmax, the position d_pos + 1; every consumed token is
// appended to the chain log. Leaves the last step's logits row in m->logits and its pick in d_argmax.
int k_decode_cluster(FcModel* m, uint32_t stream, uint32_t steps, bool chained) {
  DcState* st = (DcState*)m->dc;
  FcDevice* dev = m->dev;
  DcArgs a = st->args;
  a.steps = steps;
  a.chained = chained ? 1 : 0;
  a.kv_off = (size_t)stream * m->kv_heads * m->ctx * m->hd;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(st->cluster);
  cfg.blockDim = dim3(DC_THREADS);
  cfg.dynamicSmemBytes = (size_t)a.smem_floats * 4;
  cfg.stream = dev->stream;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = st->cluster, at.val.clusterDim.y = 1, at.val.clusterDim.z = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  FC_LAUNCH(dev, "decode_cluster", cudaLaunchKernelEx(&cfg, decode_cluster_kernel, a));
  return FC_OK;
}
