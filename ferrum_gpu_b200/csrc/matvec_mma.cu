// Batched-decode product: y[m, n] = x[m, k] . W[n, k]^T for 9 <= m <= 64 rows (concurrent streams),
// at f32-class accuracy on the tensor cores, so the weight stream stays the bound instead of fp32 FMA
// throughput (64 rows x 420 M weights is 54 GFLOP per step of the 24-layer decode configuration).
//
// The quants are small integers, exact in fp16; the block's f16 scale is applied in f32 after each
// 32-wide block, on the mma.sync accumulator registers (which is why this is mma.sync and not
// tcgen05: tensor-memory accumulators cannot be rescaled per block). x is split once into two fp16
// terms, hi = fp16(x) and lo = fp16(x - hi), 22 significant bits together; both are multiplied with
// the same integer fragment. Products are exact and accumulation is f32.
//
// One warp owns 16 weight rows. Lane (g, t) reads 8 consecutive quants of rows g and g + 8 of each
// block (Q8_0: 8 bytes, Q4_0: one word) - the mma k slots are permuted so that those 8 values are
// exactly the lane's A-fragment of the block's two k16 steps, and the matching 4 + 4 fp16 of x come
// from shared memory with one 8-byte load per step. x slices (128 k) are staged by cp.async, double
// buffered. With few output rows the K axis is split across CTAs; partial sums are combined in a
// fixed order by a second kernel (no atomics: repeated runs are bit-identical).
#include "common.cuh"

namespace {

constexpr int XS = 128;        // k per staged x slice
constexpr int XSTRIDE = XS + 16; // halves per staged row (+32 bytes: conflict-free 8-byte reads)
constexpr int ROWS_PER_CTA = 64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float gelu_f(float x) {
  const float K = 0.7978846f;
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

// x[m][k] f32 -> hi, lo fp16 [mp][k] (rows >= m are zero)
__global__ void x_split_kernel(const float* __restrict__ x, uint32_t m, uint32_t mp, uint32_t k, __half* __restrict__ xh,
                               __half* __restrict__ xl) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)mp * k) return;
  const uint32_t r = (uint32_t)(i / k);
  float v = r < m ? x[i] : 0.0f;
  v = fminf(fmaxf(v, -65504.0f), 65504.0f); // saturate instead of overflowing to infinity
  const __half h = __float2half_rn(v);
  xh[i] = h;
  xl[i] = __float2half_rn(v - __half2float(h));
}

// RMSNorm / LayerNorm of row r of x and the split of the result, in one pass: what k_rmsnorm /
// k_layernorm followed by x_split_kernel produce (the same summation order, so the same bits), for the
// products whose input is "the norm of the residual stream". One CTA of 256 threads per padded row.
__device__ __forceinline__ float block_sum_mma(float v, float* red) {
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
__global__ void __launch_bounds__(256)
    norm_split_kernel(const float* x, uint32_t m, uint32_t k, int norm, const float* __restrict__ g,
                      const float* __restrict__ b, float eps, __half* __restrict__ xh, __half* __restrict__ xl,
                      DeferredReduce pend) {
  __shared__ float red[32];
  const uint32_t r = blockIdx.x;
  __half* oh = xh + (size_t)r * k;
  __half* ol = xl + (size_t)r * k;
  if (r >= m) { // padding rows of the n-block
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) oh[i] = ol[i] = __float2half_rn(0.0f);
    return;
  }
  const float* row = x + (size_t)r * k;
  if (pend.splits) {
    // x is the result of a product whose split-K partials are still apart: finish it exactly as
    // splitk_reduce_kernel would (ascending split order, bias, residual) and store it; the block reads
    // the row back below (x is pend.y, and not declared restrict for that reason).
    float* yrow = pend.y + (size_t)r * k;
    const size_t split_stride = (size_t)pend.m * k;
    const float* prow = pend.partial + (size_t)r * k;
    for (uint32_t i = threadIdx.x * 4; i < k; i += blockDim.x * 4) { // (k is a multiple of 128; rows are 16-byte aligned)
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
      if (pend.resid) {
        const float4 rr = *reinterpret_cast<const float4*>(pend.resid + (size_t)r * k + i);
        v.x = rr.x + v.x, v.y = rr.y + v.y, v.z = rr.z + v.z, v.w = rr.w + v.w;
      }
      *reinterpret_cast<float4*>(yrow + i) = v;
    }
    __syncthreads(); // the loops below give the elements to other threads
    row = yrow;
  }
  float mean = 0.0f, inv;
  if (norm == NORM_RMS) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum_mma(ss, red);
    inv = 1.0f / sqrtf(ss / (float)k + eps);
  } else {
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) s += row[i];
    mean = block_sum_mma(s, red) / (float)k;
    float vs = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
      const float dl = row[i] - mean;
      vs = fmaf(dl, dl, vs);
    }
    inv = 1.0f / sqrtf(block_sum_mma(vs, red) / (float)k + 1e-5f);
  }
  for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
    float v = norm == NORM_RMS ? row[i] * inv * g[i] : (row[i] - mean) * inv * g[i] + b[i];
    v = fminf(fmaxf(v, -65504.0f), 65504.0f);
    const __half h = __float2half_rn(v);
    oh[i] = h;
    ol[i] = __float2half_rn(v - __half2float(h));
  }
}

// Fragments of one 32-wide block for rows g and g + 8: a[s] = {a0, a1, a2, a3} of k16 step s.
// The packed quants and scales of one block for rows g and g + 8, as loaded; kept apart from the
// conversion so that the next block's loads are in flight while the current one is multiplied.
template <int KIND>
struct BlockRegs {
  uint32_t q[KIND == FC_F16 ? 8 : kind_byte_blocks(KIND) ? 4 : 2]; // F16: the lane's 8 values of each row as they are
  __half d[2];
};
template <int KIND>
__device__ __forceinline__ void load_block(BlockRegs<KIND>& r, const QMat& w, uint32_t row_g, uint32_t row_g8, uint32_t kb, int t) {
  const uint32_t nb = w.k / QK;
  if (KIND == FC_F16) { // no scale: 16 bytes of each row
    const uint4 qa = __ldg(reinterpret_cast<const uint4*>(w.qs + ((size_t)row_g * w.k + (size_t)kb * QK + 8 * t) * 2));
    const uint4 qb = __ldg(reinterpret_cast<const uint4*>(w.qs + ((size_t)row_g8 * w.k + (size_t)kb * QK + 8 * t) * 2));
    r.q[0] = qa.x, r.q[1] = qa.y, r.q[KIND == FC_F16 ? 2 : 0] = qa.z, r.q[KIND == FC_F16 ? 3 : 0] = qa.w;
    r.q[KIND == FC_F16 ? 4 : 0] = qb.x, r.q[KIND == FC_F16 ? 5 : 0] = qb.y, r.q[KIND == FC_F16 ? 6 : 0] = qb.z,
                             r.q[KIND == FC_F16 ? 7 : 0] = qb.w;
    return;
  }
  r.d[0] = w.sc[(size_t)row_g * nb + kb];
  r.d[1] = w.sc[(size_t)row_g8 * nb + kb];
  if (kind_byte_blocks(KIND)) {
    const uint2 qa = __ldg(reinterpret_cast<const uint2*>(w.qs + (size_t)row_g * w.k + (size_t)kb * QK + 8 * t));
    const uint2 qb = __ldg(reinterpret_cast<const uint2*>(w.qs + (size_t)row_g8 * w.k + (size_t)kb * QK + 8 * t));
    r.q[0] = qa.x, r.q[1] = qa.y, r.q[kind_byte_blocks(KIND) ? 2 : 0] = qb.x, r.q[kind_byte_blocks(KIND) ? 3 : 1] = qb.y;
  } else {
    r.q[0] = __ldg(reinterpret_cast<const uint32_t*>(w.qs + (size_t)row_g * (w.k / 2) + (size_t)kb * 16 + 4 * t));
    r.q[1] = __ldg(reinterpret_cast<const uint32_t*>(w.qs + (size_t)row_g8 * (w.k / 2) + (size_t)kb * 16 + 4 * t));
  }
}
template <int KIND>
__device__ __forceinline__ void block_frags(const BlockRegs<KIND>& r, uint32_t a[2][4]) {
  if (KIND == FC_F16) { // the stored halves are the fragment
#pragma unroll
    for (int s = 0; s < 2; s++) {
      a[s][0] = r.q[KIND == FC_F16 ? 2 * s : 0];
      a[s][2] = r.q[KIND == FC_F16 ? 2 * s + 1 : 0];
      a[s][1] = r.q[KIND == FC_F16 ? 4 + 2 * s : 0];
      a[s][3] = r.q[KIND == FC_F16 ? 5 + 2 * s : 0];
    }
  } else if (KIND == FC_MXFP4) { // element order: pairs (0,1) (2,3) | (4,5) (6,7) are the two k16 steps
    uint32_t ha[4], hb[4];
    e2m1x8_to_f16x2(r.q[0], ha);
    e2m1x8_to_f16x2(r.q[1], hb);
#pragma unroll
    for (int s = 0; s < 2; s++) {
      a[s][0] = ha[2 * s];
      a[s][2] = ha[2 * s + 1];
      a[s][1] = hb[2 * s];
      a[s][3] = hb[2 * s + 1];
    }
  } else if (kind_is_fp8(KIND)) { // every code is an fp16 value
#pragma unroll
    for (int s = 0; s < 2; s++) {
      a[s][0] = fp8x2_to_f16x2<KIND>(r.q[s]);
      a[s][2] = fp8x2_to_f16x2<KIND>(r.q[s] >> 16);
      a[s][1] = fp8x2_to_f16x2<KIND>(r.q[kind_byte_blocks(KIND) ? 2 + s : 0]);
      a[s][3] = fp8x2_to_f16x2<KIND>(r.q[kind_byte_blocks(KIND) ? 2 + s : 0] >> 16);
    }
  } else if (KIND == FC_Q8_0) {
    const uint32_t wa[2] = {r.q[0] ^ 0x80808080u, r.q[1] ^ 0x80808080u};
    const uint32_t wb[2] = {r.q[KIND == FC_Q8_0 ? 2 : 0] ^ 0x80808080u, r.q[KIND == FC_Q8_0 ? 3 : 1] ^ 0x80808080u};
#pragma unroll
    for (int s = 0; s < 2; s++) {
      a[s][0] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5140), 0x64806480u);
      a[s][2] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5342), 0x64806480u);
      a[s][1] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5140), 0x64806480u);
      a[s][3] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5342), 0x64806480u);
    }
  } else {
    const uint32_t wa = r.q[0], wb = r.q[1];
#pragma unroll
    for (int s = 0; s < 2; s++) {
      a[s][0] = h2sub(((wa >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][2] = h2sub(((wa >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][1] = h2sub(((wb >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][3] = h2sub(((wb >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
    }
  }
}

// smem: [2 buffers][hi, lo][MP rows][128 halves]. A lane reads the 16 bytes of x it multiplies with one block
// in one load; the 16-byte chunk index of odd rows is XORed with 4, so that the two rows a quarter-warp reads
// lie in different halves of the banks (unpadded rows 256 bytes apart would all start on bank 0; with 8-byte
// loads and rows padded by 32 bytes half of all shared-memory wavefronts of the kernel were bank conflicts).
// RW: 16-row tiles of the weight a warp holds at once. Two tiles share every load of x from shared memory (the
// kernel's busiest unit at one tile): used for the long outputs that need no split of K, the vocabulary head.
template <int KIND, int NB, int RW>
__global__ void __launch_bounds__(128)
    qmatvec_mma_kernel(QMat w, const __half* __restrict__ xh, const __half* __restrict__ xl, uint32_t m, float* __restrict__ y,
                       float* __restrict__ partial, uint32_t blocks_per_split, Epilogue ep) {
  extern __shared__ __align__(16) __half xs[];
  constexpr int MP = NB * 8;
  constexpr int XROW = XS;            // halves per staged row
  constexpr int PART = MP * XROW;     // halves of one part of one buffer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t n = w.n, k = w.k, nblocks = k / QK;
  const uint32_t row0 = blockIdx.x * (ROWS_PER_CTA * RW) + warp * (16 * RW);
  uint32_t row_g[RW], row_g8[RW];
#pragma unroll
  for (int i = 0; i < RW; i++) row_g[i] = min(row0 + 16 * i + g, n - 1), row_g8[i] = min(row0 + 16 * i + g + 8, n - 1);
  const uint32_t kb_begin = blockIdx.y * blocks_per_split;
  const uint32_t kb_end = min(kb_begin + blocks_per_split, nblocks);
  const uint32_t n_slices = (kb_end - kb_begin + 3) / 4; // 4 blocks per staged slice

  auto stage = [&](uint32_t slice, uint32_t buf) {
    // MP rows x 128 k x 2 parts, 16-byte chunks: 16 chunks per row per part
    const uint32_t k0 = (kb_begin + slice * 4) * QK;
    for (uint32_t c = threadIdx.x; c < (uint32_t)MP * 32; c += blockDim.x) {
      const uint32_t part = c / (MP * 16), rc = c % (MP * 16), r = rc / 16, ch = rc % 16;
      const uint32_t kk = k0 + ch * 8;
      if (kk < kb_end * QK) {
        const __half* src = (part ? xl : xh) + (size_t)r * k + kk;
        cp_async16(smem_u32(xs + (size_t)buf * 2 * PART + part * PART + r * XROW + ((ch ^ ((r & 1) << 2)) * 8)), src);
      }
    }
  };

  float acc[RW][NB][4];
#pragma unroll
  for (int i = 0; i < RW; i++)
#pragma unroll
    for (int j = 0; j < NB; j++) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

  // The packed blocks of the warp's two rows are requested three blocks before they are multiplied (a ring of
  // four register sets, indexed by the block's place in its slice): a block is 8 MMAs per n-block, about 250
  // cycles of tensor work at 64 rows of x, and a load issued only one block ahead - several hundred cycles to L2 -
  // left the tensor pipe a third busy on the long rows of the vocabulary head.
  BlockRegs<KIND> ring[4][RW];
  if (n_slices > 0) {
    stage(0, 0);
    cp_async_commit();
#pragma unroll
    for (int p = 0; p < 3; p++)
      if (kb_begin + p < kb_end) {
#pragma unroll
        for (int i = 0; i < RW; i++) load_block<KIND>(ring[p][i], w, row_g[i], row_g8[i], kb_begin + p, t);
      }
  }
  for (uint32_t sl = 0; sl < n_slices; sl++) {
    const uint32_t buf = sl & 1;
    if (sl + 1 < n_slices) {
      stage(sl + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __half* xhb = xs + (size_t)buf * 2 * PART;
    const __half* xlb = xhb + PART;
    const uint32_t kb0 = kb_begin + sl * 4;
#pragma unroll
    for (int bi = 0; bi < 4; bi++) {
      if (kb0 + bi >= kb_end) break;
      if (kb0 + bi + 3 < kb_end) {
#pragma unroll
        for (int i = 0; i < RW; i++) load_block<KIND>(ring[(bi + 3) & 3][i], w, row_g[i], row_g8[i], kb0 + bi + 3, t);
      }
      uint32_t a[RW][2][4];
      float dg[RW], dg8[RW];
#pragma unroll
      for (int i = 0; i < RW; i++) {
        block_frags<KIND>(ring[bi][i], a[i]);
        dg[i] = KIND == FC_F16 ? 1.0f : block_scale_f32<KIND>(ring[bi][i].d[0]);
        dg8[i] = KIND == FC_F16 ? 1.0f : block_scale_f32<KIND>(ring[bi][i].d[1]);
      }
#pragma unroll
      for (int nb = 0; nb < NB; nb++) {
        const uint32_t off = (nb * 8 + g) * XROW + (((bi * 4 + t) ^ ((g & 1) << 2)) * 8);
        const uint4 bh = *reinterpret_cast<const uint4*>(xhb + off);
        const uint4 bl = *reinterpret_cast<const uint4*>(xlb + off);
#pragma unroll
        for (int i = 0; i < RW; i++) {
          float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          mma_16816(c, a[i][0], bh.x, bh.y);
          mma_16816(c, a[i][0], bl.x, bl.y);
          mma_16816(c, a[i][1], bh.z, bh.w);
          mma_16816(c, a[i][1], bl.z, bl.w);
          acc[i][nb][0] = fmaf(dg[i], c[0], acc[i][nb][0]);
          acc[i][nb][1] = fmaf(dg[i], c[1], acc[i][nb][1]);
          acc[i][nb][2] = fmaf(dg8[i], c[2], acc[i][nb][2]);
          acc[i][nb][3] = fmaf(dg8[i], c[3], acc[i][nb][3]);
        }
      }
    }
    __syncthreads();
  }
  // c0, c1: weight row g, batch columns 2t, 2t + 1; c2, c3: weight row g + 8
#pragma unroll
  for (int i = 0; i < RW; i++)
#pragma unroll
  for (int nb = 0; nb < NB; nb++) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t row = row0 + 16 * i + g + (j >> 1) * 8, col = nb * 8 + 2 * t + (j & 1);
      if (row >= n || col >= m) continue;
      float v = acc[i][nb][j];
      if (partial) {
        partial[((size_t)blockIdx.y * m + col) * n + row] = v;
      } else {
        if (ep.bias) v += ep.bias[row];
        if (ep.act == ACT_GELU) v = gelu_f(v);
        if (ep.resid) v = ep.resid[(size_t)col * n + row] + v;
        y[(size_t)col * n + row] = v;
      }
    }
  }
}


// The same product for 1..8 rows of x (plain and small-batch decode): one 8-column n-block, and the
// weight stream is the whole cost, so it gets a real pipeline: the CTA's 64 rows x 128 k of packed
// quants, their scales and the f32 x slice arrive by cp.async in coalesced 16-byte pieces through a
// 4-stage shared-memory ring (four-byte loads straight from global touch 16 cache lines per warp
// instruction and run into the L1 tag rate at a seventh of the HBM bandwidth). x is split into its two
// fp16 terms from the staged f32 slice, inside the kernel.
template <int KIND>
struct Mma8 {
  static constexpr int ST = 4;
  static constexpr int WBYTES = KIND == FC_F16 ? 256 : kind_byte_blocks(KIND) ? 128 : 64;  // bytes of one row of a 128-k slice
  static constexpr int WROW = KIND == FC_F16 ? 320 : kind_byte_blocks(KIND) ? 160 : 80;    // padded: lanes (g, t) read conflict-free
  static constexpr int W_STAGE = 64 * WROW;
  static constexpr int SC_STAGE = 64 * 8;                    // 4 f16 scales per row
  static constexpr int XF_STAGE = 8 * XS * 4;                // f32 x slice
  static constexpr int XS_BYTES = 2 * 8 * XSTRIDE * 2;       // hi, lo as fp16
  static constexpr int SMEM = ST * (W_STAGE + SC_STAGE + XF_STAGE) + 2 * XS_BYTES;
};
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u; // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}

template <int KIND>
__global__ void __launch_bounds__(128)
    qmatvec_mma8_kernel(QMat w, const float* __restrict__ x, uint32_t m, float* __restrict__ y, float* __restrict__ partial,
                        uint32_t blocks_per_split, Epilogue ep) {
  using C = Mma8<KIND>;
  extern __shared__ __align__(16) uint8_t sm8[];
  uint8_t* wq = sm8;
  uint8_t* scs = wq + C::ST * C::W_STAGE;
  uint8_t* xf = scs + C::ST * C::SC_STAGE;
  __half* xs = reinterpret_cast<__half*>(xf + C::ST * C::XF_STAGE);
  constexpr int PART = 8 * XSTRIDE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t n = w.n, k = w.k, nblocks = k / QK;
  const uint32_t cta_row0 = blockIdx.x * ROWS_PER_CTA;
  const uint32_t kb_begin = blockIdx.y * blocks_per_split;         // whole 4-block slices; the last split may be shorter
  const uint32_t n_slices = (min(kb_begin + blocks_per_split, nblocks) - kb_begin) / 4;

  auto issue = [&](uint32_t slice) {
    const uint32_t st = slice % C::ST, kb0 = kb_begin + slice * 4;
    // packed quants: 64 rows x WBYTES in 16-byte pieces
    constexpr int PER_ROW = C::WBYTES / 16;
#pragma unroll
    for (int j = 0; j < PER_ROW * 64 / 128; j++) {
      const uint32_t c = threadIdx.x + 128 * j, row = c / PER_ROW, ch = c % PER_ROW;
      const uint32_t grow = min(cta_row0 + row, n - 1); // rows past the end are computed and dropped
      const uint8_t* src =
          w.qs + (size_t)grow * (KIND == FC_F16 ? 2 * k : kind_byte_blocks(KIND) ? k : k / 2) + (size_t)kb0 * (C::WBYTES / 4) + ch * 16;
      cp_async16(smem_u32(wq + st * C::W_STAGE + row * C::WROW + ch * 16), src);
    }
    if (KIND != FC_F16 && threadIdx.x < 64) {
      const uint32_t grow = min(cta_row0 + threadIdx.x, n - 1);
      cp_async8(smem_u32(scs + st * C::SC_STAGE + threadIdx.x * 8), w.sc + (size_t)grow * nblocks + kb0);
    }
    // x slice: 8 rows x 128 f32, rows >= m zero-filled
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const uint32_t c = threadIdx.x + 128 * j, row = c >> 5, ch = c & 31;
      const bool valid = row < m;
      cp_async16_zfill(smem_u32(xf + st * C::XF_STAGE + (row * XS + ch * 4) * 4),
                       x + (size_t)(valid ? row : 0) * k + (size_t)kb0 * QK + ch * 4, valid);
    }
  };

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int p = 0; p < C::ST - 1; p++) { // one commit group per slice position, empty past the end
    if ((uint32_t)p < n_slices) issue(p);
    cp_async_commit();
  }
  const uint32_t r0 = warp * 16 + g, r1 = r0 + 8; // this lane's two weight rows within the CTA
  const uint32_t xr = threadIdx.x >> 4, xk = (threadIdx.x & 15) * 8; // x conversion: 8 consecutive k of one row
  for (uint32_t sl = 0; sl < n_slices; sl++) {
    const uint32_t st = sl % C::ST;
    cp_async_wait<C::ST - 2>();
    __syncthreads(); // slice sl has landed for every thread; everyone is done with slice sl - 1
    if (sl + C::ST - 1 < n_slices) issue(sl + C::ST - 1); // into the stage slice sl - 1 used
    cp_async_commit();
    { // split this slice of x into two fp16 terms
      const float* src = reinterpret_cast<const float*>(xf + st * C::XF_STAGE) + xr * XS + xk;
      const float4 xa = *reinterpret_cast<const float4*>(src), xb = *reinterpret_cast<const float4*>(src + 4);
      const float v[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      __half2 hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float c0 = fminf(fmaxf(v[2 * i], -65504.0f), 65504.0f), c1 = fminf(fmaxf(v[2 * i + 1], -65504.0f), 65504.0f);
        hi[i] = __floats2half2_rn(c0, c1); // saturated instead of overflowing to infinity
        const float2 back = __half22float2(hi[i]);
        lo[i] = __floats2half2_rn(c0 - back.x, c1 - back.y);
      }
      // (rows of 128 halves, the 16-byte chunk index of odd rows XORed with 4: see qmatvec_mma_kernel)
      __half* dst = xs + (size_t)(sl & 1) * 2 * PART + xr * XS + (((xk >> 3) ^ ((xr & 1) << 2)) << 3);
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hi);
      *reinterpret_cast<uint4*>(dst + PART) = *reinterpret_cast<const uint4*>(lo);
    }
    __syncthreads();
    const __half* xhb = xs + (size_t)(sl & 1) * 2 * PART;
    const __half* xlb = xhb + PART;
    const uint8_t* wst = wq + st * C::W_STAGE;
    const __half* sst = reinterpret_cast<const __half*>(scs + st * C::SC_STAGE);
#pragma unroll
    for (int bi = 0; bi < 4; bi++) {
      uint32_t a[2][4];
      if (KIND == FC_F16) {
        const uint4 qa = *reinterpret_cast<const uint4*>(wst + r0 * C::WROW + bi * 64 + 16 * t);
        const uint4 qb = *reinterpret_cast<const uint4*>(wst + r1 * C::WROW + bi * 64 + 16 * t);
        a[0][0] = qa.x, a[0][2] = qa.y, a[1][0] = qa.z, a[1][2] = qa.w;
        a[0][1] = qb.x, a[0][3] = qb.y, a[1][1] = qb.z, a[1][3] = qb.w;
      } else if (KIND == FC_MXFP4) {
        uint32_t ha[4], hb[4];
        e2m1x8_to_f16x2(*reinterpret_cast<const uint32_t*>(wst + r0 * C::WROW + bi * 16 + 4 * t), ha);
        e2m1x8_to_f16x2(*reinterpret_cast<const uint32_t*>(wst + r1 * C::WROW + bi * 16 + 4 * t), hb);
#pragma unroll
        for (int s = 0; s < 2; s++) {
          a[s][0] = ha[2 * s];
          a[s][2] = ha[2 * s + 1];
          a[s][1] = hb[2 * s];
          a[s][3] = hb[2 * s + 1];
        }
      } else if (kind_is_fp8(KIND)) {
        const uint2 qa = *reinterpret_cast<const uint2*>(wst + r0 * C::WROW + bi * 32 + 8 * t);
        const uint2 qb = *reinterpret_cast<const uint2*>(wst + r1 * C::WROW + bi * 32 + 8 * t);
        const uint32_t wa[2] = {qa.x, qa.y}, wb[2] = {qb.x, qb.y};
#pragma unroll
        for (int s = 0; s < 2; s++) {
          a[s][0] = fp8x2_to_f16x2<KIND>(wa[s]);
          a[s][2] = fp8x2_to_f16x2<KIND>(wa[s] >> 16);
          a[s][1] = fp8x2_to_f16x2<KIND>(wb[s]);
          a[s][3] = fp8x2_to_f16x2<KIND>(wb[s] >> 16);
        }
      } else if (KIND == FC_Q8_0) {
        const uint2 qa = *reinterpret_cast<const uint2*>(wst + r0 * C::WROW + bi * 32 + 8 * t);
        const uint2 qb = *reinterpret_cast<const uint2*>(wst + r1 * C::WROW + bi * 32 + 8 * t);
        const uint32_t wa[2] = {qa.x ^ 0x80808080u, qa.y ^ 0x80808080u}, wb[2] = {qb.x ^ 0x80808080u, qb.y ^ 0x80808080u};
#pragma unroll
        for (int s = 0; s < 2; s++) {
          a[s][0] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5140), 0x64806480u);
          a[s][2] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5342), 0x64806480u);
          a[s][1] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5140), 0x64806480u);
          a[s][3] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5342), 0x64806480u);
        }
      } else {
        const uint32_t wa = *reinterpret_cast<const uint32_t*>(wst + r0 * C::WROW + bi * 16 + 4 * t);
        const uint32_t wb = *reinterpret_cast<const uint32_t*>(wst + r1 * C::WROW + bi * 16 + 4 * t);
#pragma unroll
        for (int s = 0; s < 2; s++) {
          a[s][0] = h2sub(((wa >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
          a[s][2] = h2sub(((wa >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
          a[s][1] = h2sub(((wb >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
          a[s][3] = h2sub(((wb >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
        }
      }
      const float dg = KIND == FC_F16 ? 1.0f : block_scale_f32<KIND>(sst[r0 * 4 + bi]);
      const float dg8 = KIND == FC_F16 ? 1.0f : block_scale_f32<KIND>(sst[r1 * 4 + bi]);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const uint32_t off = g * XS + (((bi * 4 + t) ^ ((g & 1) << 2)) * 8);
      const uint4 bh = *reinterpret_cast<const uint4*>(xhb + off);
      const uint4 bl = *reinterpret_cast<const uint4*>(xlb + off);
      mma_16816(c, a[0], bh.x, bh.y);
      mma_16816(c, a[0], bl.x, bl.y);
      mma_16816(c, a[1], bh.z, bh.w);
      mma_16816(c, a[1], bl.z, bl.w);
      acc[0] = fmaf(dg, c[0], acc[0]);
      acc[1] = fmaf(dg, c[1], acc[1]);
      acc[2] = fmaf(dg8, c[2], acc[2]);
      acc[3] = fmaf(dg8, c[3], acc[3]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint32_t row = cta_row0 + warp * 16 + g + (j >> 1) * 8, col = 2 * t + (j & 1);
    if (row >= n || col >= m) continue;
    float v = acc[j];
    if (partial) {
      partial[((size_t)blockIdx.y * m + col) * n + row] = v;
    } else {
      if (ep.bias) v += ep.bias[row];
      if (ep.act == ACT_GELU) v = gelu_f(v);
      if (ep.resid) v = ep.resid[(size_t)col * n + row] + v;
      y[(size_t)col * n + row] = v;
    }
  }
}

// y = epilogue(sum over splits, ascending split index)
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, uint32_t splits, uint32_t m, uint32_t n,
                                     float* __restrict__ y, Epilogue ep) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * n) return;
  float v = 0.0f;
  for (uint32_t s = 0; s < splits; s++) v += partial[(size_t)s * m * n + i];
  const uint32_t row = (uint32_t)(i % n);
  if (ep.bias) v += ep.bias[row];
  if (ep.act == ACT_GELU) v = gelu_f(v);
  if (ep.resid) v = ep.resid[i] + v;
  y[i] = v;
}

template <int KIND, int NB, int RW = 1>
int launch(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t m, float* y, float* partial,
           uint32_t splits, uint32_t bps, const Epilogue& ep) {
  auto kern = qmatvec_mma_kernel<KIND, NB, RW>;
  const size_t smem = (size_t)2 * 2 * NB * 8 * XS * sizeof(__half);
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  dim3 grid((w.n + ROWS_PER_CTA * RW - 1) / (ROWS_PER_CTA * RW), splits);
  FC_LAUNCH(dev, "qmatvec_mma", kern<<<grid, 128, smem, dev->stream>>>(w, xh, xl, m, y, partial, bps, ep));
  return FC_OK;
}

template <int KIND>
int pick_nb(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t m, float* y, float* partial,
            uint32_t splits, uint32_t bps, const Epilogue& ep) {
  if (m <= 16) return launch<KIND, 2>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
  if (m <= 32) return launch<KIND, 4>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
  // an output long enough to fill the device many times over without a split of K: two row tiles per warp
  if (splits == 1 && (w.n + 127) / 128 >= 4 * (uint32_t)dev->prop.multiProcessorCount)
    return launch<KIND, 8, 2>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
  return launch<KIND, 8>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
}

} // namespace

bool qmatvec_mma_supports(const QMat& w, uint32_t m) {
  return (kind_has_scales(w.kind) || w.kind == FC_F16) && m >= 1 && m <= 64 && w.k % XS == 0;
}

// Device scratch the product needs: the two fp16 terms of x and the split-K partial sums.
size_t qmatvec_mma_scratch_bytes(uint32_t k, uint32_t n) {
  const uint32_t row_ctas = (n + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
  uint32_t splits = 1; // an upper bound of what k_qmatvec_mma picks on any device of up to 160 SMs
  while (splits < 16 && row_ctas * splits < 8 * 160) splits *= 2;
  return (size_t)2 * 64 * k * 2 + (size_t)splits * 64 * n * 4 + 512;
}

// 1..8 rows: x is converted inside the kernel; more CTAs than the wide variant wants (each holds few
// bytes in flight), so K is split until the grid covers the SMs about eight times
static int k_qmatvec_mma8(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep, void* scratch) {
  const uint32_t row_ctas = (w.n + ROWS_PER_CTA - 1) / ROWS_PER_CTA, slices = w.k / XS;
  const uint32_t want = 8 * (uint32_t)dev->prop.multiProcessorCount;
  uint32_t splits = (want + row_ctas - 1) / row_ctas;
  splits = splits < 1 ? 1 : splits > 16 ? 16 : splits;
  splits = splits > slices ? slices : splits;
  if ((size_t)w.n * w.k <= ((size_t)1 << 20)) splits = 1; // a second launch costs more than a few short CTAs
  const uint32_t slices_per_split = (slices + splits - 1) / splits; // whole slices; the last split may be shorter
  splits = (slices + slices_per_split - 1) / slices_per_split;
  const uint32_t bps = slices_per_split * (XS / QK);
  float* partial = (float*)(((uintptr_t)scratch + (size_t)2 * 64 * w.k * 2 + 255) & ~(uintptr_t)255);
  float* part = splits > 1 ? partial : nullptr;
  dim3 grid(row_ctas, splits);
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mma8<FC_Q8_0>::SMEM));
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mma8<FC_Q4_0>::SMEM));
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_FP8_E4M3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Mma8<FC_FP8_E4M3>::SMEM));
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_FP8_E5M2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Mma8<FC_FP8_E5M2>::SMEM));
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_MXFP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mma8<FC_MXFP4>::SMEM));
    FC_CUDA(dev, cudaFuncSetAttribute(qmatvec_mma8_kernel<FC_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mma8<FC_F16>::SMEM));
  }
  if (w.kind == FC_Q8_0)
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_Q8_0><<<grid, 128, Mma8<FC_Q8_0>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  else if (w.kind == FC_FP8_E4M3)
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_FP8_E4M3><<<grid, 128, Mma8<FC_FP8_E4M3>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  else if (w.kind == FC_FP8_E5M2)
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_FP8_E5M2><<<grid, 128, Mma8<FC_FP8_E5M2>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  else if (w.kind == FC_MXFP4)
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_MXFP4><<<grid, 128, Mma8<FC_MXFP4>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  else if (w.kind == FC_F16)
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_F16><<<grid, 128, Mma8<FC_F16>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  else
    FC_LAUNCH(dev, "qmatvec_mma8",
              qmatvec_mma8_kernel<FC_Q4_0><<<grid, 128, Mma8<FC_Q4_0>::SMEM, dev->stream>>>(w, x, m, y, part, bps, ep));
  if (splits > 1) {
    const size_t tot = (size_t)m * w.n;
    FC_LAUNCH(dev, "splitk_reduce",
              splitk_reduce_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, dev->stream>>>(partial, splits, m, w.n, y, ep));
  }
  return FC_OK;
}

// The plain reduce of a deferred product, for a consumer that cannot take it along.
int k_flush_deferred(FcDevice* dev, const DeferredReduce& d) {
  if (!d.splits) return FC_OK;
  Epilogue ep;
  ep.bias = d.bias;
  ep.resid = d.resid;
  const size_t tot = (size_t)d.m * d.n;
  FC_LAUNCH(dev, "splitk_reduce",
            splitk_reduce_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, dev->stream>>>(d.partial, d.splits, d.m, d.n, d.y, ep));
  return FC_OK;
}

void qmatvec_mma_split_ptrs(void* scratch, uint32_t m, uint32_t k, __half** xh, __half** xl, uint32_t* mp) {
  *mp = m <= 16 ? 16 : m <= 32 ? 32 : 64;
  *xh = (__half*)scratch;
  *xl = *xh + (size_t)*mp * k;
}

int k_qmatvec_mma(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep, void* scratch) {
  const bool tx = dev->matvec_choice == 0 && qgemm_tx_takes(dev, w, m, ep.defer_out != nullptr); // long outputs: the tcgen05 form (gemm_tc.cu)
  if (m <= 8 && !tx) return k_qmatvec_mma8(dev, w, x, m, y, ep, scratch);
  uint32_t mp;
  __half *xh, *xl;
  qmatvec_mma_split_ptrs(scratch, m, w.k, &xh, &xl, &mp);
  float* partial = ep.partial_at ? ep.partial_at : (float*)(((uintptr_t)(xl + (size_t)mp * w.k) + 255) & ~(uintptr_t)255);
  const size_t total = (size_t)mp * w.k;
  DeferredReduce pend;
  if (ep.pending && ep.pending->splits) {
    // taken along by the norm + split launch when it is this product's x and its partial sums lie clear
    // of the x terms that launch writes; finished on its own otherwise
    const DeferredReduce& d = *ep.pending;
    if (!ep.presplit && ep.norm != NORM_NONE && d.y == x && d.m == m && d.n == w.k &&
        (uintptr_t)d.partial >= (uintptr_t)(xl + (size_t)mp * w.k))
      pend = d;
    else
      FC_TRY(k_flush_deferred(dev, d));
  }
  if (ep.presplit) {
    // the producer of x wrote xh / xl itself
  } else if (ep.norm != NORM_NONE) // x is the raw residual stream: normalise and split in one launch
    FC_LAUNCH(dev, "norm_split",
              norm_split_kernel<<<mp, 256, 0, dev->stream>>>(x, m, w.k, ep.norm, ep.norm_g, ep.norm_b, ep.norm_eps, xh, xl, pend));
  else
    FC_LAUNCH(dev, "x_split", x_split_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(x, m, mp, w.k, xh, xl));
  if (tx) return k_qgemm_tx(dev, w, xh, xl, mp, m, y, ep);
  // split K until the grid covers the SMs about twice: whole 128-k slices per split, the last split may be
  // shorter (K = 2816 is 22 slices: 11 splits of 2, where a power-of-two rule stops at 2 splits of 11)
  const uint32_t row_ctas = (w.n + ROWS_PER_CTA - 1) / ROWS_PER_CTA, slices = w.k / XS;
  const uint32_t want = 2 * (uint32_t)dev->prop.multiProcessorCount;
  uint32_t splits = (want + row_ctas - 1) / row_ctas;
  splits = splits < 1 ? 1 : splits > 16 ? 16 : splits;
  splits = splits > slices ? slices : splits;
  const uint32_t slices_per_split = (slices + splits - 1) / splits;
  splits = (slices + slices_per_split - 1) / slices_per_split; // no empty split
  const uint32_t bps = slices_per_split * (XS / QK);
  float* part = splits > 1 ? partial : nullptr;
  if (w.kind == FC_Q8_0)
    FC_TRY(pick_nb<FC_Q8_0>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else if (w.kind == FC_FP8_E4M3)
    FC_TRY(pick_nb<FC_FP8_E4M3>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else if (w.kind == FC_FP8_E5M2)
    FC_TRY(pick_nb<FC_FP8_E5M2>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else if (w.kind == FC_MXFP4)
    FC_TRY(pick_nb<FC_MXFP4>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else if (w.kind == FC_F16)
    FC_TRY(pick_nb<FC_F16>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else
    FC_TRY(pick_nb<FC_Q4_0>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  if (splits > 1 && ep.defer_out && ep.act == ACT_NONE) { // the consumer's norm + split launch finishes the sum
    DeferredReduce& d = *ep.defer_out;
    d.partial = partial;
    d.splits = splits;
    d.m = m;
    d.n = w.n;
    d.bias = ep.bias;
    d.resid = ep.resid;
    d.y = y;
    return FC_OK;
  }
  if (splits > 1) {
    const size_t tot = (size_t)m * w.n;
    FC_LAUNCH(dev, "splitk_reduce",
              splitk_reduce_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, dev->stream>>>(partial, splits, m, w.n, y, ep));
  }
  return FC_OK;
}
