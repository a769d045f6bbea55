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

// Fragments of one 32-wide block for rows g and g + 8: a[s] = {a0, a1, a2, a3} of k16 step s.
template <int KIND>
__device__ __forceinline__ void load_a(const QMat& w, uint32_t row_g, uint32_t row_g8, uint32_t kb, int t, uint32_t a[2][4],
                                       float& dg, float& dg8) {
  const uint32_t nb = w.k / QK;
  dg = __half2float(w.sc[(size_t)row_g * nb + kb]);
  dg8 = __half2float(w.sc[(size_t)row_g8 * nb + kb]);
  if (KIND == FC_Q8_0) {
    const uint2 qa = __ldg(reinterpret_cast<const uint2*>(w.qs + (size_t)row_g * w.k + (size_t)kb * QK + 8 * t));
    const uint2 qb = __ldg(reinterpret_cast<const uint2*>(w.qs + (size_t)row_g8 * w.k + (size_t)kb * QK + 8 * t));
    const uint32_t wa[2] = {qa.x ^ 0x80808080u, qa.y ^ 0x80808080u}, wb[2] = {qb.x ^ 0x80808080u, qb.y ^ 0x80808080u};
#pragma unroll
    for (int s = 0; s < 2; s++) {
      // bytes (0,1) and (2,3) of the step's word become fp16 pairs 1024 + u, minus 1152 = the int8
      a[s][0] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5140), 0x64806480u);
      a[s][2] = h2sub(__byte_perm(wa[s], 0x64646464u, 0x5342), 0x64806480u);
      a[s][1] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5140), 0x64806480u);
      a[s][3] = h2sub(__byte_perm(wb[s], 0x64646464u, 0x5342), 0x64806480u);
    }
  } else {
    const uint32_t wa = __ldg(reinterpret_cast<const uint32_t*>(w.qs + (size_t)row_g * (w.k / 2) + (size_t)kb * 16 + 4 * t));
    const uint32_t wb = __ldg(reinterpret_cast<const uint32_t*>(w.qs + (size_t)row_g8 * (w.k / 2) + (size_t)kb * 16 + 4 * t));
#pragma unroll
    for (int s = 0; s < 2; s++) {
      // mask pair p of the word = elements (2p, 2p + 1); 0x6400 | nib = 1024 + nib, minus 1032 = nib - 8
      a[s][0] = h2sub(((wa >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][2] = h2sub(((wa >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][1] = h2sub(((wb >> (8 * s)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
      a[s][3] = h2sub(((wb >> (8 * s + 4)) & 0x000f000fu) | 0x64006400u, 0x64086408u);
    }
  }
}

// smem: [2 buffers][hi, lo][MP rows][XSTRIDE halves]
template <int KIND, int NB>
__global__ void __launch_bounds__(128)
    qmatvec_mma_kernel(QMat w, const __half* __restrict__ xh, const __half* __restrict__ xl, uint32_t m, float* __restrict__ y,
                       float* __restrict__ partial, uint32_t blocks_per_split, Epilogue ep) {
  extern __shared__ __align__(16) __half xs[];
  constexpr int MP = NB * 8;
  constexpr int PART = MP * XSTRIDE;  // halves of one part of one buffer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t n = w.n, k = w.k, nblocks = k / QK;
  const uint32_t row0 = blockIdx.x * ROWS_PER_CTA + warp * 16;
  const uint32_t row_g = min(row0 + g, n - 1), row_g8 = min(row0 + g + 8, n - 1);
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
        cp_async16(smem_u32(xs + (size_t)buf * 2 * PART + part * PART + r * XSTRIDE + ch * 8), src);
      }
    }
  };

  float acc[NB][4];
#pragma unroll
  for (int i = 0; i < NB; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

  if (n_slices > 0) {
    stage(0, 0);
    cp_async_commit();
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
#pragma unroll 1
    for (uint32_t bi = 0; bi < 4 && kb0 + bi < kb_end; bi++) {
      uint32_t a[2][4];
      float dg, dg8;
      load_a<KIND>(w, row_g, row_g8, kb0 + bi, t, a, dg, dg8);
#pragma unroll
      for (int nb = 0; nb < NB; nb++) {
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t off = (nb * 8 + g) * XSTRIDE + bi * QK + 8 * t;
#pragma unroll
        for (int s = 0; s < 2; s++) {
          const uint2 bh = *reinterpret_cast<const uint2*>(xhb + off + 4 * s);
          const uint2 bl = *reinterpret_cast<const uint2*>(xlb + off + 4 * s);
          mma_16816(c, a[s], bh.x, bh.y);
          mma_16816(c, a[s], bl.x, bl.y);
        }
        acc[nb][0] = fmaf(dg, c[0], acc[nb][0]);
        acc[nb][1] = fmaf(dg, c[1], acc[nb][1]);
        acc[nb][2] = fmaf(dg8, c[2], acc[nb][2]);
        acc[nb][3] = fmaf(dg8, c[3], acc[nb][3]);
      }
    }
    __syncthreads();
  }
  // c0, c1: weight row g, batch columns 2t, 2t + 1; c2, c3: weight row g + 8
#pragma unroll
  for (int nb = 0; nb < NB; nb++) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t row = row0 + g + (j >> 1) * 8, col = nb * 8 + 2 * t + (j & 1);
      if (row >= n || col >= m) continue;
      float v = acc[nb][j];
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

template <int KIND, int NB>
int launch(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t m, float* y, float* partial,
           uint32_t splits, uint32_t bps, const Epilogue& ep) {
  auto kern = qmatvec_mma_kernel<KIND, NB>;
  const size_t smem = (size_t)2 * 2 * NB * 8 * XSTRIDE * sizeof(__half);
  static bool attr = false;
  if (!attr) {
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = true;
  }
  dim3 grid((w.n + ROWS_PER_CTA - 1) / ROWS_PER_CTA, splits);
  FC_LAUNCH(dev, "qmatvec_mma", kern<<<grid, 128, smem, dev->stream>>>(w, xh, xl, m, y, partial, bps, ep));
  return FC_OK;
}

template <int KIND>
int pick_nb(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t m, float* y, float* partial,
            uint32_t splits, uint32_t bps, const Epilogue& ep) {
  if (m <= 16) return launch<KIND, 2>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
  if (m <= 32) return launch<KIND, 4>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
  return launch<KIND, 8>(dev, w, xh, xl, m, y, partial, splits, bps, ep);
}

} // namespace

bool qmatvec_mma_supports(const QMat& w, uint32_t m) {
  return (w.kind == FC_Q8_0 || w.kind == FC_Q4_0) && m > 8 && m <= 64 && w.k % XS == 0;
}

// Device scratch the product needs: the two fp16 terms of x and the split-K partial sums.
size_t qmatvec_mma_scratch_bytes(uint32_t k, uint32_t n) {
  const uint32_t row_ctas = (n + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
  uint32_t splits = 1; // an upper bound of what k_qmatvec_mma picks on any device of up to 160 SMs
  while (splits < 16 && row_ctas * splits < 2 * 160) splits *= 2;
  return (size_t)2 * 64 * k * 2 + (size_t)splits * 64 * n * 4 + 512;
}

int k_qmatvec_mma(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep, void* scratch) {
  const uint32_t mp = m <= 16 ? 16 : m <= 32 ? 32 : 64;
  __half* xh = (__half*)scratch;
  __half* xl = xh + (size_t)mp * w.k;
  float* partial = (float*)(((uintptr_t)(xl + (size_t)mp * w.k) + 255) & ~(uintptr_t)255);
  const size_t total = (size_t)mp * w.k;
  FC_LAUNCH(dev, "x_split", x_split_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(x, m, mp, w.k, xh, xl));
  // split K until the grid covers the SMs about twice (slices stay whole 128-k units)
  const uint32_t row_ctas = (w.n + ROWS_PER_CTA - 1) / ROWS_PER_CTA, slices = w.k / XS;
  uint32_t splits = 1;
  const uint32_t want = 2 * (uint32_t)dev->prop.multiProcessorCount;
  while (splits < 16 && row_ctas * splits < want && slices / (splits * 2) >= 1 && slices % (splits * 2) == 0) splits *= 2;
  const uint32_t bps = (w.k / QK) / splits;
  float* part = splits > 1 ? partial : nullptr;
  if (w.kind == FC_Q8_0)
    FC_TRY(pick_nb<FC_Q8_0>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  else
    FC_TRY(pick_nb<FC_Q4_0>(dev, w, xh, xl, m, y, part, splits, bps, ep));
  if (splits > 1) {
    const size_t tot = (size_t)m * w.n;
    FC_LAUNCH(dev, "splitk_reduce",
              splitk_reduce_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, dev->stream>>>(partial, splits, m, w.n, y, ep));
  }
  return FC_OK;
}
