// Causal attention for the scoring path, fp16 operands with f32 softmax and accumulation, never
// materialising the [t, t] probabilities. Replaces attn_gqa_scores.wgsl + attn_softmax.wgsl +
// attn_gqa_pv.wgsl and their MHA twins (ferrum_wgpu/src/ops/llama.rs:L119-L146,
// ops/mod.rs:L108-L127), which write and re-read a [batch * heads * t, t] buffer.
//
// One CTA of 4 warps owns 64 * MT query rows of one (sequence, head); each warp MT tiles of 16 rows,
// which share every K / V fragment it loads (MT = 2 halves the shared-memory traffic per MMA). K and
// V tiles of 64 keys stream through a double-buffered, XOR-swizzled shared-memory ring (cp.async);
// S = Q K^T and O += P V run on mma.sync m16n8k16 with ldmatrix-fed fragments, the running row
// maximum and sum live in registers (online softmax). head_dim is 64.
#include "gemm_tc.cuh"

namespace {

constexpr int BKV = 64, HD = 64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// address of 16-byte chunk `ch` of row `row` in a [rows][64] fp16 tile with the XOR swizzle
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, uint32_t row, uint32_t ch) {
  return tile + row * 128 + ((ch ^ (row & 7)) << 4);
}

// 64 rows x 64 fp16 from `src` (row stride `stride` elements; rows clamped to max_row) into a tile
__device__ __forceinline__ void load_tile(uint32_t tile, const __half* src, uint32_t row0, uint32_t max_row, size_t stride) {
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t c = threadIdx.x + 128 * i;
    const uint32_t row = c >> 3, ch = c & 7;
    const uint32_t gr = min(row0 + row, max_row);
    cp_async16(tile_addr(tile, row, ch), src + (size_t)gr * stride + ch * 8);
  }
}

template <int MT>
__global__ void __launch_bounds__(128)
    attn_causal_f16_kernel(const __half* __restrict__ qkv, uint32_t t, uint32_t heads, uint32_t kv_heads,
                           __half* __restrict__ out) {
  constexpr int BQ = 64 * MT;
  __shared__ __align__(1024) uint8_t sm[BQ * 128 + 2 * 2 * BKV * 128];
  const uint32_t q_tile = smem_u32(sm);
  const uint32_t kv_tiles = q_tile + BQ * 128;

  const uint32_t qd = heads * HD, kvd = kv_heads * HD;
  const size_t stride = qd + 2 * kvd;
  const uint32_t qb = gridDim.x - 1 - blockIdx.x; // heaviest (latest) query blocks first
  const uint32_t h = blockIdx.y, seq = blockIdx.z;
  const uint32_t kvh = h / (heads / kv_heads);
  const __half* base = qkv + (size_t)seq * t * stride;
  const __half* qsrc = base + (size_t)h * HD;
  const __half* ksrc = base + qd + (size_t)kvh * HD;
  const __half* vsrc = ksrc + kvd;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const uint32_t q0 = qb * BQ;
  const uint32_t wrow0 = q0 + warp * 16 * MT;                        // first query row of this warp
  const uint32_t n_kv = min((q0 + BQ + BKV - 1) / BKV, (t + BKV - 1) / BKV); // causal: key blocks up to the last row's

#pragma unroll
  for (int i = 0; i < MT; i++) load_tile(q_tile + i * 64 * 128, qsrc, q0 + i * 64, t - 1, stride);
  load_tile(kv_tiles, ksrc, 0, t - 1, stride);
  load_tile(kv_tiles + BKV * 128, vsrc, 0, t - 1, stride);
  cp_async_commit();

  float o[MT][8][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.0f;
  }
  uint32_t qf[MT][4][4];
  const float sl2 = 0.125f * 1.4426950408889634f; // 1/sqrt(64) * log2(e)

  for (uint32_t kb = 0; kb < n_kv; kb++) {
    const uint32_t buf = kb & 1;
    const uint32_t k_tile = kv_tiles + buf * (2 * BKV * 128), v_tile = k_tile + BKV * 128;
    if (kb + 1 < n_kv) { // prefetch the next K/V pair into the other buffer
      const uint32_t nk = kv_tiles + (buf ^ 1) * (2 * BKV * 128);
      load_tile(nk, ksrc, (kb + 1) * BKV, t - 1, stride);
      load_tile(nk + BKV * 128, vsrc, (kb + 1) * BKV, t - 1, stride);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (kb == 0) {
#pragma unroll
      for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
          const uint32_t row = warp * 16 * MT + mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          ldmatrix_x4(tile_addr(q_tile, row, 2 * ks + (lane >> 4)), qf[mt][ks][0], qf[mt][ks][1], qf[mt][ks][2], qf[mt][ks][3]);
        }
    }
    // every key of this block lies after every row of this warp: nothing to do but keep the barriers
    if (kb * BKV <= wrow0 + 16 * MT - 1) {
      // S = Q K^T: MT x (16 x 64) per warp, each K fragment used by all MT row tiles
      float s[MT][8][4];
#pragma unroll
      for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < 8; i++) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
#pragma unroll
        for (int nb = 0; nb < 8; nb += 2) {
          uint32_t b0, b1, b2, b3;
          const uint32_t key = nb * 8 + (lane & 7) + 8 * (lane >> 4);
          ldmatrix_x4(tile_addr(k_tile, key, 2 * ks + ((lane >> 3) & 1)), b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < MT; mt++) {
            mma_16816(s[mt][nb], qf[mt][ks], b0, b1);
            mma_16816(s[mt][nb + 1], qf[mt][ks], b2, b3);
          }
        }
      }
      uint32_t pf[MT][4][4]; // P as A fragments: k-step ks covers keys 16ks..16ks+15 = n-blocks 2ks, 2ks+1
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        // causal mask where the block reaches past the tile's first row, then online softmax
        const uint32_t qi0 = wrow0 + mt * 16 + g;
        if (kb * BKV + BKV - 1 > wrow0 + mt * 16) {
#pragma unroll
          for (int nb = 0; nb < 8; nb++) {
            const uint32_t kj = kb * BKV + nb * 8 + 2 * tq;
            if (kj > qi0) s[mt][nb][0] = -INFINITY;
            if (kj + 1 > qi0) s[mt][nb][1] = -INFINITY;
            if (kj > qi0 + 8) s[mt][nb][2] = -INFINITY;
            if (kj + 1 > qi0 + 8) s[mt][nb][3] = -INFINITY;
          }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
          mx[0] = fmaxf(mx[0], fmaxf(s[mt][nb][0], s[mt][nb][1]));
          mx[1] = fmaxf(mx[1], fmaxf(s[mt][nb][2], s[mt][nb][3]));
        }
        float corr[2], msc[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
          // key 0 is never masked and block 0 is never skipped, so the running maximum is finite from
          // the first processed block on; a fully masked row of a later block keeps it
          const float m_new = fmaxf(m_run[mt][r], mx[r]);
          corr[r] = ex2((m_run[mt][r] - m_new) * sl2);
          m_run[mt][r] = m_new;
          msc[r] = m_new * sl2;
          l_run[mt][r] *= corr[r];
        }
        float ls[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
          const float p0 = ex2(s[mt][nb][0] * sl2 - msc[0]), p1 = ex2(s[mt][nb][1] * sl2 - msc[0]);
          const float p2 = ex2(s[mt][nb][2] * sl2 - msc[1]), p3 = ex2(s[mt][nb][3] * sl2 - msc[1]);
          ls[0] += p0 + p1;
          ls[1] += p2 + p3;
          pf[mt][nb >> 1][(nb & 1) * 2] = pack_f16(p0, p1);     // row g
          pf[mt][nb >> 1][(nb & 1) * 2 + 1] = pack_f16(p2, p3); // row g + 8
        }
        l_run[mt][0] += ls[0];
        l_run[mt][1] += ls[1];
#pragma unroll
        for (int db = 0; db < 8; db++) {
          o[mt][db][0] *= corr[0];
          o[mt][db][1] *= corr[0];
          o[mt][db][2] *= corr[1];
          o[mt][db][3] *= corr[1];
        }
      }
      // O += P V, each V fragment used by all MT row tiles
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
#pragma unroll
        for (int db = 0; db < 8; db += 2) {
          uint32_t b0, b1, b2, b3;
          const uint32_t key = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          ldmatrix_x4_trans(tile_addr(v_tile, key, db + (lane >> 4)), b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < MT; mt++) {
            mma_16816(o[mt][db], pf[mt][ks], b0, b1);
            mma_16816(o[mt][db + 1], pf[mt][ks], b2, b3);
          }
        }
      }
    }
    __syncthreads(); // everyone is done with this buffer before the next prefetch overwrites it
  }
  // row sums live per thread: combine the 4 threads of a row, normalise, store
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      l_run[mt][r] += __shfl_xor_sync(0xffffffffu, l_run[mt][r], 1);
      l_run[mt][r] += __shfl_xor_sync(0xffffffffu, l_run[mt][r], 2);
    }
    const float inv0 = 1.0f / l_run[mt][0], inv1 = 1.0f / l_run[mt][1];
    const uint32_t r0 = wrow0 + mt * 16 + g, r1 = r0 + 8;
#pragma unroll
    for (int db = 0; db < 8; db++) {
      const uint32_t col = h * HD + db * 8 + 2 * tq;
      if (r0 < t)
        *reinterpret_cast<uint32_t*>(out + ((size_t)seq * t + r0) * qd + col) = pack_f16(o[mt][db][0] * inv0, o[mt][db][1] * inv0);
      if (r1 < t)
        *reinterpret_cast<uint32_t*>(out + ((size_t)seq * t + r1) * qd + col) = pack_f16(o[mt][db][2] * inv1, o[mt][db][3] * inv1);
    }
  }
}

} // namespace

// attn_tmem.cu
bool attn_tmem_supports(uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads, uint32_t hd);
int k_attn_causal_tmem(FcDevice* dev, const __half* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                       uint32_t hd, __half* out);

// variant: 0 picks by sequence length, 1 / 2 the mma.sync kernel with one / two row tiles per warp,
// 3 the tcgen05 kernel
int k_attn_causal_f16_variant(FcDevice* dev, const __half* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads,
                              uint32_t kv_heads, uint32_t hd, __half* out, int variant) {
  if (!n_seqs || !t) return FC_OK;
  if (hd != HD) return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-core attention is built for head_dim 64, not %u", hd);
  if (n_seqs > 65535) return fc_fail(dev, FC_ERR_UNSUPPORTED, "%u sequences exceed one attention launch", n_seqs);
  if (!kv_heads || heads % kv_heads) return fc_fail(dev, FC_ERR_SHAPE, "%u query heads over %u kv heads", heads, kv_heads);
  if (variant == 0) variant = (t > 128 && attn_tmem_supports(n_seqs, t, heads, kv_heads, hd)) ? 3 : 1;
  if (variant == 3) return k_attn_causal_tmem(dev, qkv, n_seqs, t, heads, kv_heads, hd, out);
  if (variant == 2) {
    dim3 grid((t + 127) / 128, heads, n_seqs);
    FC_LAUNCH(dev, "attn_causal_f16", attn_causal_f16_kernel<2><<<grid, 128, 0, dev->stream>>>(qkv, t, heads, kv_heads, out));
  } else {
    dim3 grid((t + 63) / 64, heads, n_seqs);
    FC_LAUNCH(dev, "attn_causal_f16", attn_causal_f16_kernel<1><<<grid, 128, 0, dev->stream>>>(qkv, t, heads, kv_heads, out));
  }
  return FC_OK;
}

int k_attn_causal_f16(FcDevice* dev, const __half* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                      uint32_t hd, __half* out) {
  return k_attn_causal_f16_variant(dev, qkv, n_seqs, t, heads, kv_heads, hd, out, 0);
}

// Stand-alone causal attention over a packed fp16 [n_seqs * t][(heads + 2 kv_heads) * 64] host buffer
// (q heads | k heads | v heads per row); the result is fp16 [n_seqs * t][heads * 64]. Test and
// measurement hook: `iters` back-to-back launches, the average device time of one is returned.
FC_API int fc_debug_attention_f16(FcDevice* dev, const uint16_t* qkv_host, uint32_t n_seqs, uint32_t t, uint32_t heads,
                                  uint32_t kv_heads, uint16_t* out_host, int variant, int iters, float* ms_out) {
  if (!dev || !qkv_host || !out_host) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  if (!n_seqs || !t || !heads || !kv_heads) return fc_fail(dev, FC_ERR_SHAPE, "empty attention problem");
  const size_t rows = (size_t)n_seqs * t, in_elems = rows * (heads + 2 * kv_heads) * HD, out_elems = rows * heads * HD;
  __half *d_in = nullptr, *d_out = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int rc = FC_OK;
  auto body = [&]() -> int {
    FC_CUDA(dev, cudaMalloc(&d_in, in_elems * 2));
    FC_CUDA(dev, cudaMalloc(&d_out, out_elems * 2));
    FC_CUDA(dev, cudaMemcpyAsync(d_in, qkv_host, in_elems * 2, cudaMemcpyHostToDevice, dev->stream));
    FC_CUDA(dev, cudaMemsetAsync(d_out, 0, out_elems * 2, dev->stream));
    FC_CUDA(dev, cudaEventCreate(&e0));
    FC_CUDA(dev, cudaEventCreate(&e1));
    FC_TRY(k_attn_causal_f16_variant(dev, d_in, n_seqs, t, heads, kv_heads, HD, d_out, variant)); // warm-up, checked below
    FC_CUDA(dev, cudaEventRecord(e0, dev->stream));
    for (int i = 0; i < iters; i++) FC_TRY(k_attn_causal_f16_variant(dev, d_in, n_seqs, t, heads, kv_heads, HD, d_out, variant));
    FC_CUDA(dev, cudaEventRecord(e1, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(out_host, d_out, out_elems * 2, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    FC_TRY(tc_check_errors(dev));
    if (ms_out) {
      float ms = 0.0f;
      FC_CUDA(dev, cudaEventElapsedTime(&ms, e0, e1));
      *ms_out = iters > 0 ? ms / (float)iters : 0.0f;
    }
    return FC_OK;
  };
  rc = body();
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (d_in) cudaFree(d_in);
  if (d_out) cudaFree(d_out);
  return rc;
}
