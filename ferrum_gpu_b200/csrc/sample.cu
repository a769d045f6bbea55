// Candidate selection for sampled decoding on the device: the repetition penalty and the exact top-k of
// a logits row in the reference's order, so that a sampled token costs k (index, value) pairs over the
// bus instead of the whole row (vocab x 4 bytes per token and stream in the reference's loop,
// ferrum_gpu_core/src/engine/mod.rs:L230-L240). The order is the one `sampling::sample` builds
// (ferrum_model/src/sampling.rs:L57-L66): non-NaN logits, descending by f32::total_cmp (so +0 before
// -0), ties keep the lower index first, truncated to top_k. The softmax over the k candidates, the
// nucleus cut and the draw stay with the caller's own `sample` (they are a few dozen flops and keep the
// draw bit-identical to the host path); greedy decoding keeps using the argmax kernel.
//
// One CTA of 1024 threads: a four-pass radix select over the sortable 32-bit keys finds the k-th largest
// key T and how many logits equal to T belong to the set, a second sweep gathers every key > T plus
// the first such ties in index order, and a bitonic sort of at most 1024 (key, ~index) words in shared
// memory puts them in order. The row (<= a few hundred KB) is read from L2 six times.
#include "common.cuh"

namespace {

constexpr int SEL_THREADS = 1024;
constexpr uint32_t MAX_K = 1024;

__device__ __forceinline__ uint32_t order_key(uint32_t bits) { return bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u); }
__device__ __forceinline__ uint32_t key_bits(uint32_t key) { return key ^ ((key >> 31) ? 0x80000000u : 0xffffffffu); }
__device__ __forceinline__ bool is_nan_bits(uint32_t bits) { return (bits & 0x7fffffffu) > 0x7f800000u; }

// sampling.rs:L44-L54: in the order of `recent`; a token listed twice is penalised twice
__global__ void penalty_kernel(float* __restrict__ l, uint32_t vocab, const int32_t* __restrict__ recent, uint32_t n, float pen) {
  if (blockIdx.x || threadIdx.x) return;
  for (uint32_t i = 0; i < n; i++) {
    const int32_t t = recent[i];
    if (t >= 0 && (uint32_t)t < vocab) {
      const float v = l[t];
      l[t] = v > 0.0f ? v / pen : v * pen;
    }
  }
}

__global__ void __launch_bounds__(SEL_THREADS)
    topk_kernel(const float* __restrict__ l, uint32_t vocab, uint32_t k, int32_t* __restrict__ out_idx, float* __restrict__ out_val,
                uint32_t* __restrict__ out_n) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_all, s_cnt;
  __shared__ uint32_t scan[SEL_THREADS];
  __shared__ unsigned long long cand[MAX_K];
  const uint32_t tid = threadIdx.x;
  const uint32_t* lb = reinterpret_cast<const uint32_t*>(l);
  if (tid == 0) {
    s_prefix = 0;
    s_need = k;
    s_all = 0;
    s_cnt = 0;
  }
  if (tid < MAX_K) cand[tid] = 0ull;
  __syncthreads();
  // radix select, most significant byte first: after the pass at `shift`, keys that agree with
  // s_prefix on the bytes above it are still in play and s_need of them (from the top) are wanted
  uint32_t mask = 0;
  for (int shift = 24; shift >= 0 && !s_all; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (uint32_t i = tid; i < vocab; i += SEL_THREADS) {
      const uint32_t b = lb[i];
      if (is_nan_bits(b)) continue;
      const uint32_t key = order_key(b);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t cum = 0, need = s_need;
      int d = 255;
      for (; d >= 0; d--) {
        if (cum + hist[d] >= need) break;
        cum += hist[d];
      }
      if (d < 0) {
        s_all = 1; // fewer candidates than k: all of them
      } else {
        s_need = need - cum; // still wanted among the keys with this digit
        s_prefix = prefix | ((uint32_t)d << shift);
      }
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const bool all = s_all != 0;
  const uint32_t T = s_prefix, need_eq = s_need;
  // gather: every key above T in any order; the first need_eq keys equal to T in index order
  const uint32_t chunk = (vocab + SEL_THREADS - 1) / SEL_THREADS;
  const uint32_t i0 = tid * chunk, i1 = min(i0 + chunk, vocab);
  uint32_t eq = 0;
  for (uint32_t i = i0; i < i1; i++) {
    const uint32_t b = lb[i];
    if (is_nan_bits(b)) continue;
    const uint32_t key = order_key(b);
    if (all || key > T) {
      const uint32_t p = atomicAdd(&s_cnt, 1u);
      if (p < MAX_K) cand[p] = ((unsigned long long)key << 32) | (0xffffffffu - i);
    } else if (key == T) {
      eq++;
    }
  }
  scan[tid] = eq;
  __syncthreads();
  for (uint32_t off = 1; off < SEL_THREADS; off <<= 1) { // inclusive scan of the tie counts
    const uint32_t v = tid >= off ? scan[tid - off] : 0u;
    __syncthreads();
    scan[tid] += v;
    __syncthreads();
  }
  const uint32_t n_gt = s_cnt; // every thread has appended by the barriers above
  __syncthreads();
  if (!all && eq) {
    uint32_t rank = scan[tid] - eq; // ties before this thread's range
    for (uint32_t i = i0; i < i1 && rank < need_eq; i++) {
      const uint32_t b = lb[i];
      if (!is_nan_bits(b) && order_key(b) == T) {
        cand[n_gt + rank] = ((unsigned long long)T << 32) | (0xffffffffu - i);
        rank++;
      }
    }
  }
  __syncthreads();
  const uint32_t n_sel = all ? n_gt : n_gt + min(need_eq, scan[SEL_THREADS - 1]);
  // bitonic sort, descending, of the 1024 words (unused slots are 0 and sink to the end)
  for (uint32_t size = 2; size <= MAX_K; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      const uint32_t j = tid ^ stride;
      if (j > tid) {
        const unsigned long long a = cand[tid], b2 = cand[j];
        const bool desc = (tid & size) == 0;
        if (desc ? a < b2 : a > b2) {
          cand[tid] = b2;
          cand[j] = a;
        }
      }
      __syncthreads();
    }
  }
  if (tid < n_sel) {
    const unsigned long long c = cand[tid];
    out_idx[tid] = (int32_t)(0xffffffffu - (uint32_t)c);
    out_val[tid] = __uint_as_float(key_bits((uint32_t)(c >> 32)));
  }
  if (tid == 0) *out_n = n_sel;
}

} // namespace

// `logits` is a device row of `vocab` floats; `scratch` holds at least topk_scratch_bytes(vocab, k,
// n_recent) bytes. Results land in host memory when the call returns (it synchronises the stream).
size_t topk_scratch_bytes(uint32_t vocab, uint32_t k, uint32_t n_recent) {
  return ((size_t)vocab * 4 + 255) / 256 * 256 + ((size_t)n_recent * 4 + 255) / 256 * 256 + (size_t)k * 8 + 256;
}

int k_topk(FcDevice* dev, const float* logits, uint32_t vocab, uint32_t k, float rep_penalty, const int32_t* recent_host,
           uint32_t n_recent, void* scratch, int32_t* idx_out, float* val_out, uint32_t* n_out) {
  if (k == 0 || k > MAX_K) return fc_fail(dev, FC_ERR_UNSUPPORTED, "device top-k takes 1..%u candidates, not %u", MAX_K, k);
  if (!vocab) return fc_fail(dev, FC_ERR_SHAPE, "empty logits row");
  char* p = (char*)scratch;
  float* row = (float*)p;
  p += ((size_t)vocab * 4 + 255) / 256 * 256;
  int32_t* d_recent = (int32_t*)p;
  p += ((size_t)n_recent * 4 + 255) / 256 * 256;
  int32_t* d_idx = (int32_t*)p;
  float* d_val = (float*)(p + (size_t)k * 4);
  uint32_t* d_n = (uint32_t*)(p + (size_t)k * 8);
  const float* src = logits;
  if (rep_penalty != 1.0f && n_recent) {
    FC_CUDA(dev, cudaMemcpyAsync(row, logits, (size_t)vocab * 4, cudaMemcpyDeviceToDevice, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(d_recent, recent_host, (size_t)n_recent * 4, cudaMemcpyHostToDevice, dev->stream));
    FC_LAUNCH(dev, "sample_penalty", penalty_kernel<<<1, 32, 0, dev->stream>>>(row, vocab, d_recent, n_recent, rep_penalty));
    src = row;
  }
  FC_LAUNCH(dev, "sample_topk", topk_kernel<<<1, SEL_THREADS, 0, dev->stream>>>(src, vocab, k, d_idx, d_val, d_n));
  uint32_t n = 0;
  FC_CUDA(dev, cudaMemcpyAsync(&n, d_n, 4, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (n > k) return fc_fail(dev, FC_ERR_DEVICE, "top-k selection returned %u of %u candidates", n, k);
  if (n) {
    FC_CUDA(dev, cudaMemcpyAsync(idx_out, d_idx, (size_t)n * 4, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaMemcpyAsync(val_out, d_val, (size_t)n * 4, cudaMemcpyDeviceToHost, dev->stream));
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  }
  *n_out = n;
  return FC_OK;
}

FC_API int fc_topk_dev(FcDevice* dev, const float* logits_dev, uint32_t vocab, uint32_t k, float repetition_penalty,
                       const int32_t* recent, uint32_t n_recent, int32_t* idx_out, float* val_out, uint32_t* n_out) {
  if (!dev || !logits_dev || !idx_out || !val_out || !n_out || (n_recent && !recent)) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  void* scratch = nullptr;
  FC_CUDA(dev, cudaMalloc(&scratch, topk_scratch_bytes(vocab, k ? k : 1, n_recent)));
  const int rc = k_topk(dev, logits_dev, vocab, k, repetition_penalty, recent, n_recent, scratch, idx_out, val_out, n_out);
  cudaFree(scratch);
  return rc;
}

#include "model.cuh"

// Row `row` of the logits the model's last decode step left on the device (row i belongs to the i-th
// stream of that fc_model_feed_batch call; fc_model_feed and fc_model_prefill leave row 0).
FC_API int fc_model_topk(FcModel* m, uint32_t row, uint32_t k, float repetition_penalty, const int32_t* recent,
                         uint32_t n_recent, int32_t* idx_out, float* val_out, uint32_t* n_out) {
  if (!m || !idx_out || !val_out || !n_out || (n_recent && !recent)) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  cudaSetDevice(dev->ordinal);
  if (row >= m->max_streams) return fc_fail(dev, FC_ERR_RANGE, "logits row %u of %u", row, m->max_streams);
  if (m->n_shards != 1) return fc_fail(dev, FC_ERR_UNSUPPORTED, "top-k needs the whole head on this device");
  FC_TRY(arena_reserve(m, topk_scratch_bytes(m->vocab, k ? k : 1, n_recent)));
  void* scratch = arena_take(m, topk_scratch_bytes(m->vocab, k ? k : 1, n_recent));
  return k_topk(dev, m->logits + (size_t)row * m->vocab, m->vocab, k, repetition_penalty, recent, n_recent, scratch, idx_out,
                val_out, n_out);
}
