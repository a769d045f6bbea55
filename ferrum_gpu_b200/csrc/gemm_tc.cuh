// Host interface of the f16 tensor-core product (gemm_tc.cu) and its companions (ops_tc.cu).
#pragma once
#include <cuda.h>

#include "common.cuh"

// What the epilogue does with the f32 accumulator tile.
enum {
  EPI_F32 = 0,    // out_f32[m][ldo]  = acc + bias
  EPI_F16 = 1,   // out_f16[m][ldo] = f16(act(acc + bias))
  EPI_RESID = 2,  // out_f32[m][ldo] += acc + bias          (residual stream, in place)
  EPI_SWIGLU = 3, // out_f16[m][n/2] = f16(silu(gate) * up); weight rows alternate gate, up
  EPI_LSE = 4     // partial[tile][m][4] = (max, sum exp, target logit | -inf, first argmax)
};

struct TcArgs {
  uint32_t m = 0, n = 0, k = 0;
  const float* bias = nullptr;
  float* out_f32 = nullptr;
  __half* out_f16 = nullptr;
  uint32_t ldo = 0;
  int act = ACT_NONE;
  const int32_t* targets = nullptr;
  uint32_t v0 = 0;
  float* partial = nullptr;
  int* err_flag = nullptr;
  uint32_t out_tma = 0; // (set by the launch code) results leave through shared memory and TMA
};

constexpr uint32_t TC_BM = 256, TC_BN = 128, TC_BK = 64; // weight rows per tile (TC_BN), K slice; TC_BM: activation rows of the head's tile

// y = a[m][k] (f16, row-major, device) . W^T with the epilogue `epi`. k % 64 == 0.
int k_qgemm_tc_f16(FcDevice* dev, const QMat& w, const __half* a, int epi, TcArgs args);
// Reads and clears the device-side error word the tensor kernels report bounded-wait failures in.
int tc_check_errors(FcDevice* dev);

// ops_tc.cu
int k_f32_to_f16(FcDevice* dev, const float* x, size_t n, __half* y);
int k_norm_f16(FcDevice* dev, bool layernorm, const float* x, const float* g, const float* b, uint32_t rows, uint32_t d,
                float eps, __half* y);
int k_rope_f16(FcDevice* dev, __half* qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                const float* cos, const float* sin, uint32_t rope_dim, uint32_t type, const int32_t* positions);
int k_kv_store_f16(FcDevice* dev, const __half* qkv, uint32_t t, uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t slot,
                   uint32_t start, uint32_t ctx, float* k_cache, float* v_cache);
int k_attn_causal_f16(FcDevice* dev, const __half* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads,
                       uint32_t kv_heads, uint32_t hd, __half* out);
int k_partial_merge(FcDevice* dev, const float* tiles, uint32_t n_tiles, uint32_t rows, float* out);
int k_permute_rows(FcDevice* dev, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t row_bytes, uint32_t half,
                   uint32_t group);
