/*
 * ferrum_cuda.h - C ABI of libferrum_cuda.so, the sm_100a implementation of ferrum-gpu's
 * quantised-weight inference hot path (Q8_0 / Q4_0 packed-weight matrix products behind
 * KV-cached decode and full-sequence scoring, decode attention, and the fused elementwise ops
 * between them).
 *
 * This is what the one `unsafe` Rust crate (`ferrum_cuda`) binds, and what the C++ mirror in
 * ferrum_cuda.hpp and the Python ctypes harness call. Plain pointers and sizes only.
 *
 * Conventions
 *  - Every call returns an `int` status: FC_OK (0) or a negative FC_ERR_* code. Nothing aborts
 *    the process. A human-readable message for the last failure on a device is available from
 *    fc_last_error(); the messages for user errors are the reference's own strings.
 *  - "host" pointers are ordinary process memory. Entry points whose name ends in `_dev` take
 *    device pointers (memory on the GPU the handle belongs to) and enqueue on the handle's
 *    stream without synchronising.
 *  - Weight matrices are handed over exactly as the reference's host model structs hold them:
 *    f32, row-major `[in, out]` (ferrum_ref/src/models/llama/mod.rs:L100-L147). A bias or an
 *    optional tensor that is absent is a NULL pointer.
 *  - One caller per handle at a time; handles may be used from any thread.
 */
#ifndef FERRUM_CUDA_H
#define FERRUM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
enum {
  FC_OK = 0,
  FC_ERR_SHAPE = -1,        /* a length does not match its declared shape (ops/mod.rs:L31-L40) */
  FC_ERR_RANGE = -2,        /* token id >= vocab (ops/mod.rs:L45-L49): an error, never clamped  */
  FC_ERR_CONTEXT_FULL = -3, /* "context of N tokens is full" (models/llama/mod.rs:L354-L356)   */
  FC_ERR_OOM = -4,          /* allocation refused, or plan over budget before allocating       */
  FC_ERR_DEVICE = -5,       /* a CUDA call failed; sticky for the device handle                */
  FC_ERR_INJECTED = -6,     /* a launch refused by fc_debug_fail_after (test hook)             */
  FC_ERR_TIMEOUT = -7,      /* a bounded device-side wait ran out                              */
  FC_ERR_ARG = -8,          /* NULL handle / pointer, bad enum value                           */
  FC_ERR_UNSUPPORTED = -9   /* shape outside what a kernel was built for                       */
};

/* Stored precision of a weight matrix. Replaces ferrum_wgpu::ops::quant::QKind
 * (ferrum_wgpu/src/ops/quant.rs:L27-L44), restricted to the kinds on this path. */
/* FC_F16: plain f16 values, no scale, compute stays f32 - QKind::F16 (ops/quant.rs:L33-L36).
 * FC_FP8_E4M3 / FC_FP8_E5M2: one-byte floats with an f16 scale per 32, in Q8_0's block layout -
 * QKind::Fp8E4M3 / Fp8E5M2 (ops/quant.rs:L38-L41, codec ferrum_gguf/src/codec/fp8.rs).
 * FC_MXFP4: 4-bit E2M1 values with a power-of-two scale byte per 32, 17-byte blocks (ggml type 39) -
 * QKind::Fp4 (ops/quant.rs:L36-L37, codec ferrum_gguf/src/codec/mxfp4.rs).
 * FC_Q2_K: 2-bit values in super-blocks of 256 with 4-bit sub-block scales and mins, 84-byte blocks -
 * QKind::Q2K (ops/quant.rs:L42-L43, codec ferrum_gguf/src/codec/q2k.rs, decode blocks.rs:L199-L220). A width
 * that is whole 32s but not whole 256s is stored as Q4_0 instead (`effective`, ops/quant.rs:L134-L144). */
enum { FC_F32 = 0, FC_Q8_0 = 1, FC_Q4_0 = 2, FC_F16 = 3, FC_FP8_E4M3 = 4, FC_FP8_E5M2 = 5, FC_MXFP4 = 6, FC_Q2_K = 7 };

/* RoPE pairing, ferrum_ref/src/models/llama/ops.rs:L9-L15. */
enum { FC_ROPE_NORM = 0, FC_ROPE_NEOX = 1 };

/* Arithmetic of the batched (scoring / forward_all) matrix products.
 * FC_EXACT_F32: f32 FMA with f32 accumulation, same path as decode (parity <= 1e-5).
 * FC_TENSOR_F16: weights dequantised to fp16 in shared memory, fp16 activations, tcgen05 MMA with fp32
 * accumulators in tensor memory (parity <= 2e-2 max-abs per logit, 1e-3 mean NLL). */
enum { FC_EXACT_F32 = 0, FC_TENSOR_F16 = 1 };

typedef struct FcDevice FcDevice;
typedef struct FcQWeight FcQWeight;
typedef struct FcModel FcModel;
typedef struct FcGroup FcGroup;

/* ---- device ------------------------------------------------------------------------------ */
/* Replaces ferrum_wgpu::device::Gpu::open / GpuBackend::open (device/mod.rs:L98-L176,
 * ferrum_gpu_core/src/engine/gpu.rs:L18-L40). Opens CUDA device `ordinal`, creates the stream
 * every call on this handle uses. */
int fc_device_open(int ordinal, FcDevice** out);
int fc_device_close(FcDevice* dev);
/* Adapter name as Backend::name() reports it (engine/mod.rs:L259-L270). */
int fc_device_name(FcDevice* dev, char* buf, size_t buf_len);
/* Multiprocessor count and total memory, for the pre-flight plan check. */
int fc_device_props(FcDevice* dev, int* sm_count, uint64_t* total_mem_bytes);
/* Message of the most recent failing call on this device ("" if none). The pointer stays valid
 * until the next failing call on the same device. `dev` may be NULL: then it is the message of
 * the last failure that had no device (fc_device_open itself). */
const char* fc_last_error(FcDevice* dev);
/* The CUDA stream (a cudaStream_t) all work of this handle is enqueued on, and a full
 * synchronise of it. */
void* fc_device_stream(FcDevice* dev);
/* Waits for the stream and reports what the enqueued work could not report when it was launched: FC_ERR_TIMEOUT
 * when a kernel since the last synchronisation gave up one of its bounded waits (its results are incomplete;
 * the status is cleared), FC_ERR_DEVICE for a CUDA failure. Callers of the *_dev entry points, which return
 * before the work runs, learn of such a failure here. */
int fc_device_sync(FcDevice* dev);
/* Test hook: sets the status word a kernel raises when it gives up a wait, so that the reporting path can be
 * tested without a kernel that times out. */
int fc_debug_raise_status(FcDevice* dev, int value);
/* Kernels launched by this library on this device since it was opened. */
uint64_t fc_device_launch_count(FcDevice* dev);
/* Host-side fault injection, replaces Gpu::fail_after / sweep_faults
 * (ferrum_wgpu/src/device/runtime.rs:L214-L256): after `n_launches` more kernel launches every
 * further launch is refused with FC_ERR_INJECTED *before it reaches the device*; a negative
 * value disarms the hook. No GPU fault is ever produced. */
int fc_debug_fail_after(FcDevice* dev, int64_t n_launches);
/* Which kernel multiplies 1..8 rows of x by a packed matrix in exact-f32 mode: 0 = the library's own rule
 * (one row of a block format: the streamed tensor-core kernel; 2..8 rows: the small-batch mma.sync kernel),
 * 1 = the f32 FMA kernel, 2 = the small-batch mma.sync kernel. Measurement hook; results stay within the
 * exact path's tolerance whichever runs. */
int fc_debug_matvec_kernel(FcDevice* dev, int choice);
/* Per-kernel device timing, the counterpart of the reference's one-kernel-at-a-time profiler
 * (ferrum_wgpu/benches/profile_train.rs:L15-L25): while enabled every launch is bracketed by a pair
 * of CUDA events on the device's stream. The report is a JSON object
 * {"kernel": {"launches": n, "ms": total}, ...} of the launches since the previous report; it
 * synchronises the stream. Off by default. */
int fc_debug_profile(FcDevice* dev, int enable);
int fc_debug_profile_report(FcDevice* dev, char* buf, size_t buf_len);
/* The scoring path's causal attention on its own: the fused replacement of the reference's
 * attn_gqa_scores + attn_softmax + attn_gqa_pv dispatches (ferrum_wgpu/src/ops/llama.rs:L119-L146;
 * MHA when kv_heads == heads, ops/mod.rs:L108-L127). `qkv_host` is fp16 (IEEE binary16 bit patterns)
 * [n_seqs * t][(heads + 2 * kv_heads) * 64], each row q heads | k heads | v heads, head_dim 64;
 * `out_host` receives fp16 [n_seqs * t][heads * 64]. `variant`: 0 = what the model passes use,
 * 1 / 2 = the mma.sync kernel with one / two row tiles per warp, 3 = the tcgen05 / tensor-memory
 * kernel. After one warm-up launch `iters` launches are timed with CUDA events and their mean
 * (milliseconds) is written to `ms_out` when it is not NULL. Test and measurement hook. */
int fc_debug_attention_f16(FcDevice* dev, const uint16_t* qkv_host, uint32_t n_seqs, uint32_t t, uint32_t heads,
                           uint32_t kv_heads, uint16_t* out_host, int variant, int iters, float* ms_out);

/* ---- stand-alone quantised weights and products ------------------------------------------ */
/* Bytes of a GGUF tensor of `n_elems` elements (ferrum_gguf/src/codec/quant.rs:L17-L46);
 * 0 when the count does not fill whole 32-element blocks. */
size_t fc_block_bytes(int kind, size_t n_elems);

/* Quantise an f32 `[k, n]` ([in, out]) host matrix and keep it packed on the device. Replaces
 * ops::quant::upload_quantised = quantise_matrix + pack + upload
 * (ferrum_wgpu/src/ops/quant.rs:L238-L288). The encoder runs on the device and produces the
 * same blocks as ferrum_gguf::quant::encode (codec/quant.rs:L111-L133). `k` must be a multiple
 * of 32 unless `kind` is FC_F32. FC_F16 stores the transposed matrix as f16 (round to nearest even,
 * ferrum_gguf/src/f16.rs:L25-L53). */
int fc_qweight_create(FcDevice* dev, int kind, const float* w_in_out, uint32_t k, uint32_t n,
                      FcQWeight** out);
/* Same from GGUF block bytes: `n` rows of `k / 32` blocks of 34 (Q8_0, FP8), 18 (Q4_0) or 17 (MXFP4)
 * bytes, or of `k` f16 values (F16).
 * Replaces ops::quant::upload_qweight (ops/quant.rs:L266-L277). */
int fc_qweight_create_from_blocks(FcDevice* dev, int kind, const uint8_t* blocks, size_t n_bytes,
                                  uint32_t k, uint32_t n, FcQWeight** out);
int fc_qweight_destroy(FcQWeight* w);
/* kind / k / n / packed device bytes: QWeight::{kind,k,n,device_bytes} (ops/quant.rs:L158-L183). */
int fc_qweight_info(const FcQWeight* w, int* kind, uint32_t* k, uint32_t* n, uint64_t* dev_bytes);
/* The GGUF block bytes the device holds (`n` rows of `k/32` blocks), re-assembled from the
 * packed planes: the inverse of the upload repack. `out` has fc_block_bytes(kind, k*n) bytes. */
int fc_qweight_blocks(FcQWeight* w, uint8_t* out, size_t out_bytes);
/* The f32 values the kernels compute with, `[n, k]` row-major (row = output column), decoded on
 * the device; bit-identical to ferrum_gguf::quant::decode (codec/quant.rs:L50-L88). Replaces
 * ops::quant::dequantise_bytes (ops/quant.rs:L254-L264). */
int fc_dequant(FcQWeight* w, float* out_n_k, size_t out_elems);

/* `y[m, n] = x[m, k] * W` with host buffers (copies inside). Replaces ops::quant::linear_q
 * (ferrum_wgpu/src/ops/quant.rs:L326-L381). `mode` is FC_EXACT_F32 or FC_TENSOR_F16. */
int fc_qmatmul(FcQWeight* w, const float* x, uint32_t m, float* y, int mode);
/* The same on device buffers, enqueued on the device's stream, no synchronisation. `x_dev` and `y_dev` must be
 * 16-byte aligned (the kernels move 16-byte pieces; a misaligned pointer is refused with FC_ERR_ARG before any
 * launch). A kernel that gives up a bounded wait is reported by the next fc_device_sync, not here. */
int fc_qmatmul_dev(FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev, int mode);

/* The tensor-core product of fc_qmatmul_dev (mode FC_TENSOR_F16) for callers that must not trigger a
 * device allocation. This entry point has no counterpart in the reference. fc_qmatmul_dev keeps its
 * fp16 copy of `x` in a buffer it cudaMalloc's and grows per weight; that is unusable from inside a
 * stream capture, under a memory plan that was checked once and may not grow, or in a loop that
 * cannot afford the device-wide synchronisation an allocation implies. Here the copy lives in a
 * fixed 8 MiB array inside the library's device image (every GPU that loads the library carries it
 * until the process exits), so `m * k` may be at most 4 Mi elements (4 194 304); larger products are
 * refused with FC_ERR_SHAPE. `x_dev` and `y_dev` are the caller's. The first call on a device looks
 * up the array's device address; make that call before starting any stream capture. All calls share
 * the one array: two of them overlapping on the GPU (different streams or devices' handles on the
 * same GPU) race, and the array keeps the previous call's contents between calls. `x_dev` and `y_dev` must be
 * 16-byte aligned. While per-kernel timing (fc_debug_profile) is on, the library creates CUDA events around the
 * launches, which is an allocation of the driver's: leave it off where none is allowed. A kernel that gives up a
 * bounded wait is reported by the next fc_device_sync. */
int fc_qmatmul_dev_noalloc(FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev);

/* ---- resident models ---------------------------------------------------------------------- */
/* ferrum_ref::llama::Config + RopeScaling (ferrum_ref/src/models/llama/mod.rs:L24-L52,
 * ops.rs:L17-L35). */
typedef struct {
  uint32_t vocab, ctx, dim, heads, kv_heads, head_dim, layers, hidden, rope_dim;
  uint32_t rope_type; /* FC_ROPE_NORM | FC_ROPE_NEOX */
  float rope_base, eps;
  float rope_linear_factor;  /* 1.0 = none */
  uint32_t n_freq_factors;   /* 0 or rope_dim / 2 */
  const float* freq_factors; /* may be NULL when n_freq_factors == 0 */
  uint32_t tied;             /* head is the transposed embedding */
} FcLlamaConfig;

/* ferrum_ref::llama::Block (models/llama/mod.rs:L100-L128); biases NULL when absent. */
typedef struct {
  const float *attn_norm, *wq, *bq, *wk, *bk, *wv, *bv, *wo, *ffn_norm, *gate, *up, *down;
} FcLlamaBlock;

/* ferrum_ref::llama::Llama (models/llama/mod.rs:L130-L147). */
typedef struct {
  const float* tok;           /* [vocab, dim] */
  const FcLlamaBlock* blocks; /* cfg.layers of them */
  const float* out_norm;      /* [dim] */
  const float* head;          /* [dim, vocab] */
} FcLlamaWeights;

/* ferrum_ref::gpt2::Config (ferrum_ref/src/models/gpt2/mod.rs:L15-L30). */
typedef struct {
  uint32_t vocab, ctx, dim, heads, layers, hidden;
} FcGpt2Config;

/* ferrum_ref::gpt2::Block (models/gpt2/mod.rs:L62-L96). */
typedef struct {
  const float *ln1_g, *ln1_b, *wq, *bq, *wk, *bk, *wv, *bv, *wo, *bo, *ln2_g, *ln2_b, *w1, *b1,
      *w2, *b2;
} FcGpt2Block;

/* ferrum_ref::gpt2::Gpt2 (models/gpt2/mod.rs:L98-L114). */
typedef struct {
  const float* tok; /* [vocab, dim] */
  const float* pos; /* [ctx, dim] */
  const FcGpt2Block* blocks;
  const float *lnf_g, *lnf_b;
  const float* head; /* [dim, vocab] */
} FcGpt2Weights;

/* One weight tensor as the host hands it over. kind FC_F32: `data` is an f32 `[in, out]` row-major matrix (the layout
 * of ferrum_ref::llama::Llama, models/llama/mod.rs:L100-L147; a token table: `[vocab, dim]`). A block kind (FC_Q8_0,
 * FC_Q4_0, FC_F16, ...): `data` is the tensor's GGUF bytes exactly as ferrum_gguf::Gguf::tensor_bytes returns them
 * (ferrum_gguf/src/io/reader.rs:L298): `out` rows of `in / 32` blocks (a token table: `vocab` rows of `dim / 32`). */
typedef struct {
  const void* data;
  int kind;
} FcTensor;
typedef struct {
  const float* attn_norm;
  FcTensor wq;
  const float* bq;
  FcTensor wk;
  const float* bk;
  FcTensor wv;
  const float* bv;
  FcTensor wo;
  const float* ffn_norm;
  FcTensor gate, up, down;
} FcLlamaBlockT;
typedef struct {
  FcTensor tok;
  const FcLlamaBlockT* blocks;
  const float* out_norm;
  FcTensor head;
} FcLlamaTensors;
typedef struct {
  const float *ln1_g, *ln1_b;
  FcTensor wq;
  const float* bq;
  FcTensor wk;
  const float* bk;
  FcTensor wv;
  const float* bv;
  FcTensor wo;
  const float* bo;
  const float *ln2_g, *ln2_b;
  FcTensor w1;
  const float* b1;
  FcTensor w2;
  const float* b2;
} FcGpt2BlockT;
typedef struct {
  FcTensor tok;
  const float* pos;
  const FcGpt2BlockT* blocks;
  const float *lnf_g, *lnf_b;
  FcTensor head;
} FcGpt2Tensors;

/* Device bytes a resident model of this shape needs (weights, RoPE tables, KV caches for
 * `max_streams` streams, decode scratch). Replaces models::llama::plan
 * (ferrum_wgpu/src/models/llama/mod.rs:L108-L182). 0 for an invalid config. */
uint64_t fc_llama_plan_bytes(const FcLlamaConfig* cfg, int qkind, uint32_t max_streams);
uint64_t fc_gpt2_plan_bytes(const FcGpt2Config* cfg, int qkind, uint32_t max_streams);

/* Upload a model: quantise every eligible matrix to `qkind` (FC_F32 keeps f32), build RoPE
 * tables, zero the KV caches of `max_streams` independent streams. Replaces GpuLlama::new
 * (ferrum_wgpu/src/models/llama/mod.rs:L219-L314). `budget_bytes` (0 = the device's free
 * memory) refuses the plan *before* anything is allocated (L241-L243). */
int fc_llama_create(FcDevice* dev, const FcLlamaConfig* cfg, const FcLlamaWeights* w, int qkind,
                    uint32_t max_streams, uint64_t budget_bytes, FcModel** out);
/* Replaces GpuGpt2::new (ferrum_wgpu/src/models/gpt2.rs:L134-L190); `qkind` other than FC_F32
 * is new: the reference's resident GPT-2 is f32 only. */
int fc_gpt2_create(FcDevice* dev, const FcGpt2Config* cfg, const FcGpt2Weights* w, int qkind,
                   uint32_t max_streams, uint64_t budget_bytes, FcModel** out);
/* The same from tensors that may each be f32 or packed blocks: a block tensor is repacked on the device as it is -
 * what Lin::upload wants to do with a file's quantised tensors instead of dequantise -> transpose -> requantise
 * (ferrum_wgpu/src/models/llama/lin.rs:L30-L62) - and the result is bit-identical to the f32 route by the
 * reference's identity test (ferrum_wgpu/src/ops/quant/tests.rs:L89-L104); an f32 tensor is quantised to `qkind` as
 * in fc_llama_create. The tensors stacked into one weight (q, k, v; gate, up) must end up in the same format. A
 * token table given as blocks is decoded on the device (the table stays f32 there). */
int fc_llama_create_from_tensors(FcDevice* dev, const FcLlamaConfig* cfg, const FcLlamaTensors* w, int qkind,
                                 uint32_t max_streams, uint64_t budget_bytes, FcModel** out);
int fc_gpt2_create_from_tensors(FcDevice* dev, const FcGpt2Config* cfg, const FcGpt2Tensors* w, int qkind,
                                uint32_t max_streams, uint64_t budget_bytes, FcModel** out);
int fc_model_destroy(FcModel* m);

/* GpuLlama::{pos, reset} (models/llama/mod.rs:L331-L340) per stream. reset only rewinds the
 * position; the cache is overwritten as new tokens arrive. */
int fc_model_pos(FcModel* m, uint32_t stream_id, uint32_t* pos_out);
int fc_model_reset(FcModel* m, uint32_t stream_id);
/* vocab, ctx, max_streams, qkind and packed weight bytes of a resident model. */
int fc_model_info(FcModel* m, uint32_t* vocab, uint32_t* ctx, uint32_t* max_streams, int* qkind,
                  uint64_t* weight_bytes);

/* Consume one token at the stream's next position. Replaces GpuLlama::feed / GpuGpt2::feed
 * (models/llama/mod.rs:L352-L438, models/gpt2.rs:L192-L265). `logits_out` (vocab floats, host)
 * and `argmax_out` (first maximum, NaN never wins: ferrum_model/src/sampling.rs:L32-L40) may
 * each be NULL. A failed call leaves the position unchanged. */
int fc_model_feed(FcModel* m, uint32_t stream_id, int32_t token, float* logits_out,
                  int32_t* argmax_out);
/* One decode step for `n` distinct streams at once (new: the reference decodes batch 1 only,
 * serving/routes.rs:L301-L309). `logits_out` is `[n, vocab]` or NULL, `argmax_out` `[n]` or
 * NULL. */
int fc_model_feed_batch(FcModel* m, uint32_t n, const uint32_t* stream_ids, const int32_t* tokens,
                        float* logits_out, int32_t* argmax_out);
/* `steps` greedy decode steps of `n` streams in one call (new: the reference's generate loop reads every
 * token back before it feeds it, engine/mod.rs:L230-L240): step 0 feeds `first_tokens`, every further step
 * feeds the previous step's first-maximum picks, chained on the device without a host round trip.
 * `tokens_out` is `[steps][n]`: the picks of every step, exactly what `steps` calls of fc_model_feed_batch
 * with `argmax_out` would return. Every stream needs room for `steps` more positions. */
int fc_model_decode_greedy(FcModel* m, uint32_t n, const uint32_t* stream_ids, const int32_t* first_tokens,
                           uint32_t steps, int32_t* tokens_out);
/* Candidates for sampled decoding, selected on the device (new: the reference reads the whole logits
 * row back for every sampled token, engine/mod.rs:L230-L240). Applies the repetition penalty of
 * `sampling::sample` over `recent` (in order, a repeated token is penalised again,
 * ferrum_model/src/sampling.rs:L44-L54; 1.0 = off) and returns the at most `k` (1..1024) non-NaN logits
 * that `sample` would keep for top_k = k, in its order: descending by f32::total_cmp, ties lower index
 * first (sampling.rs:L57-L66). `idx_out` / `val_out` hold `k` entries, `n_out` receives the count
 * (fewer than k only when the row has fewer non-NaN logits). The caller runs its own softmax / top_p /
 * draw over these candidates, which reproduces `sample(row, top_k = k, ...)` exactly. The row is row
 * `row` of the last fc_model_feed_batch call (row 0 after fc_model_feed; after fc_model_prefill only if
 * that call was asked for logits or the argmax). fc_topk_dev does the same for any device row. */
int fc_model_topk(FcModel* m, uint32_t row, uint32_t k, float repetition_penalty, const int32_t* recent,
                  uint32_t n_recent, int32_t* idx_out, float* val_out, uint32_t* n_out);
int fc_topk_dev(FcDevice* dev, const float* logits_dev, uint32_t vocab, uint32_t k, float repetition_penalty,
                const int32_t* recent, uint32_t n_recent, int32_t* idx_out, float* val_out, uint32_t* n_out);
/* Feed `n` prompt tokens of one stream in one batched pass (new: the reference feeds a prompt
 * token by token, engine/mod.rs:L226-L229). FC_EXACT_F32: equivalent to n calls of fc_model_feed, at any
 * position of the stream. FC_TENSOR_F16: the prompt runs through the scoring kernels (fp16 operands, f32
 * accumulation; logits within the scoring tolerance) and its k and v land in the stream's f32 cache, so
 * decode continues with fc_model_feed; the stream must be empty. Returns the last position's logits /
 * argmax when asked. */
int fc_model_prefill(FcModel* m, uint32_t stream_id, const int32_t* ids, uint32_t n,
                     float* logits_out, int32_t* argmax_out, int mode);
/* Stateless full causal forward, every position's logits `[n, vocab]`. Replaces
 * GpuLlama::forward_all / GpuGpt2::forward_all (models/llama/forward.rs:L13-L17). */
int fc_model_forward_all(FcModel* m, const int32_t* ids, uint32_t n, float* logits_out, int mode);
/* Score `n_seqs` sequences of `seq_len` ids each: for each i < seq_len-1 the log-probability of
 * ids[i+1] given ids[..=i] and whether it is the first argmax. Replaces GpuLlama::score
 * (models/llama/forward.rs:L74-L88) + ops::score (ops/mod.rs:L158-L175), batched over
 * sequences. `logprob_out` / `greedy_out` are `[n_seqs, seq_len-1]` (nullable);
 * `nll_sum_out[n_seqs]` is each sequence's -sum of log-probabilities accumulated in f64 in
 * ascending position (serving/decoder.rs:L69-L83). */
int fc_model_score(FcModel* m, const int32_t* ids, uint32_t n_seqs, uint32_t seq_len, int mode,
                   float* logprob_out, uint8_t* greedy_out, double* nll_sum_out);
/* Scoring with the ids already on the device and results left there: the timed kernel-only
 * region of the benchmark. `ids_dev` is `[n_seqs, seq_len]` int32, `nll_sum_dev[n_seqs]` f64;
 * `logprob_dev` / `greedy_dev` nullable. Enqueues without synchronising. */
int fc_model_score_dev(FcModel* m, const int32_t* ids_dev, uint32_t n_seqs, uint32_t seq_len,
                       int mode, float* logprob_dev, uint8_t* greedy_dev, double* nll_sum_dev);

/* ---- vocabulary-split head (multi-GPU scoring) --------------------------------------------
 * Precedent: Lin::Sharded splits a `[k, n]` weight by output columns, each block quantised and
 * multiplied on its own (ferrum_wgpu/src/models/llama/lin.rs:L41-L53,L76-L90). Here the blocks
 * live on different GPUs of one box. Rank r of `n_shards` keeps head rows
 * [r*ceil(V/n_shards), min(V, (r+1)*ceil(V/n_shards))). */
/* Restrict the resident model's head to one vocabulary shard (call once, after create). */
int fc_model_set_head_shard(FcModel* m, uint32_t shard, uint32_t n_shards);
/* Trunk only: final-norm hidden states of every position, `[n_seqs*seq_len, dim]` bf16 (mode
 * FC_TENSOR_F16) or f32 (FC_EXACT_F32), written to `hidden_dev`. */
int fc_model_trunk_dev(FcModel* m, const int32_t* ids_dev, uint32_t n_seqs, uint32_t seq_len,
                       int mode, void* hidden_dev);
/* Head over this rank's vocabulary shard for `rows` hidden rows: per row the local maximum, the
 * local sum of exp(logit - local max), the target's logit if this shard owns the target (else
 * -inf), and the local first argmax as a global vocabulary index: `partial_dev[rows][4]` f32
 * (the index is stored as a float-exact integer < 2^24). */
int fc_model_head_partial_dev(FcModel* m, const void* hidden_dev, const int32_t* targets_dev,
                              uint32_t rows, int mode, float* partial_dev);
/* Combine `n_shards` partials (all-gathered into `[n_shards][rows][4]`) into log-probabilities,
 * greedy flags and per-sequence NLL sums; rows = n_seqs * rows_per_seq. */
int fc_score_combine_dev(FcDevice* dev, const float* partials_dev, uint32_t n_shards,
                         const int32_t* targets_dev, uint32_t n_seqs, uint32_t rows_per_seq,
                         float* logprob_dev, uint8_t* greedy_dev, double* nll_sum_dev);

/* ---- scoring callers: unequal lengths and sliding windows ------------------------------------ */
/* Score `n_seqs` sequences of different lengths in batched passes (new: the server scores its concurrent
 * requests one after another, ferrum_gpu_core/src/serving/routes.rs:L301-L309, limits.rs:L32). Sequence s is
 * ids[offsets[s] .. offsets[s + 1]) (2 .. ctx + 1 ids; `offsets` has n_seqs + 1 entries). Per sequence the
 * results are those of fc_model_score on it alone; they are packed: sequence s owns entries
 * offsets[s] - s .. offsets[s + 1] - (s + 1) of `logprob_out` / `greedy_out` (nullable), and
 * `nll_sum_out[s]` (nullable) is its -sum of log-probabilities in f64, ascending position. */
int fc_model_score_ragged(FcModel* m, const int32_t* ids, const uint32_t* offsets, uint32_t n_seqs, int mode,
                          float* logprob_out, uint8_t* greedy_out, double* nll_sum_out);
/* The window partition of serving::score::token_logprobs (ferrum_gpu_core/src/serving/score.rs:L27-L49) for a
 * stream of `n_ids` ids scored from target index `from` (clamped to 1) with a context of `ctx` positions:
 * window w is ids[start[w] .. end[w]) (at most ctx + 1 ids) and contributes targets first[w] .. end[w]; every
 * target is scored exactly once with at least half a context of history. Returns the number of windows and
 * fills at most `cap` entries of each (nullable) array. Pure host arithmetic. */
uint32_t fc_score_windows(uint32_t n_ids, uint32_t from, uint32_t ctx, uint32_t* start_out, uint32_t* end_out,
                          uint32_t* first_out, uint32_t cap);
/* token_logprobs for `n_streams` id streams at once: stream j is ids[offsets[j] .. offsets[j + 1]), scored
 * from target index from[j] (`from` NULL = 1 everywhere). All windows of all streams go through one
 * fc_model_score_ragged batch; `logprob_out[j]` is the f64 sum of log p over the stream's targets in ascending
 * order, `n_tokens_out[j]` their count, `greedy_out[j]` 1 when every one was the first argmax
 * (Score { logprob, n_tokens, greedy }, score.rs:L9-L17; a stream with nothing to score gives (0, 0, 1)). */
int fc_model_token_logprobs(FcModel* m, const int32_t* ids, const uint32_t* offsets, const uint32_t* from,
                            uint32_t n_streams, int mode, double* logprob_out, uint64_t* n_tokens_out,
                            uint8_t* greedy_out);

/* ---- groups of GPUs (multi-GPU scoring behind the ABI) ----------------------------------------
 * A group is `world` ranks, each with its own open device and resident model, in one or several processes
 * (one thread per rank inside a process). It owns its NCCL communicators; NCCL is loaded at run time
 * (libnccl.so.2), so everything else in this header works without it. With `vocab_shards` == 1 every rank
 * holds the whole head and scores sequences rank, rank + world, ...; with more, consecutive ranks form groups
 * that split the head by vocabulary rows (Lin::Sharded's column blocks on different GPUs,
 * ferrum_wgpu/src/models/llama/lin.rs:L41-L53,L76-L90) and exchange final hidden states and per-row
 * (max, sum-exp, target logit, first argmax) partials through local HBM. */
/* Sequences part, part + parts, ... below n_seqs (the rule both partitions use). Returns their count. */
uint32_t fc_group_sequences(uint32_t n_seqs, uint32_t part, uint32_t parts, uint32_t* out, uint32_t cap);
/* The rendezvous token (128 bytes): made by one rank, carried to the others by the caller. */
int fc_group_unique_id(uint8_t* id_out, size_t id_bytes);
/* Join the group as `rank` of `world`. Collective: every rank calls it with the same token. With
 * vocab_shards > 1 the model's head is restricted to this rank's shard (fc_model_set_head_shard). */
int fc_group_create(FcDevice* dev, FcModel* model, uint32_t rank, uint32_t world, uint32_t vocab_shards,
                    const uint8_t* id, size_t id_bytes, FcGroup** out);
int fc_group_destroy(FcGroup* g);
/* Total NLL of each of `n_seqs` sequences of `seq_len` ids (host, the same array on every rank);
 * `nll_sum_out[n_seqs]` is filled on every rank. Collective. */
int fc_group_score(FcGroup* g, const int32_t* ids, uint32_t n_seqs, uint32_t seq_len, int mode, double* nll_sum_out);
/* Device milliseconds of the last fc_group_score call's exchanges: [0] all-gather of hidden states, [1] of the
 * partials (0 without a split head), [2] the all-reduce of the NLL sums. */
int fc_group_last_exchange_ms(FcGroup* g, float* ms_out);

#ifdef __cplusplus
}
#endif
#endif /* FERRUM_CUDA_H */
