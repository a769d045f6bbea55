// Scoring over the GPUs of one box behind the C ABI: every rank (a process, or a thread of one process)
// holds an open device and a resident model and joins a group that owns its NCCL communicators.
//
// Sequences are independent (so are the server's sliding windows, serving/score.rs:L27-L49): with one
// vocabulary shard every rank scores sequences rank, rank + world, ... on its replica and the per-sequence
// NLL sums meet in one all-reduce over disjoint slots. With `vocab_shards` > 1 the ranks form
// world / vocab_shards sequence groups of vocab_shards ranks each; the precedent is Lin::Sharded, which splits
// a [k, n] weight by output columns, each block multiplied on its own
// (ferrum_wgpu/src/models/llama/lin.rs:L41-L53,L76-L90) - here the blocks of the head live on different GPUs.
// Inside a group the trunk is sequence-parallel, the final hidden states are all-gathered into local HBM,
// every rank runs the fused head over its vocabulary rows, and the per-row (max, sum-exp, target logit, first
// argmax) partials are all-gathered and merged. Remote data always lands in local memory, through NCCL, before
// a kernel reads it: no kernel is given a peer pointer and nothing here uses a multicast load.
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library loads, and every single-GPU entry point
// works, on a machine without it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "model.cuh"

namespace {

struct Nccl {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!n.lib) return;
    auto sym = [&](const char* name) { return dlsym(n.lib, name); };
    n.GetUniqueId = (decltype(n.GetUniqueId))sym("ncclGetUniqueId");
    n.CommInitRank = (decltype(n.CommInitRank))sym("ncclCommInitRank");
    n.CommSplit = (decltype(n.CommSplit))sym("ncclCommSplit");
    n.CommDestroy = (decltype(n.CommDestroy))sym("ncclCommDestroy");
    n.AllGather = (decltype(n.AllGather))sym("ncclAllGather");
    n.AllReduce = (decltype(n.AllReduce))sym("ncclAllReduce");
    n.GetErrorString = (decltype(n.GetErrorString))sym("ncclGetErrorString");
    n.ok = n.GetUniqueId && n.CommInitRank && n.CommSplit && n.CommDestroy && n.AllGather && n.AllReduce && n.GetErrorString;
  });
  return n;
}

#define FC_NCCL(dev, expr)                                                                       \
  do {                                                                                           \
    ncclResult_t _r = (expr);                                                                    \
    if (_r != ncclSuccess) return fc_fail((dev), FC_ERR_DEVICE, "%s: %s", #expr, nccl().GetErrorString(_r)); \
  } while (0)

// out[idx[i]] = src[i]
__global__ void scatter_f64_kernel(const double* __restrict__ src, const uint32_t* __restrict__ idx, uint32_t n,
                                   double* __restrict__ out) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[idx[i]] = src[i];
}

size_t al(size_t v) { return (v + 255) & ~(size_t)255; }

} // namespace

struct FcGroup {
  FcDevice* dev = nullptr;
  FcModel* model = nullptr;
  uint32_t rank = 0, world = 1, vocab_shards = 1;
  ncclComm_t comm = nullptr;   // all ranks
  ncclComm_t shard_comm = nullptr; // the ranks that share this rank's sequences (vocab_shards of them)
  void* ws = nullptr;          // device workspace of fc_group_score, grown on demand
  size_t ws_bytes = 0;
  // device time of the last fc_group_score call's two exchanges (hidden states, partials) and of the final
  // all-reduce, measured with events on the device's stream
  cudaEvent_t ev[6] = {};
  float last_ms[3] = {0, 0, 0};
};

// Which sequences a rank scores: `rank, rank + world, ...` (one shard), or for sequence group g of `groups`:
// g, g + groups, ...
FC_API uint32_t fc_group_sequences(uint32_t n_seqs, uint32_t part, uint32_t parts, uint32_t* out, uint32_t cap) {
  uint32_t n = 0;
  if (parts == 0) return 0;
  for (uint32_t s = part; s < n_seqs; s += parts, n++)
    if (out && n < cap) out[n] = s;
  return n;
}

// The rendezvous token: made by one rank, handed to every rank by the caller's own means (a broadcast of its
// process group, a file, a pipe), then passed to fc_group_create by all of them.
FC_API int fc_group_unique_id(uint8_t* id_out, size_t id_bytes) {
  if (!id_out || id_bytes < sizeof(ncclUniqueId)) return FC_ERR_ARG;
  if (!nccl().ok) return fc_fail(nullptr, FC_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  const ncclResult_t r = nccl().GetUniqueId(&id);
  if (r != ncclSuccess) return fc_fail(nullptr, FC_ERR_DEVICE, "ncclGetUniqueId: %s", nccl().GetErrorString(r));
  memcpy(id_out, &id, sizeof id);
  return FC_OK;
}

FC_API int fc_group_create(FcDevice* dev, FcModel* model, uint32_t rank, uint32_t world, uint32_t vocab_shards,
                           const uint8_t* id, size_t id_bytes, FcGroup** out) {
  if (!dev || !model || !out || !id) return FC_ERR_ARG;
  *out = nullptr;
  if (model->dev != dev) return fc_fail(dev, FC_ERR_ARG, "the model lives on another device handle");
  if (world == 0 || rank >= world) return fc_fail(dev, FC_ERR_ARG, "rank %u of %u", rank, world);
  if (vocab_shards == 0 || world % vocab_shards)
    return fc_fail(dev, FC_ERR_ARG, "%u ranks cannot form groups of %u vocabulary shards", world, vocab_shards);
  if (id_bytes < sizeof(ncclUniqueId)) return fc_fail(dev, FC_ERR_ARG, "the rendezvous token has %zu bytes, not %zu", id_bytes, sizeof(ncclUniqueId));
  if (!nccl().ok) return fc_fail(dev, FC_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded");
  cudaSetDevice(dev->ordinal);
  FcGroup* g = new FcGroup();
  g->dev = dev, g->model = model, g->rank = rank, g->world = world, g->vocab_shards = vocab_shards;
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof uid);
  ncclResult_t r = nccl().CommInitRank(&g->comm, (int)world, uid, (int)rank);
  if (r == ncclSuccess && vocab_shards > 1) // colour = sequence group, key = shard
    r = nccl().CommSplit(g->comm, (int)(rank / vocab_shards), (int)(rank % vocab_shards), &g->shard_comm, nullptr);
  if (r != ncclSuccess) {
    const int rc = fc_fail(dev, FC_ERR_DEVICE, "joining the group failed: %s", nccl().GetErrorString(r));
    if (g->comm) nccl().CommDestroy(g->comm);
    delete g;
    return rc;
  }
  if (vocab_shards > 1) {
    const int rc = fc_model_set_head_shard(model, rank % vocab_shards, vocab_shards);
    if (rc != FC_OK) {
      nccl().CommDestroy(g->shard_comm);
      nccl().CommDestroy(g->comm);
      delete g;
      return rc;
    }
  }
  for (auto& e : g->ev) cudaEventCreate(&e);
  *out = g;
  return FC_OK;
}

FC_API int fc_group_destroy(FcGroup* g) {
  if (!g) return FC_OK;
  cudaSetDevice(g->dev->ordinal);
  cudaStreamSynchronize(g->dev->stream);
  if (g->shard_comm) nccl().CommDestroy(g->shard_comm);
  if (g->comm) nccl().CommDestroy(g->comm);
  if (g->ws) cudaFree(g->ws);
  for (auto& e : g->ev)
    if (e) cudaEventDestroy(e);
  delete g;
  return FC_OK;
}

// Device milliseconds of the last fc_group_score call: [0] all-gather of hidden states, [1] all-gather of
// partials (both 0 without a split head), [2] the all-reduce of the NLL sums.
FC_API int fc_group_last_exchange_ms(FcGroup* g, float* ms_out) {
  if (!g || !ms_out) return FC_ERR_ARG;
  for (int i = 0; i < 3; i++) ms_out[i] = g->last_ms[i];
  return FC_OK;
}

// Total NLL of every sequence of `ids` ([n_seqs][seq_len] int32 on the host, the same array on every rank);
// `nll_sum_out[n_seqs]` (f64, host) is filled on every rank. Every rank of the group must make the call.
FC_API int fc_group_score(FcGroup* g, const int32_t* ids, uint32_t n_seqs, uint32_t seq_len, int mode, double* nll_sum_out) {
  if (!g || !ids || !nll_sum_out) return FC_ERR_ARG;
  FcDevice* dev = g->dev;
  FcModel* m = g->model;
  cudaSetDevice(dev->ordinal);
  if (seq_len < 2) return fc_fail(dev, FC_ERR_SHAPE, "scoring needs at least 2 tokens");
  if (seq_len - 1 > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", seq_len - 1, m->ctx);
  if (mode != FC_EXACT_F32 && mode != FC_TENSOR_F16) return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
  for (size_t i = 0; i < (size_t)n_seqs * seq_len; i++)
    if (ids[i] < 0 || (uint32_t)ids[i] >= m->vocab)
      return fc_fail(dev, FC_ERR_RANGE, "index %d is out of range for %u entries", ids[i], m->vocab);
  if (n_seqs == 0) return FC_OK;
  const uint32_t t = seq_len - 1, vs = g->vocab_shards;
  const uint32_t groups = g->world / vs, group_id = g->rank / vs, shard = g->rank % vs;
  // this rank's sequences: of the whole job (one shard), or its slice of its group's sequences, padded with
  // repeats of the group's last sequence so that every rank of the group gathers equal counts
  std::vector<uint32_t> group_seqs(fc_group_sequences(n_seqs, group_id, groups, nullptr, 0));
  fc_group_sequences(n_seqs, group_id, groups, group_seqs.data(), (uint32_t)group_seqs.size());
  const uint32_t per = vs > 1 ? (uint32_t)((group_seqs.size() + vs - 1) / vs) : (uint32_t)group_seqs.size();
  std::vector<uint32_t> padded = group_seqs;
  if (!padded.empty()) padded.resize((size_t)per * vs, group_seqs.back());
  const uint32_t rows_mine = per * t, rows_all = vs * per * t;
  const size_t hid_el = mode == FC_TENSOR_F16 ? 2 : 4;
  // workspace: out[n_seqs] f64 | ids of my sequences | nll | idx | (split head:) hidden, all hidden, targets,
  // partial, all partials, logprob
  size_t need = al((size_t)n_seqs * 8) + al((size_t)per * seq_len * 4) + al((size_t)vs * per * 8) + al((size_t)vs * per * 4);
  if (vs > 1)
    need += al((size_t)rows_mine * m->dim * hid_el) + al((size_t)rows_all * m->dim * hid_el) + al((size_t)rows_all * 4) +
            al((size_t)rows_all * 16) + al((size_t)vs * rows_all * 16) + al((size_t)rows_all * 4);
  if (need > g->ws_bytes) {
    FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (g->ws) cudaFree(g->ws);
    g->ws = nullptr, g->ws_bytes = 0;
    FC_CUDA(dev, cudaMalloc(&g->ws, need));
    g->ws_bytes = need;
  }
  uint8_t* p = (uint8_t*)g->ws;
  auto take = [&](size_t bytes) {
    void* r = p;
    p += al(bytes);
    return r;
  };
  double* d_out = (double*)take((size_t)n_seqs * 8);
  int32_t* d_ids = (int32_t*)take((size_t)per * seq_len * 4);
  double* d_nll = (double*)take((size_t)vs * per * 8);
  uint32_t* d_idx = (uint32_t*)take((size_t)vs * per * 4);
  FC_CUDA(dev, cudaMemsetAsync(d_out, 0, (size_t)n_seqs * 8, dev->stream));
  void* pin;
  g->last_ms[0] = g->last_ms[1] = g->last_ms[2] = 0.0f;
  bool timed_split = false;
  if (per > 0) {
    const size_t pin_bytes = al((size_t)per * seq_len * 4) + al((size_t)vs * per * 4) + al((size_t)rows_all * 4);
    FC_TRY(fc_pinned(dev, pin_bytes, &pin));
    int32_t* h_ids = (int32_t*)pin;
    uint32_t* h_idx = (uint32_t*)((uint8_t*)pin + al((size_t)per * seq_len * 4));
    int32_t* h_tgt = (int32_t*)((uint8_t*)h_idx + al((size_t)vs * per * 4));
    if (vs == 1) {
      for (uint32_t i = 0; i < per; i++) {
        memcpy(h_ids + (size_t)i * seq_len, ids + (size_t)group_seqs[i] * seq_len, (size_t)seq_len * 4);
        h_idx[i] = group_seqs[i];
      }
      FC_CUDA(dev, cudaMemcpyAsync(d_ids, h_ids, (size_t)per * seq_len * 4, cudaMemcpyHostToDevice, dev->stream));
      FC_CUDA(dev, cudaMemcpyAsync(d_idx, h_idx, (size_t)per * 4, cudaMemcpyHostToDevice, dev->stream));
      FC_CUDA(dev, cudaStreamSynchronize(dev->stream)); // (the pinned buffer is the device handle's: the model calls reuse it)
      FC_TRY(fc_model_score_dev(m, d_ids, per, seq_len, mode, nullptr, nullptr, d_nll));
      FC_LAUNCH(dev, "scatter_nll", scatter_f64_kernel<<<(per + 255) / 256, 256, 0, dev->stream>>>(d_nll, d_idx, per, d_out));
    } else {
      void* hidden = take((size_t)rows_mine * m->dim * hid_el);
      void* all_hidden = take((size_t)rows_all * m->dim * hid_el);
      int32_t* d_tgt = (int32_t*)take((size_t)rows_all * 4);
      float* partial = (float*)take((size_t)rows_all * 16);
      float* all_partial = (float*)take((size_t)vs * rows_all * 16);
      float* d_lp = (float*)take((size_t)rows_all * 4);
      // inputs of my sequences (the first t ids of each), targets of all of the group's (ids 1..)
      for (uint32_t i = 0; i < per; i++) memcpy(h_ids + (size_t)i * t, ids + (size_t)padded[shard * per + i] * seq_len, (size_t)t * 4);
      for (uint32_t i = 0; i < vs * per; i++) {
        memcpy(h_tgt + (size_t)i * t, ids + (size_t)padded[i] * seq_len + 1, (size_t)t * 4);
        h_idx[i] = padded[i];
      }
      FC_CUDA(dev, cudaMemcpyAsync(d_ids, h_ids, (size_t)per * t * 4, cudaMemcpyHostToDevice, dev->stream));
      FC_CUDA(dev, cudaMemcpyAsync(d_tgt, h_tgt, (size_t)rows_all * 4, cudaMemcpyHostToDevice, dev->stream));
      FC_CUDA(dev, cudaMemcpyAsync(d_idx, h_idx, (size_t)vs * per * 4, cudaMemcpyHostToDevice, dev->stream));
      FC_CUDA(dev, cudaStreamSynchronize(dev->stream)); // (the pinned buffer is the device handle's: the model calls reuse it)
      FC_TRY(fc_model_trunk_dev(m, d_ids, per, t, mode, hidden));
      cudaEventRecord(g->ev[0], dev->stream);
      FC_NCCL(dev, nccl().AllGather(hidden, all_hidden, (size_t)rows_mine * m->dim * hid_el, ncclUint8, g->shard_comm, dev->stream));
      cudaEventRecord(g->ev[1], dev->stream);
      FC_TRY(fc_model_head_partial_dev(m, all_hidden, d_tgt, rows_all, mode, partial));
      cudaEventRecord(g->ev[2], dev->stream);
      FC_NCCL(dev, nccl().AllGather(partial, all_partial, (size_t)rows_all * 4, ncclFloat32, g->shard_comm, dev->stream));
      cudaEventRecord(g->ev[3], dev->stream);
      timed_split = true;
      FC_TRY(fc_score_combine_dev(dev, all_partial, vs, d_tgt, vs * per, t, d_lp, nullptr, d_nll));
      if (shard == 0) // one rank of the group reports its sequences (repeats of the last one write the same value)
        FC_LAUNCH(dev, "scatter_nll",
                  scatter_f64_kernel<<<(vs * per + 255) / 256, 256, 0, dev->stream>>>(d_nll, d_idx, vs * per, d_out));
    }
  }
  cudaEventRecord(g->ev[4], dev->stream);
  if (g->world > 1) FC_NCCL(dev, nccl().AllReduce(d_out, d_out, n_seqs, ncclFloat64, ncclSum, g->comm, dev->stream)); // disjoint slots: a sum is a gather
  cudaEventRecord(g->ev[5], dev->stream);
  FC_CUDA(dev, cudaMemcpyAsync(nll_sum_out, d_out, (size_t)n_seqs * 8, cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (mode == FC_TENSOR_F16) FC_TRY(tc_check_errors(dev));
  if (timed_split) {
    cudaEventElapsedTime(&g->last_ms[0], g->ev[0], g->ev[1]);
    cudaEventElapsedTime(&g->last_ms[1], g->ev[2], g->ev[3]);
  }
  cudaEventElapsedTime(&g->last_ms[2], g->ev[4], g->ev[5]);
  return FC_OK;
}
