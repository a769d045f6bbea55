// The scoring callers above the resident model: sequences of unequal length in one batched pass
// (the server scores its concurrent requests one after another, ferrum_gpu_core/src/serving/routes.rs:L301-L309)
// and the sliding-window partition of a long id stream (serving/score.rs:L27-L49). Host logic only: the
// arithmetic is fc_model_score's.
#include <algorithm>
#include <numeric>
#include <vector>

#include "model.cuh"

// serving/score.rs:L27-L49 (`token_logprobs`): the windows that score ids[from..] with a context of
// `ctx` positions. Window w covers ids[start[w] .. end[w]) (at most ctx + 1 ids) and contributes the
// targets first[w] .. end[w]; the first window starts at 0, every later one half a context before its
// first target. Returns the number of windows; fills at most `cap` entries.
FC_API uint32_t fc_score_windows(uint32_t n_ids, uint32_t from, uint32_t ctx, uint32_t* start_out, uint32_t* end_out,
                                 uint32_t* first_out, uint32_t cap) {
  if (from < 1) from = 1;               // L28
  if (from >= n_ids || ctx == 0) return 0; // L29-L31
  const uint32_t t = ctx;
  const uint32_t half = t / 2 > 1 ? t / 2 : 1; // L33
  uint32_t n = 0, next = from;
  while (next < n_ids) {
    const uint32_t start = next <= t ? 0 : next - half;                    // L37
    const uint64_t e = (uint64_t)start + t + 1;                            // L38
    const uint32_t end = e < n_ids ? (uint32_t)e : n_ids;
    if (n < cap) {
      if (start_out) start_out[n] = start;
      if (end_out) end_out[n] = end;
      if (first_out) first_out[n] = next;
    }
    n++;
    next = end; // L46
  }
  return n;
}

// Sequences of unequal length: sequence s is ids[offsets[s] .. offsets[s + 1]). They are scored in groups of
// similar length, each group padded with id 0 to its longest member - causal attention keeps a padded tail from
// touching the positions before it - and one batched pass per group. Results are packed: sequence s owns
// offsets[s] - s .. offsets[s + 1] - (s + 1) of logprob_out / greedy_out (len - 1 entries each).
FC_API int fc_model_score_ragged(FcModel* m, const int32_t* ids, const uint32_t* offsets, uint32_t n_seqs, int mode,
                                 float* logprob_out, uint8_t* greedy_out, double* nll_sum_out) {
  if (!m || !ids || !offsets) return FC_ERR_ARG;
  FcDevice* dev = m->dev;
  if (n_seqs == 0) return FC_OK;
  std::vector<uint32_t> order(n_seqs);
  for (uint32_t s = 0; s < n_seqs; s++) {
    if (offsets[s + 1] < offsets[s]) return fc_fail(dev, FC_ERR_ARG, "offsets must not decrease");
    const uint32_t len = offsets[s + 1] - offsets[s];
    if (len < 2) return fc_fail(dev, FC_ERR_SHAPE, "scoring needs at least 2 tokens");
    if (len - 1 > m->ctx) return fc_fail(dev, FC_ERR_SHAPE, "sequence length %u must be in 1..=%u", len - 1, m->ctx);
    order[s] = s;
  }
  auto len_of = [&](uint32_t s) { return offsets[s + 1] - offsets[s]; };
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return len_of(a) > len_of(b); });
  std::vector<int32_t> padded;
  std::vector<float> lp;
  std::vector<uint8_t> gr;
  for (uint32_t g0 = 0; g0 < n_seqs;) {
    // a group: the longest sequence left and every one at least 7/8 as long (at most an eighth of the rows is padding)
    const uint32_t L = len_of(order[g0]);
    uint32_t g1 = g0 + 1;
    while (g1 < n_seqs && (uint64_t)len_of(order[g1]) * 8 >= (uint64_t)L * 7) g1++;
    const uint32_t ng = g1 - g0;
    padded.assign((size_t)ng * L, 0);
    for (uint32_t i = 0; i < ng; i++) {
      const uint32_t s = order[g0 + i];
      std::copy(ids + offsets[s], ids + offsets[s + 1], padded.begin() + (size_t)i * L);
    }
    lp.resize((size_t)ng * (L - 1));
    gr.resize((size_t)ng * (L - 1));
    FC_TRY(fc_model_score(m, padded.data(), ng, L, mode, lp.data(), gr.data(), nullptr));
    for (uint32_t i = 0; i < ng; i++) {
      const uint32_t s = order[g0 + i], n = len_of(s) - 1;
      const size_t dst = (size_t)offsets[s] - s;
      const float* row = lp.data() + (size_t)i * (L - 1);
      if (logprob_out) std::copy(row, row + n, logprob_out + dst);
      if (greedy_out) std::copy(gr.begin() + (size_t)i * (L - 1), gr.begin() + (size_t)i * (L - 1) + n, greedy_out + dst);
      if (nll_sum_out) { // serving/decoder.rs:L69-L83: f64, ascending position
        double acc = 0.0;
        for (uint32_t p = 0; p < n; p++) acc += (double)row[p];
        nll_sum_out[s] = -acc;
      }
    }
    g0 = g1;
  }
  return FC_OK;
}

// `token_logprobs` for `n_streams` id streams at once (stream j is ids[offsets[j] .. offsets[j + 1]), scored
// from target index from[j]): every stream is cut into its windows, all windows of all streams go through one
// ragged batch, and each stream's sum runs over its targets in ascending order in f64, every target exactly once.
// logprob_out[j] = sum of log p, n_tokens_out[j] = targets scored, greedy_out[j] = every target was the first
// argmax (1) or not (0); a stream with nothing to score reports (0, 0, 1) like the reference's ZERO.
FC_API int fc_model_token_logprobs(FcModel* m, const int32_t* ids, const uint32_t* offsets, const uint32_t* from,
                                   uint32_t n_streams, int mode, double* logprob_out, uint64_t* n_tokens_out,
                                   uint8_t* greedy_out) {
  if (!m || !ids || !offsets) return FC_ERR_ARG;
  struct Win {
    uint32_t stream, start, end, first;
  };
  std::vector<Win> wins;
  std::vector<uint32_t> ws, we, wf;
  for (uint32_t j = 0; j < n_streams; j++) {
    if (offsets[j + 1] < offsets[j]) return fc_fail(m->dev, FC_ERR_ARG, "offsets must not decrease");
    const uint32_t n = offsets[j + 1] - offsets[j], f = from ? from[j] : 1;
    const uint32_t nw = fc_score_windows(n, f, m->ctx, nullptr, nullptr, nullptr, 0);
    ws.resize(nw), we.resize(nw), wf.resize(nw);
    fc_score_windows(n, f, m->ctx, ws.data(), we.data(), wf.data(), nw);
    for (uint32_t w = 0; w < nw; w++) wins.push_back({j, ws[w], we[w], wf[w]});
  }
  for (uint32_t j = 0; j < n_streams; j++) {
    if (logprob_out) logprob_out[j] = 0.0;
    if (n_tokens_out) n_tokens_out[j] = 0;
    if (greedy_out) greedy_out[j] = 1;
  }
  if (wins.empty()) return FC_OK;
  std::vector<int32_t> flat;
  std::vector<uint32_t> offs(1, 0);
  for (const Win& w : wins) {
    const int32_t* src = ids + offsets[w.stream];
    flat.insert(flat.end(), src + w.start, src + w.end);
    offs.push_back((uint32_t)flat.size());
  }
  std::vector<float> lp(flat.size() - wins.size());
  std::vector<uint8_t> gr(lp.size());
  FC_TRY(fc_model_score_ragged(m, flat.data(), offs.data(), (uint32_t)wins.size(), mode, lp.data(), gr.data(), nullptr));
  for (size_t i = 0; i < wins.size(); i++) { // windows of a stream are in ascending order: so are the targets
    const Win& w = wins[i];
    const size_t base = (size_t)offs[i] - i;
    for (uint32_t target = w.first; target < w.end; target++) { // score.rs:L40-L45
      const size_t at = base + (target - w.start - 1);
      if (logprob_out) logprob_out[w.stream] += (double)lp[at];
      if (n_tokens_out) n_tokens_out[w.stream] += 1;
      if (greedy_out) greedy_out[w.stream] &= gr[at] ? 1 : 0;
    }
  }
  return FC_OK;
}
