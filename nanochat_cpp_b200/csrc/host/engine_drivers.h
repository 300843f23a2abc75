// The host-side loops above a model, written once for every backend: sampling loop, scoring, the RL step. `Model`
// is anything with NewCache / Prefill / Decode / ForwardLoss / Backward / ZeroGrad / losses / logits / valid_targets
// (the CPU engine itself, or a view of a device engine); logits and losses reach these loops in host memory.
// Semantics follow the reference (src/generate.cc:458-576, src/eval.cc:87-204, src/rl.cc).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "core.h"

namespace ncb {

template <typename Model>
std::vector<GeneratedRow> GenerateBatchOn(Model* model, const int* prompt, int length, const GenerateOptions& opt,
                                          int first_row = 0) {
  const int rows = std::max(1, opt.num_samples);
  std::vector<GeneratedRow> out(static_cast<std::size_t>(rows));
  for (int r = 0; r < rows; ++r) {
    GeneratedRow& row = out[r];
    row.tokens.assign(prompt, prompt + length);
    row.mask.assign(static_cast<std::size_t>(length), 0);
    auto cache = model->NewCache(length + opt.max_tokens + 1);
    std::vector<float> logits;
    model->Prefill(cache.get(), prompt, length, &logits);
    Rng rng(MixSeed(opt.seed, static_cast<std::uint64_t>(first_row + r)));   // one stream per (seed, row)
    const int row_stop = r < static_cast<int>(opt.stop_ids.size()) ? opt.stop_ids[r] : -1;
    for (int step = 0; step < opt.max_tokens; ++step) {
      const int tok = SampleToken(logits.data(), static_cast<int>(logits.size()), opt.temperature, opt.top_k, &rng);
      if ((opt.stop_id >= 0 && tok == opt.stop_id) || (opt.bos_id >= 0 && tok == opt.bos_id) ||
          (row_stop >= 0 && tok == row_stop))
        break;
      row.tokens.push_back(tok);
      row.mask.push_back(1);
      if (step + 1 == opt.max_tokens) break;
      model->Decode(cache.get(), tok, &logits);
    }
  }
  return out;
}

template <typename Model>
std::vector<ScoreRow> ScoreBatchOn(Model* model, const int* tokens, int batch, int seq, const int* lengths,
                                   const FocusRequest* focus) {
  constexpr float kCap = 15.0f;
  const int V = model->config().vocab_size, PV = model->config().padded_vocab_size;
  std::vector<int> targets(static_cast<std::size_t>(batch) * seq, -1);
  auto len_of = [&](int b) { return std::min(std::max(lengths ? lengths[b] : seq, 0), seq); };
  for (int b = 0; b < batch; ++b)
    for (int p = 0; p + 1 < len_of(b); ++p)
      targets[static_cast<std::size_t>(b) * seq + p] = tokens[static_cast<std::size_t>(b) * seq + p + 1];
  model->ForwardLoss(tokens, targets.data(), batch, seq, true);
  const std::vector<float>& losses = model->losses();
  const std::vector<float>& logits = model->logits();
  std::vector<ScoreRow> out(static_cast<std::size_t>(batch));
  for (int b = 0; b < batch; ++b) {
    ScoreRow& r = out[b];
    r.nll.assign(static_cast<std::size_t>(seq), 0.0f);
    r.argmax.assign(static_cast<std::size_t>(seq), -1);
    for (int p = 0; p + 1 < len_of(b); ++p) {
      const std::size_t row = static_cast<std::size_t>(b) * seq + p;
      r.nll[p] = losses[row];
      const float* lr = &logits[row * PV];
      int best = 0;
      for (int j = 1; j < V; ++j)
        if (lr[j] > lr[best]) best = j;
      r.argmax[p] = best;
    }
    if (focus != nullptr && focus[b].position >= 0 && focus[b].position < seq) {
      const float* lr = &logits[(static_cast<std::size_t>(b) * seq + focus[b].position) * PV];
      for (int id : focus[b].ids) r.focus_logits.push_back(id >= 0 && id < V ? kCap * std::tanh(lr[id] / kCap) : 0.0f);
    }
  }
  return out;
}

template <typename Model, typename Optim>
float RlStepOn(Model* model, Optim* opt, const int* tokens, const int* targets, const float* advantages, int batch,
               int seq, int num_passes, int examples_per_rank, int step) {
  model->ZeroGrad();
  const float loss = model->ForwardLoss(tokens, targets, batch, seq);
  const std::int64_t valid = model->valid_targets();
  if (valid == 0) return loss;
  const double divisor = static_cast<double>(valid) * num_passes * examples_per_rank;
  model->Backward(1.0f, advantages, divisor);
  if (opt != nullptr) opt->Step(step);
  return loss;
}

}  // namespace ncb
