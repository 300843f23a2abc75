// The CPU engine: the same model, optimizer and generation loop as the GPU package, in plain C++ with fp32
// storage and double-precision reductions. It is the engine behind the C ABI (hosts in other languages, machines
// without a GPU) and an independent oracle for the kernels. Arithmetic follows the reference CPU backend
// (backends/cpu/kernels.cc) and graph (src/model.cc, src/optim.cc, src/generate.cc).
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "core.h"

namespace ncb {

enum class ParamKind { kLmHead, kWte, kValueEmbed, kResid, kX0, kSmear, kMatrix };

struct CpuParam {
  std::string name;
  std::vector<std::int64_t> shape;
  int rows = 0, cols = 0;  // 0 for scalars and vectors
  ParamKind kind = ParamKind::kMatrix;
  int layer = -1;
  std::size_t offset = 0, count = 0;
};

struct EngineConfig : ModelConfig {
  int short_window_override = 0;  // 0: ceil(seq/4/128)*128
  int head_dim() const { return hidden_dim / num_heads; }
  int query_dim() const { return num_heads * head_dim(); }
  int kv_dim() const { return num_kv_heads * head_dim(); }
  int mlp_dim() const { return 4 * hidden_dim; }
  int backout_layer() const { return num_layers / 2; }
  bool has_value_embedding(int layer) const { return value_embedding && layer % 2 == (num_layers - 1) % 2; }
  int short_window() const {
    return short_window_override > 0 ? short_window_override : ((seq_len / 4 + 127) / 128) * 128;
  }
  int window_left(int layer) const;  // -1: full context
};

class KvCache;

class CpuModel {
 public:
  explicit CpuModel(const EngineConfig& cfg);
  ~CpuModel();
  const EngineConfig& config() const { return cfg_; }
  void InitWeights(std::uint64_t seed);

  // Mean cross entropy over the valid targets; keeps what Backward needs. `keep_logits` also keeps the raw
  // (un-capped) logits [B*T, padded_vocab] and the per-row losses for scoring.
  float ForwardLoss(const int* tokens, const int* targets, int batch, int seq, bool keep_logits = false);
  // grad += d(scale * sum_rows(w_row * nll_row) / divisor) / d(param); divisor <= 0 means the valid-target count.
  void Backward(float scale, const float* row_weights = nullptr, double divisor = 0.0);
  void ZeroGrad();

  const std::vector<CpuParam>& params() const { return params_; }
  const CpuParam* Find(const std::string& name) const;
  float* value(const CpuParam& p) { return value_.data() + p.offset; }
  float* grad(const CpuParam& p) { return grad_.data() + p.offset; }
  std::vector<float>& values() { return value_; }
  std::vector<float>& grads() { return grad_; }
  const std::vector<float>& losses() const { return losses_; }
  const std::vector<float>& logits() const { return logits_; }
  std::int64_t valid_targets() const { return valid_; }

  bool Save(const std::string& path, std::string* error) const;
  bool Load(const std::string& path, std::string* error);
  // The same container with the optimizer records and the step beside the parameters (a resumable checkpoint).
  bool SaveWithOptimizer(const std::string& path, const class CpuOptimizer& opt, std::uint64_t step,
                         std::uint32_t world_size, std::string* error) const;
  // `opt` may be null (weights only: a warm start keeps fresh optimizer state). `step` receives the stored step.
  bool LoadWithOptimizer(const std::string& path, class CpuOptimizer* opt, std::uint64_t* step, std::string* error);

  // Inference with a contiguous KV cache, one sequence at a time (soft-capped logits over the real vocabulary).
  std::unique_ptr<KvCache> NewCache(int max_seq) const;
  void Prefill(KvCache* cache, const int* tokens, int count, std::vector<float>* last_logits);
  void Decode(KvCache* cache, int token, std::vector<float>* logits);

 private:
  struct Saved;
  void Trunk(const int* tokens, int B, int T, Saved* save, std::vector<float>* xn);
  void Step(KvCache* cache, const int* tokens, int count, std::vector<float>* logits);
  EngineConfig cfg_;
  std::vector<CpuParam> params_;
  std::vector<float> value_, grad_, losses_, logits_;
  std::unique_ptr<Saved> saved_;
  std::int64_t valid_ = 0;
};

struct OptimConfig {
  float unembedding_lr = 0.004f, embedding_lr = 0.2f, matrix_lr = 0.02f, scalar_lr = 0.5f, weight_decay = 0.0f;
  int muon_ns_steps = 5;
  float muon_beta2 = 0.9f, adam_eps = 1e-10f, clip = 1.0f, init_lr_frac = 1.0f;
  int num_iterations = 0, warmup_steps = 0;
  float warmdown_ratio = 0.65f, final_lr_frac = 0.0f, weight_decay_base = 0.0f;
  float muon_momentum_warmup_steps = 400.0f, muon_momentum_start = 0.85f, muon_momentum_peak = 0.97f,
        muon_momentum_final = 0.90f;
  float LrMultiplier(int step) const;
  float MuonMomentum(int step) const;
  float WeightDecay(int step) const;
};

class CpuOptimizer {
 public:
  CpuOptimizer(CpuModel* model, const OptimConfig& cfg);
  void Step(int step);  // 1-based
  float grad_norm() const { return grad_norm_; }
  const OptimConfig& config() const { return cfg_; }
  // Optimizer records in the checkpoint's naming: `adamw.<kind>.{m,v}` (the parameters of a kind concatenated),
  // `muon.<rows>x<cols>.{buf1,buf2}` (stacked over the group), all fp32.
  void ExportState(std::vector<TensorRecord>* out) const;
  bool ImportState(const std::vector<TensorRecord>& records, std::string* error);

 private:
  struct AdamGroup {
    ParamKind kind;
    float lr, beta1, beta2, wd;
    std::vector<const CpuParam*> params;
    std::vector<std::vector<float>> m, v;
  };
  struct MuonGroup {
    int rows, cols;
    float lr;
    std::vector<const CpuParam*> params;
    std::vector<std::vector<float>> buf1, buf2;
  };
  void MuonUpdate(MuonGroup* g, std::size_t index, float lr, float momentum, float wd, float grad_scale);
  CpuModel* model_;
  OptimConfig cfg_;
  std::vector<AdamGroup> adam_;
  std::vector<MuonGroup> muon_;
  float grad_norm_ = 0.0f;
};

struct GenerateOptions {
  int num_samples = 1, max_tokens = 64;
  float temperature = 0.0f;
  int top_k = 0;
  std::uint64_t seed = 0;
  int stop_id = -1, bos_id = -1;
  std::vector<int> stop_ids;  // optional, one per sample
};
struct GeneratedRow {
  std::vector<int> tokens;
  std::vector<std::uint8_t> mask;  // 1 = sampled
};
// `num_samples` continuations of one prompt; a row ends at its stop token (not appended) or at max_tokens.
std::vector<GeneratedRow> GenerateBatch(CpuModel* model, const int* prompt, int length, const GenerateOptions& opt,
                                        int first_row = 0);

struct ScoreRow {
  std::vector<float> nll;
  std::vector<int> argmax;
  std::vector<float> focus_logits;
};
struct FocusRequest {
  int position = -1;
  std::vector<int> ids;
};
std::vector<ScoreRow> ScoreBatch(CpuModel* model, const int* tokens, int batch, int seq, const int* lengths,
                                 const FocusRequest* focus);

// Muon for one matrix on the host (momentum + Nesterov, row equilibration, Polar Express, Muon+, NorMuon,
// cautious decay; reference backends/cpu/kernels.cc:1614-1810). `w` fp32 [rows, cols] is updated in place, `b1`
// [rows, cols] and `b2` [max(rows, cols) lines] are the two state buffers. Also used by the GPU engine for the few
// matrices that are too small for its batched kernels (the 12-channel value gates).
void MuonUpdateHost(float* w, const float* grad, float* b1, float* b2, int rows, int cols, float lr, float momentum,
                    float wd, float beta2, int ns_steps, float grad_scale);

// One policy-gradient step (reference src/rl.cc): returns the loss; `valid * num_passes * examples_per_rank` divides.
float RlStep(CpuModel* model, CpuOptimizer* opt, const int* tokens, const int* targets, const float* advantages,
             int batch, int seq, int num_passes, int examples_per_rank, int step);

}  // namespace ncb

#include "engine_drivers.h"
