// Native planning layer: model specification, device profile, the operator plan and the training-run plan.
//
// Three small contracts kept apart, as in the reference (include/nanochat/model_spec.h, device_profile.h, plan.h;
// src/model_spec.cc, src/device_profile.cc, src/plan.cc):
//   * ModelSpec      a closed JSON description of the model (unknown keys and unknown block kinds are errors);
//   * DeviceProfile  what a device declares: capability names, precisions, peak rates (`caps/*.json`);
//   * BuildPlan      a pure function of the two: per operation family, the fused kernel when the device declares its
//                    capability, otherwise the composition of primitive operators; a model whose `requires` the
//                    device does not meet is rejected with the missing names.
// and the training-run plan of the reference's Python planner (python/nanochat_cpp/plan.py, which mirrors upstream
// `scripts/base_train.py`): horizon, batch size, learning-rate and weight-decay scaling from depth and vocabulary.
// Everything here is host-only and needs no device.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "engine.h"
#include "perf.h"

namespace ncb {

// ---- a strict little JSON reader (objects keep their key order) --------------------------------------------------
struct Json {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* Find(const std::string& key) const;
  bool Has(const std::string& key) const { return Find(key) != nullptr; }
};
bool ParseJson(const std::string& text, Json* out, std::string* error);
std::string JsonQuote(const std::string& s);

// ---- model specification ----------------------------------------------------------------------------------------
struct BlockSpec {
  std::string norm = "rms_norm", attention = "causal", attention_variant = "mha", position = "rope",
              mlp = "relu_square", residual = "blend", dtype = "build_default";
  bool value_embedding = false;
};
struct ModelSpec {
  std::string name;
  std::vector<std::string> requires_;
  int num_heads = 0, num_kv_heads = 0, hidden_dim = 0, seq_len = 2048, vocab_size = 32768, padded_vocab_size = 0;
  double rope_base = 100000.0;
  std::vector<BlockSpec> blocks;
  int backout_layer = -1;
};
bool ParseModelSpec(const std::string& json_text, ModelSpec* out, std::string* error);
bool SpecToConfig(const ModelSpec& spec, EngineConfig* out, std::string* error);

// ---- device profile ---------------------------------------------------------------------------------------------
struct DeviceProfile {
  std::string device;
  std::vector<std::string> match, features, precisions;
  std::map<std::string, double> peaks;
  bool Has(const std::string& feature) const;
};
bool ParseDeviceProfile(const std::string& json_text, DeviceProfile* out, std::string* error);

// ---- operator plan ----------------------------------------------------------------------------------------------
struct PlanRow {
  std::string family, choice, detail;  // choice: "kernel" | "composition"
};
struct OperatorPlan {
  std::string model, device, precision, graph;
  std::vector<PlanRow> rows;
};
// graph: train | prefill | decode | generate | eval
bool BuildPlan(const ModelSpec& spec, const DeviceProfile& profile, const std::string& precision,
               const std::string& graph, OperatorPlan* out, std::string* error);
std::string PlanJson(const OperatorPlan& plan);

// ---- training-run plan ------------------------------------------------------------------------------------------
struct TrainPlanInputs {
  int depth = 12, aspect_ratio = 64, head_dim = 128, seq_len = 2048, vocab_size = 32768, device_batch_size = 32;
  int num_kv_heads = 0;  // 0: as many as query heads
  std::string window_pattern = "SSSL";
  double rope_base = 100000.0;
  std::int64_t total_batch_size = -1, num_iterations = 0;
  double target_flops = 0.0;
  int target_param_data_ratio = 12;
  double embedding_lr = 0.3, unembedding_lr = 0.008, weight_decay = 0.28, matrix_lr = 0.02, scalar_lr = 0.5;
  int warmup_steps = 40;
  double warmdown_ratio = 0.65, final_lr_frac = 0.05;
};
struct TrainPlan {
  EngineConfig config;
  ParamCounts counts;
  std::int64_t num_matmul_params = 0, scaling_params = 0, target_tokens = 0, total_batch_size = 0, grad_accum = 0,
               num_iterations = 0;
  double flops_per_token = 0, batch_lr_scale = 1.0, embedding_lr = 0, unembedding_lr = 0, matrix_lr = 0, scalar_lr = 0,
         weight_decay = 0;
  int warmup_steps = 0;
  double warmdown_ratio = 0, final_lr_frac = 0;
};
// The model shape of a depth: hidden = depth * aspect_ratio rounded up to a multiple of head_dim, one head per
// head_dim channels, vocabulary padded to a multiple of 64.
EngineConfig ConfigForDepth(int depth, int aspect_ratio, int head_dim, int seq_len, int vocab_size, int num_kv_heads,
                            const std::string& window_pattern, double rope_base);
bool ComputeTrainPlan(const TrainPlanInputs& in, TrainPlan* out, std::string* error);
std::string TrainPlanJson(const TrainPlanInputs& in, const TrainPlan& plan);

}  // namespace ncb
