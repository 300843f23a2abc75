// Parameter / FLOP counting and the analytic roofline of one training step (native counterpart of the Python
// `perf/roofline.py`; same rows, same arithmetic). Counting rules of the reference's performance model
// (src/performance_model.cc:233-380): flops per token = 6 * matmul parameters + 12 * heads * head_dim * window per
// layer; Muon's Newton-Schulz flops are reported separately; the report schema is `nanochat.roofline.v3`
// (include/nanochat/mfu.h). Gradient synchronisation is modelled as the owner-sharded one-hop exchange.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "engine.h"

namespace ncb {

struct ParamCounts {
  std::int64_t total = 0, transformer_matrices = 0, lm_head = 0, embeddings = 0, scalars = 0;
};
ParamCounts CountParams(const EngineConfig& cfg);
std::int64_t NumMatmulParams(const EngineConfig& cfg);
double FlopsPerToken(const EngineConfig& cfg);  // sliding layers count min(window, seq) keys
double MuonFlopsPerStep(const EngineConfig& cfg, int ns_steps);
double PrefillFlops(const EngineConfig& cfg, int prompt_tokens);            // forward only
double DecodeFlopsPerToken(const EngineConfig& cfg, int context_tokens);    // one new token against a KV cache
double ComputeMfu(double tokens_per_second, double flops_per_token, double peak_flops);

struct DeviceLimits {
  std::string name;
  double bf16 = 0, fp8 = 0, fp32 = 0;  // FLOP/s
  double hbm_bytes_per_s = 0, launch_seconds = 3e-6, link_bytes_per_s = 0;
  double Peak(const std::string& precision) const;
};
// "b200" (measured sustained cuBLAS rate and copy bandwidth when given, else the pool's documented fallback),
// "h100", "t4" (the reference's table), "cpu".
bool LookupDevice(const std::string& name, double measured_bf16_tflops, double measured_hbm_gbs, DeviceLimits* out);

struct RooflinePlan {
  std::string device = "b200", precision = "bf16";
  int batch = 32, grad_accum = 1, world_size = 1;
  std::int64_t total_tokens = 0;
  double link_gbps = 0.0, latency_us = 5.0, overlap = 0.0;
  int muon_ns_steps = 5;
  double measured_bf16_tflops = 0.0, measured_hbm_gbs = 0.0;
};

struct RooflineRow {
  std::string name, phase, precision, limit;
  double flops = 0, bytes = 0;
  int launches = 0;
  double compute_seconds = 0, memory_seconds = 0, bound_seconds = 0, mfu = 0;
};

struct RooflineEstimate {
  std::string device, precision, shape;
  std::vector<RooflineRow> rows;
  double forward_seconds = 0, backward_seconds = 0, optimizer_seconds = 0, sync_seconds = 0, step_seconds = 0;
  std::int64_t steps = 1, tokens_per_step = 0;
  double run_seconds = 0, tokens_per_second = 0, weighted_peak_flops = 0, model_mfu = 0, optim_mfu = 0,
         optimizer_flops = 0;
};

bool EstimatePerformance(const EngineConfig& cfg, const RooflinePlan& plan, RooflineEstimate* out, std::string* error);
std::string RooflineJson(const RooflineEstimate& e);
std::string RooflineTable(const RooflineEstimate& e);

}  // namespace ncb
