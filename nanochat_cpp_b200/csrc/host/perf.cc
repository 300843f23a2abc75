#include "perf.h"

#include <algorithm>
#include <cmath>
#include <cstdio>

namespace ncb {

namespace {
constexpr int kGateChannels = 12, kSmearChannels = 24;

int Window(const EngineConfig& c, int layer) {
  const int left = c.window_left(layer);
  return left < 0 ? c.seq_len : std::min(left, c.seq_len);
}
double ElementBytes(const std::string& p) { return p == "fp32" ? 4.0 : p == "fp8" ? 1.0 : 2.0; }
}  // namespace

std::int64_t NumMatmulParams(const EngineConfig& c) {
  const std::int64_t C = c.hidden_dim;
  const std::int64_t per_layer = c.query_dim() * C + 2 * c.kv_dim() * C + C * C + 2 * C * c.mlp_dim();
  std::int64_t value_layers = 0;
  for (int i = 0; i < c.num_layers; ++i) value_layers += c.has_value_embedding(i) ? 1 : 0;
  // every linear map of the token stream counts: the block matrices, the LM head, the value gates and the smear
  // gate (reference src/performance_model.cc:233-249); the embeddings are gathers and do not
  return c.num_layers * per_layer + static_cast<std::int64_t>(c.padded_vocab_size) * C +
         value_layers * c.num_kv_heads * kGateChannels + kSmearChannels;
}

ParamCounts CountParams(const EngineConfig& c) {
  ParamCounts p;
  const std::int64_t L = c.num_layers, C = c.hidden_dim, V = c.padded_vocab_size;
  std::int64_t value_layers = 0;
  for (int i = 0; i < c.num_layers; ++i) value_layers += c.has_value_embedding(i) ? 1 : 0;
  p.lm_head = V * C;
  p.embeddings = V * C + value_layers * V * c.kv_dim();
  p.transformer_matrices = L * (C * c.query_dim() + 2 * C * c.kv_dim() + C * C + 2 * C * c.mlp_dim()) +
                           value_layers * c.num_kv_heads * kGateChannels;
  p.scalars = 2 * L + kSmearChannels + 2;
  p.total = p.lm_head + p.embeddings + p.transformer_matrices + p.scalars;
  return p;
}

double FlopsPerToken(const EngineConfig& c) {
  double attn = 0.0;
  for (int i = 0; i < c.num_layers; ++i) attn += 12.0 * c.num_heads * c.head_dim() * Window(c, i);
  return 6.0 * static_cast<double>(NumMatmulParams(c)) + attn;
}

double MuonFlopsPerStep(const EngineConfig& c, int ns_steps) {
  const double C = c.hidden_dim;
  const double shapes[6][2] = {{static_cast<double>(c.query_dim()), C}, {static_cast<double>(c.kv_dim()), C},
                               {static_cast<double>(c.kv_dim()), C},    {C, C},
                               {static_cast<double>(c.mlp_dim()), C},   {C, static_cast<double>(c.mlp_dim())}};
  double total = 0.0;
  for (const auto& s : shapes) {
    const double k = std::min(s[0], s[1]), n = std::max(s[0], s[1]);
    total += c.num_layers * ns_steps * (4.0 * k * k * n + 2.0 * k * k * k);
  }
  return total;
}

double PrefillFlops(const EngineConfig& c, int prompt_tokens) {
  double attn = 0.0;
  for (int i = 0; i < c.num_layers; ++i) {
    const int left = c.window_left(i);
    const double keys = left < 0 ? prompt_tokens / 2.0 : std::min<double>(left, prompt_tokens / 2.0);
    attn += 4.0 * c.num_heads * c.head_dim() * keys;
  }
  return prompt_tokens * (2.0 * static_cast<double>(NumMatmulParams(c)) + attn);
}

double DecodeFlopsPerToken(const EngineConfig& c, int context_tokens) {
  double attn = 0.0;
  for (int i = 0; i < c.num_layers; ++i) {
    const int left = c.window_left(i);
    const double keys = left < 0 ? context_tokens : std::min(left, context_tokens);
    attn += 4.0 * c.num_heads * c.head_dim() * keys;
  }
  return 2.0 * static_cast<double>(NumMatmulParams(c)) + attn;
}

double ComputeMfu(double tokens_per_second, double flops_per_token, double peak_flops) {
  return peak_flops > 0 ? tokens_per_second * flops_per_token / peak_flops : 0.0;
}

double DeviceLimits::Peak(const std::string& p) const { return p == "bf16" ? bf16 : p == "fp8" ? fp8 : p == "fp32" ? fp32 : 0.0; }

bool LookupDevice(const std::string& name, double measured_bf16_tflops, double measured_hbm_gbs, DeviceLimits* d) {
  d->name = name;
  if (name == "b200") {
    // sustained cuBLAS bf16 rate under the power cap and copy bandwidth: measured values when the caller has
    // them, else the fallback figures documented for this pool (1.4 PFLOP/s sustained, 6.65 TB/s)
    const double bf16 = (measured_bf16_tflops > 0 ? measured_bf16_tflops : 1400.0) * 1e12;
    d->bf16 = bf16, d->fp8 = 2 * bf16, d->fp32 = bf16 / 16.0;
    d->hbm_bytes_per_s = (measured_hbm_gbs > 0 ? measured_hbm_gbs : 6650.0) * 1e9;
    d->launch_seconds = 2.5e-6, d->link_bytes_per_s = 770e9;
    return true;
  }
  if (name == "h100") {
    d->bf16 = 989e12, d->fp8 = 1979e12, d->fp32 = 67e12, d->hbm_bytes_per_s = 3.35e12, d->launch_seconds = 3e-6;
    d->link_bytes_per_s = 450e9;
    return true;
  }
  if (name == "t4") {
    d->bf16 = 0, d->fp8 = 0, d->fp32 = 8.1e12, d->hbm_bytes_per_s = 320e9, d->launch_seconds = 3e-6;
    return true;
  }
  if (name == "cpu") {
    d->bf16 = 0, d->fp8 = 0, d->fp32 = 0.5e12, d->hbm_bytes_per_s = 50e9, d->launch_seconds = 0;
    return true;
  }
  return false;
}

namespace {
RooflineRow MakeRow(const DeviceLimits& lim, const std::string& name, const std::string& phase,
                    const std::string& precision, double flops, double bytes, int launches, double divisor) {
  RooflineRow r;
  r.name = name, r.phase = phase, r.precision = precision, r.flops = flops, r.bytes = bytes, r.launches = launches;
  const double peak = lim.Peak(precision);
  r.compute_seconds = (peak > 0 && flops > 0) ? (flops / divisor) / peak : 0.0;
  r.memory_seconds = lim.hbm_bytes_per_s > 0 ? (bytes / divisor) / lim.hbm_bytes_per_s : 0.0;
  const double lat = launches * lim.launch_seconds;
  r.bound_seconds = std::max({r.compute_seconds, r.memory_seconds, lat});
  r.limit = r.bound_seconds == r.compute_seconds ? "compute" : r.bound_seconds == r.memory_seconds ? "memory" : "launch";
  if (r.bound_seconds > 0 && peak > 0) r.mfu = (flops / divisor) / (r.bound_seconds * peak);
  return r;
}
}  // namespace

bool EstimatePerformance(const EngineConfig& c, const RooflinePlan& plan, RooflineEstimate* e, std::string* error) {
  DeviceLimits lim;
  if (!LookupDevice(plan.device, plan.measured_bf16_tflops, plan.measured_hbm_gbs, &lim)) {
    if (error) *error = "unknown device '" + plan.device + "'";
    return false;
  }
  const int world = std::max(1, plan.world_size), accum = std::max(1, plan.grad_accum);
  const double tokens = static_cast<double>(plan.batch) * c.seq_len * accum * world;
  const std::string prec = plan.precision;
  const std::string row_prec = (prec == "bf16" || prec == "fp8") ? "bf16" : prec;
  *e = RooflineEstimate();
  e->device = lim.name, e->precision = prec;
  e->shape = "L" + std::to_string(c.num_layers) + "-h" + std::to_string(c.hidden_dim) + "-s" +
             std::to_string(c.seq_len) + "-b" + std::to_string(plan.batch) + "x" + std::to_string(accum) + "x" +
             std::to_string(world);
  const double h = c.hidden_dim, q = c.query_dim(), kv = c.kv_dim(), mlp = c.mlp_dim(), V = c.padded_vocab_size;
  struct Group {
    const char* name;
    double n, k;
    int count;
    std::string p;
  };
  const Group groups[] = {{"qkv", q + 2 * kv, h, c.num_layers, prec},
                          {"attn_proj", h, q, c.num_layers, prec},
                          {"mlp_fc", mlp, h, c.num_layers, prec},
                          {"mlp_proj", h, mlp, c.num_layers, prec},
                          {"lm_head", V, h, 1, row_prec}};
  for (const Group& g : groups) {
    const double params = g.n * g.k * g.count, el = ElementBytes(g.p);
    const double fwd_bytes = el * (tokens * g.k * g.count + params + tokens * g.n * g.count);
    e->rows.push_back(MakeRow(lim, std::string("gemm_") + g.name, "forward", g.p, 2.0 * params * tokens, fwd_bytes,
                              g.count * accum, world));
    e->rows.push_back(MakeRow(lim, std::string("gemm_") + g.name, "backward", g.p, 4.0 * params * tokens,
                              2.0 * fwd_bytes, 2 * g.count * accum, world));
  }
  double att_f = 0.0, att_b = 0.0;
  for (int layer = 0; layer < c.num_layers; ++layer) {
    const double per_tok = static_cast<double>(c.num_heads) * c.head_dim() * Window(c, layer);
    att_f += 4.0 * per_tok * tokens;
    att_b += 8.0 * per_tok * tokens;
  }
  const double rb = ElementBytes(row_prec);
  const double att_bytes = rb * tokens * 4.0 * c.num_heads * c.head_dim() * c.num_layers;
  e->rows.push_back(MakeRow(lim, "attention", "forward", row_prec, att_f, att_bytes, c.num_layers * accum, world));
  e->rows.push_back(MakeRow(lim, "attention", "backward", row_prec, att_b, 2.0 * att_bytes, 3 * c.num_layers * accum, world));
  const double width = c.num_layers * (6.0 * h + 2.0 * q + 4.0 * kv + 2.0 * mlp + c.num_kv_heads);
  const double pw = rb * tokens * width;
  e->rows.push_back(MakeRow(lim, "norms_and_pointwise", "forward", row_prec, 0.0, pw / 2, 4 * c.num_layers * accum, world));
  e->rows.push_back(MakeRow(lim, "norms_and_pointwise", "backward", row_prec, 0.0, pw / 2, 4 * c.num_layers * accum, world));
  const double cls = 2.0 * rb * tokens * V;
  e->rows.push_back(MakeRow(lim, "classifier", "forward", row_prec, 0.0, cls / 2, accum, world));
  e->rows.push_back(MakeRow(lim, "classifier", "backward", row_prec, 0.0, cls / 2, accum, world));
  const double emb = 2.0 * rb * tokens * h;
  e->rows.push_back(MakeRow(lim, "embedding", "forward", row_prec, 0.0, emb / 2, 1, world));
  e->rows.push_back(MakeRow(lim, "embedding", "backward", row_prec, 0.0, emb / 2, 1, world));
  const double total_params = static_cast<double>(CountParams(c).total);
  e->rows.push_back(MakeRow(lim, "optimizer", "optimizer", "fp32", 0.0, 16.0 * total_params, 8, world));
  const double muon = MuonFlopsPerStep(c, plan.muon_ns_steps);
  if (muon > 0) {
    e->optimizer_flops = muon;
    e->rows.push_back(MakeRow(lim, "muon_orthogonalisation", "optimizer", row_prec, muon, 0.0, 40, world));
  }
  const double link = plan.link_gbps > 0 ? plan.link_gbps * 1e9 : lim.link_bytes_per_s;
  if (world > 1 && link > 0) {
    const double pull = (world - 1.0) / world * 4.0 * total_params;
    const double push = (world - 1.0) / world * 2.0 * total_params;
    const double full = std::max(pull, push) / link + plan.latency_us * 1e-6;
    e->sync_seconds = (1.0 - std::min(1.0, std::max(0.0, plan.overlap))) * full;
  }
  for (const RooflineRow& r : e->rows) {
    e->step_seconds += r.bound_seconds;
    if (r.phase == "forward") e->forward_seconds += r.bound_seconds;
    else if (r.phase == "backward") e->backward_seconds += r.bound_seconds;
    else e->optimizer_seconds += r.bound_seconds;
  }
  e->step_seconds += e->sync_seconds;
  e->tokens_per_step = static_cast<std::int64_t>(tokens + 0.5);
  e->steps = plan.total_tokens > 0 ? std::max<std::int64_t>(1, static_cast<std::int64_t>(std::ceil(plan.total_tokens / tokens))) : 1;
  e->run_seconds = e->step_seconds * e->steps;
  e->tokens_per_second = e->step_seconds > 0 ? tokens / e->step_seconds : 0.0;
  double mf = 0.0, mp = 0.0;
  for (const RooflineRow& r : e->rows) {
    const double peak = lim.Peak(r.precision);
    if (r.phase != "optimizer" && r.flops > 0 && peak > 0) {
      mf += r.flops;
      mp += r.flops / peak;
    }
  }
  if (mp > 0) {
    e->weighted_peak_flops = mf / mp;
    if (e->step_seconds > 0) e->model_mfu = (mf / world) / (e->step_seconds * e->weighted_peak_flops);
  }
  if (e->optimizer_flops > 0 && e->step_seconds > 0 && lim.Peak(row_prec) > 0)
    e->optim_mfu = (e->optimizer_flops / world) / (e->step_seconds * lim.Peak(row_prec));
  return true;
}

std::string RooflineJson(const RooflineEstimate& e) {
  std::string s = "{\"schema\": \"nanochat.roofline.v3\", \"device\": \"" + e.device + "\", \"precision\": \"" +
                  e.precision + "\", \"shape\": \"" + e.shape + "\", \"rows\": [";
  char buf[1024];
  for (std::size_t i = 0; i < e.rows.size(); ++i) {
    const RooflineRow& r = e.rows[i];
    const std::string family = r.name.rfind("gemm", 0) == 0 ? "gemm" : r.name;
    std::snprintf(buf, sizeof(buf),
                  "%s{\"name\": \"%s\", \"family\": \"%s\", \"phase\": \"%s\", \"precision\": \"%s\", \"shape\": \"%s\", "
                  "\"flops\": %.17g, \"issued_flops\": %.17g, \"bytes\": %.17g, \"launches\": %d, "
                  "\"compute_seconds\": %.17g, \"memory_seconds\": %.17g, \"bound_seconds\": %.17g, \"ms\": %.17g, "
                  "\"limit\": \"%s\", \"gflops\": %.17g, \"work_ratio\": %.1f, \"mfu\": %.17g}",
                  i ? ", " : "", r.name.c_str(), family.c_str(), r.phase.c_str(), r.precision.c_str(), e.shape.c_str(),
                  r.flops, r.flops, r.bytes, r.launches, r.compute_seconds, r.memory_seconds, r.bound_seconds,
                  r.bound_seconds * 1e3, r.limit.c_str(), r.bound_seconds > 0 ? r.flops / r.bound_seconds / 1e9 : 0.0,
                  r.flops > 0 ? 1.0 : 0.0, r.mfu);
    s += buf;
  }
  std::snprintf(buf, sizeof(buf),
                "], \"forward_seconds\": %.17g, \"backward_seconds\": %.17g, \"sync_seconds\": %.17g, "
                "\"optimizer_seconds\": %.17g, \"step_seconds\": %.17g, \"steps\": %lld, \"run_seconds\": %.17g, "
                "\"tokens_per_step\": %lld, \"tokens_per_second\": %.17g, \"weighted_peak_flops\": %.17g, "
                "\"model_mfu\": %.17g, \"optim_mfu\": %.17g, \"optimizer_flops\": %.17g}",
                e.forward_seconds, e.backward_seconds, e.sync_seconds, e.optimizer_seconds, e.step_seconds,
                static_cast<long long>(e.steps), e.run_seconds, static_cast<long long>(e.tokens_per_step),
                e.tokens_per_second, e.weighted_peak_flops, e.model_mfu, e.optim_mfu, e.optimizer_flops);
  return s + buf;
}

std::string RooflineTable(const RooflineEstimate& e) {
  char buf[512];
  std::snprintf(buf, sizeof(buf), "%-30s %-9s %6s %14s %14s %12s %10s\n", "operation", "phase", "prec", "compute (ms)",
                "memory (ms)", "bound (ms)", "limit");
  std::string s = buf;
  for (const RooflineRow& r : e.rows) {
    std::snprintf(buf, sizeof(buf), "%-30s %-9s %6s %14.3f %14.3f %12.3f %10s\n", r.name.c_str(), r.phase.c_str(),
                  r.precision.c_str(), r.compute_seconds * 1e3, r.memory_seconds * 1e3, r.bound_seconds * 1e3,
                  r.limit.c_str());
    s += buf;
  }
  std::snprintf(buf, sizeof(buf),
                "phases: forward %.3f | backward %.3f | optimizer %.3f | sync %.3f (ms)\nstep bound %.3f ms  (%.1f s over "
                "%lld steps)\nat the bound: %.0f tokens/s | model_mfu %.1f%% | optim_mfu %.1f%% | weighted peak %.1f TFLOP/s\n",
                e.forward_seconds * 1e3, e.backward_seconds * 1e3, e.optimizer_seconds * 1e3, e.sync_seconds * 1e3,
                e.step_seconds * 1e3, e.run_seconds, static_cast<long long>(e.steps), e.tokens_per_second,
                e.model_mfu * 100, e.optim_mfu * 100, e.weighted_peak_flops / 1e12);
  return s + buf;
}

}  // namespace ncb
