// C ABI of the in-process mesh runtime and its training driver (declared in include/nanochat/capi.h; the
// reference's entries are include/nanochat/capi.h:195-370, implemented in bindings/nanochat_capi.cc).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <thread>

#include "capi_internal.h"
#include "mesh.h"
#include "perf.h"
#include "plan.h"

struct nanochat_mesh {
  ncb::MeshSpec spec;
};
struct nanochat_runtime {
  std::unique_ptr<ncb::MeshRuntime> rt;
};

namespace {

ncb::OptimConfig ToOptim(const nanochat_optim_config* c) {
  ncb::OptimConfig o;
  if (c == nullptr) return o;
  o.unembedding_lr = c->unembedding_lr, o.embedding_lr = c->embedding_lr, o.matrix_lr = c->matrix_lr;
  o.scalar_lr = c->scalar_lr, o.weight_decay = c->weight_decay, o.muon_ns_steps = c->muon_ns_steps;
  o.muon_beta2 = c->muon_beta2, o.adam_eps = c->adam_eps, o.clip = c->clip;
  o.num_iterations = c->num_iterations, o.warmup_steps = c->warmup_steps, o.warmdown_ratio = c->warmdown_ratio;
  o.final_lr_frac = c->final_lr_frac, o.weight_decay_base = c->weight_decay_base;
  o.muon_momentum_warmup_steps = c->muon_momentum_warmup_steps, o.muon_momentum_start = c->muon_momentum_start;
  o.muon_momentum_peak = c->muon_momentum_peak, o.muon_momentum_final = c->muon_momentum_final;
  return o;
}

bool ToEngine(const nanochat_config* config, ncb::EngineConfig* cfg, const char* who) {
  if (config == nullptr) {
    ncb_set_error(std::string(who) + ": config is null");
    return false;
  }
  static_cast<ncb::ModelConfig&>(*cfg) = ncb_to_model_config(*config);
  cfg->short_window_override = ncb_short_window_override();
  std::string err;
  if (!cfg->Validate(&err)) {
    ncb_set_error(std::string(who) + ": " + err);
    return false;
  }
  return true;
}

template <typename F>
bool Try(const char* who, F&& f) {
  try {
    return f();
  } catch (const std::exception& e) {
    ncb_set_error(std::string(who) + ": " + e.what());
    return false;
  }
}

}  // namespace

int& ncb_short_window_override() {
  static int value = 0;
  return value;
}

extern "C" {

void ncb_set_short_window(int tokens) { ncb_short_window_override() = tokens > 0 ? tokens : 0; }

nanochat_mesh* nanochat_mesh_create(const int* indices, int count) {
  auto* m = new nanochat_mesh();
  count = std::max(1, count);
  for (int i = 0; i < count; ++i) m->spec.devices.push_back(indices != nullptr ? indices[i] : i);
  return m;
}
void nanochat_mesh_free(nanochat_mesh* mesh) { delete mesh; }
int nanochat_mesh_size(nanochat_mesh* mesh) { return mesh != nullptr ? mesh->spec.size() : 0; }

nanochat_runtime* nanochat_runtime_create(const nanochat_mesh* mesh, const nanochat_config* config,
                                          const nanochat_optim_config* optim, int batch, int grad_accum, int seq,
                                          uint64_t seed) {
  ncb::EngineConfig cfg;
  if (mesh == nullptr) {
    ncb_set_error("nanochat_runtime_create: mesh is null");
    return nullptr;
  }
  if (!ToEngine(config, &cfg, "nanochat_runtime_create")) return nullptr;
  auto* h = new nanochat_runtime();
  std::string err;
  const bool ok = Try("nanochat_runtime_create", [&] {
    h->rt = std::make_unique<ncb::MeshRuntime>(mesh->spec, cfg, ToOptim(optim), batch, grad_accum, seq, seed, &err);
    return h->rt->ok();
  });
  if (!ok) {
    if (!err.empty()) ncb_set_error("nanochat_runtime_create: " + err);
    delete h;
    return nullptr;
  }
  return h;
}
void nanochat_runtime_free(nanochat_runtime* runtime) { delete runtime; }
int nanochat_runtime_world_size(nanochat_runtime* runtime) { return runtime ? runtime->rt->world() : 0; }

float nanochat_runtime_train_step(nanochat_runtime* runtime, const int* tokens, const int* targets) {
  if (runtime == nullptr || tokens == nullptr || targets == nullptr) {
    ncb_set_error("nanochat_runtime_train_step: null argument");
    return 0.0f;
  }
  float loss = 0.0f;
  std::string err;
  Try("nanochat_runtime_train_step", [&] {
    loss = runtime->rt->TrainStep(tokens, targets, &err);
    return true;
  });
  if (!err.empty()) ncb_set_error("nanochat_runtime_train_step: " + err);
  return loss;
}

nanochat_status nanochat_runtime_metrics(nanochat_runtime* runtime, nanochat_metrics* out) {
  if (runtime == nullptr || out == nullptr) return NANOCHAT_STATUS_ERROR;
  const ncb::MeshMetrics& m = runtime->rt->metrics();
  out->device_count = runtime->rt->world();
  out->loss = m.loss.data();
  out->grad_norm = m.grad_norm;
  out->step_seconds = m.step_seconds;
  return NANOCHAT_STATUS_OK;
}

int nanochat_runtime_param_count(nanochat_runtime* runtime, int replica) {
  ncb::CpuModel* m = runtime ? runtime->rt->replica(replica) : nullptr;
  return m ? static_cast<int>(m->params().size()) : 0;
}
int nanochat_runtime_param_info(nanochat_runtime* runtime, int replica, int index, nanochat_param* out) {
  ncb::CpuModel* m = runtime ? runtime->rt->replica(replica) : nullptr;
  if (m == nullptr || out == nullptr || index < 0 || index >= static_cast<int>(m->params().size())) return 0;
  const ncb::CpuParam& p = m->params()[static_cast<std::size_t>(index)];
  out->name = p.name.c_str();
  out->value = m->value(p);
  out->grad = m->grad(p);
  out->count = static_cast<int64_t>(p.count);
  out->rows = p.rows, out->cols = p.cols;
  return 1;
}
int64_t nanochat_runtime_param_read(nanochat_runtime* runtime, int replica, int index, int grad, int64_t offset,
                                    int64_t count, void* data) {
  ncb::CpuModel* m = runtime ? runtime->rt->replica(replica) : nullptr;
  if (m == nullptr || data == nullptr || index < 0 || index >= static_cast<int>(m->params().size())) return -1;
  const ncb::CpuParam& p = m->params()[static_cast<std::size_t>(index)];
  if (offset < 0 || offset > static_cast<int64_t>(p.count)) return -1;
  const int64_t n = std::min<int64_t>(count, static_cast<int64_t>(p.count) - offset);
  if (n > 0) std::memcpy(data, (grad ? m->grad(p) : m->value(p)) + offset, static_cast<std::size_t>(n) * sizeof(float));
  return std::max<int64_t>(n, 0);
}
nanochat_status nanochat_runtime_param_digest(nanochat_runtime* runtime, int replica, uint64_t* out) {
  if (runtime == nullptr || out == nullptr || runtime->rt->replica(replica) == nullptr) {
    ncb_set_error("nanochat_runtime_param_digest: bad replica index or null output");
    return NANOCHAT_STATUS_ERROR;
  }
  *out = runtime->rt->ParamDigest(replica);
  return NANOCHAT_STATUS_OK;
}

void nanochat_runtime_save(nanochat_runtime* runtime, const char* path) {
  std::string err;
  if (runtime == nullptr || path == nullptr || !runtime->rt->Save(path, &err)) ncb_set_error("nanochat_runtime_save: " + err);
}
void nanochat_runtime_load(nanochat_runtime* runtime, const char* path) {
  std::string err;
  if (runtime == nullptr || path == nullptr || !runtime->rt->Load(path, &err)) ncb_set_error("nanochat_runtime_load: " + err);
}
void nanochat_runtime_load_weights(nanochat_runtime* runtime, const char* path) {
  std::string err;
  if (runtime == nullptr || path == nullptr || !runtime->rt->LoadWeights(path, &err))
    ncb_set_error("nanochat_runtime_load_weights: " + err);
}
int nanochat_runtime_step(nanochat_runtime* runtime) { return runtime ? runtime->rt->step() : -1; }
void ncb_runtime_inject_drop(nanochat_runtime* runtime, int from, int timeout_ms) {
  if (runtime == nullptr) return;
  runtime->rt->set_timeout_ms(timeout_ms);
  runtime->rt->InjectDrop(from);
}

static float RunTrain(const nanochat_mesh_train_config* c, nanochat_mesh_train_summary* out, const ncb::DistConfig* dist);

float nanochat_mesh_train_run(const nanochat_mesh_train_config* c, nanochat_mesh_train_summary* out) {
  return RunTrain(c, out, nullptr);
}

// One rank of a multi-process CPU data-parallel job: `config->run.batch` is the per-rank micro-batch, the mesh
// field is ignored, ranks meet on 127.0.0.1:`port`; rank 0 writes the checkpoint, metrics.jsonl and summary.json.
float ncb_dist_train_run(const nanochat_mesh_train_config* c, int rank, int world, int port, int timeout_ms,
                         nanochat_mesh_train_summary* out) {
  ncb::DistConfig d;
  d.rank = rank, d.world = world, d.port = port;
  if (timeout_ms > 0) d.timeout_ms = timeout_ms;
  return RunTrain(c, out, &d);
}

static float RunTrain(const nanochat_mesh_train_config* c, nanochat_mesh_train_summary* out, const ncb::DistConfig* dist) {
  if (c == nullptr) {
    ncb_set_error("nanochat_mesh_train_run: config is null");
    return 0.0f;
  }
  ncb::MeshTrainConfig cfg;
  if (!ToEngine(&c->model, &cfg.model, "nanochat_mesh_train_run")) return 0.0f;
  if (c->mesh != nullptr) cfg.mesh = c->mesh->spec;
  else cfg.mesh.devices = {0};
  if (c->optimizer != nullptr) {
    cfg.optim = ToOptim(c->optimizer);
  } else {
    nanochat_optim_config preset;
    if (nanochat_optim_config_preset(c->preset != nullptr ? c->preset : "default", &preset) != NANOCHAT_STATUS_OK)
      return 0.0f;
    cfg.optim = ToOptim(&preset);
  }
  auto str = [](const char* s) { return std::string(s != nullptr ? s : ""); };
  cfg.warm_start_path = str(c->warm_start_path);
  cfg.flops_per_token = c->flops_per_token, cfg.peak_flops = c->peak_flops;
  for (int i = 0; i < c->data.parquet_count; ++i) cfg.parquet.push_back(str(c->data.parquet[i]));
  cfg.tokenizer_path = str(c->data.tokenizer_path), cfg.packed_rows_path = str(c->data.packed_rows_path);
  cfg.data_seed = c->data.data_seed;
  cfg.batch = c->run.batch, cfg.grad_accum = c->run.grad_accum, cfg.seq = c->run.seq, cfg.seed = c->run.seed;
  cfg.num_iterations = c->run.num_iterations, cfg.log_every = c->run.log_every, cfg.save_every = c->run.save_every;
  cfg.resume = c->run.resume != 0;
  cfg.out_dir = str(c->output.out_dir), cfg.checkpoint_path = str(c->output.checkpoint_path);
  ncb::MeshTrainSummary s;
  std::string err;
  float last = 0.0f;
  Try("nanochat_mesh_train_run", [&] {
    last = dist != nullptr ? ncb::RunDistributedTrain(cfg, *dist, &s, &err) : ncb::RunMeshTrain(cfg, &s, &err);
    return true;
  });
  if (!err.empty()) ncb_set_error("nanochat_mesh_train_run: " + err);
  if (out != nullptr) {
    out->steps = s.steps, out->interrupted = s.interrupted ? 1 : 0;
    out->mean_loss = s.mean_loss, out->steady_mfu = s.steady_mfu;
    std::snprintf(out->checkpoint, sizeof(out->checkpoint), "%s", s.checkpoint.c_str());
  }
  return last;
}

nanochat_status nanochat_params_get(const nanochat_config* config, nanochat_params* out) {
  ncb::EngineConfig c;
  if (out == nullptr || !ToEngine(config, &c, "nanochat_params_get")) return NANOCHAT_STATUS_ERROR;
  const ncb::ParamCounts p = ncb::CountParams(c);
  out->total = p.total, out->transformer_matrices = p.transformer_matrices, out->lm_head = p.lm_head;
  out->embeddings = p.embeddings, out->scalars = p.scalars;
  out->flops_per_token = ncb::FlopsPerToken(c);
  return NANOCHAT_STATUS_OK;
}

// The analytic roofline as `nanochat.roofline.v3` JSON (or the text table with `as_table`). Returns the length
// needed (without the terminator); the text is truncated to `capacity - 1`. Negative on error.
int64_t ncb_roofline(const nanochat_config* config, const char* device, const char* precision, int batch, int grad_accum,
                     int world_size, int64_t total_tokens, double link_gbps, double latency_us, double overlap,
                     int muon_ns_steps, double measured_bf16_tflops, double measured_hbm_gbs, int as_table, char* out,
                     int64_t capacity) {
  ncb::EngineConfig c;
  if (!ToEngine(config, &c, "ncb_roofline")) return -1;
  ncb::RooflinePlan plan;
  plan.device = device != nullptr ? device : "b200";
  plan.precision = precision != nullptr ? precision : "bf16";
  plan.batch = batch, plan.grad_accum = grad_accum, plan.world_size = world_size, plan.total_tokens = total_tokens;
  plan.link_gbps = link_gbps, plan.latency_us = latency_us, plan.overlap = overlap, plan.muon_ns_steps = muon_ns_steps;
  plan.measured_bf16_tflops = measured_bf16_tflops, plan.measured_hbm_gbs = measured_hbm_gbs;
  ncb::RooflineEstimate e;
  std::string err;
  if (!ncb::EstimatePerformance(c, plan, &e, &err)) {
    ncb_set_error("ncb_roofline: " + err);
    return -1;
  }
  const std::string text = as_table ? ncb::RooflineTable(e) : ncb::RooflineJson(e);
  if (out != nullptr && capacity > 0) {
    const std::size_t n = std::min<std::size_t>(text.size(), static_cast<std::size_t>(capacity - 1));
    std::memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return static_cast<int64_t>(text.size());
}
namespace {
int64_t CopyOut(const std::string& text, char* out, int64_t capacity) {
  if (out != nullptr && capacity > 0) {
    const std::size_t n = std::min<std::size_t>(text.size(), static_cast<std::size_t>(capacity - 1));
    std::memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return static_cast<int64_t>(text.size());
}
bool ReadTextFile(const char* path, std::string* text) {
  if (path == nullptr) return false;
  std::FILE* f = std::fopen(path, "rb");
  if (f == nullptr) return false;
  char buf[1 << 14];
  std::size_t n;
  while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) text->append(buf, n);
  std::fclose(f);
  return true;
}
}  // namespace

// The operator plan of a model specification on a device profile as `nanochat.plan.v1` JSON: for every operation
// family, the fused kernel the device declares or the composition of primitive operators. Both arguments are paths
// of JSON files. A device that lacks a capability the model requires is an error that names it. Returns the text
// length, negative on error.
int64_t ncb_plan_json(const char* spec_path, const char* caps_path, const char* precision, const char* graph, char* out,
                      int64_t capacity) {
  std::string spec_text, caps_text, err;
  if (!ReadTextFile(spec_path, &spec_text) || !ReadTextFile(caps_path, &caps_text)) {
    ncb_set_error("ncb_plan_json: cannot read the model specification or the device declaration");
    return -1;
  }
  ncb::ModelSpec spec;
  ncb::DeviceProfile profile;
  ncb::OperatorPlan plan;
  if (!ncb::ParseModelSpec(spec_text, &spec, &err) || !ncb::ParseDeviceProfile(caps_text, &profile, &err) ||
      !ncb::BuildPlan(spec, profile, precision != nullptr ? precision : "bf16", graph != nullptr ? graph : "train", &plan,
                      &err)) {
    ncb_set_error("ncb_plan_json: " + err);
    return -1;
  }
  return CopyOut(ncb::PlanJson(plan), out, capacity);
}

// The model configuration a specification file describes. `out->window_pattern` points into `pattern`, a buffer of
// the caller (`pattern_capacity` bytes, at least layers + 1).
nanochat_status ncb_spec_config(const char* spec_path, nanochat_config* out, char* pattern, int pattern_capacity) {
  std::string text, err;
  ncb::ModelSpec spec;
  ncb::EngineConfig c;
  if (out == nullptr || pattern == nullptr || pattern_capacity <= 0 || !ReadTextFile(spec_path, &text) || !ncb::ParseModelSpec(text, &spec, &err) ||
      !ncb::SpecToConfig(spec, &c, &err)) {
    ncb_set_error("ncb_spec_config: " + (err.empty() ? std::string("cannot read the specification") : err));
    return NANOCHAT_STATUS_ERROR;
  }
  out->num_layers = c.num_layers, out->num_heads = c.num_heads, out->num_kv_heads = c.num_kv_heads;
  out->hidden_dim = c.hidden_dim, out->seq_len = c.seq_len, out->vocab_size = c.vocab_size;
  out->padded_vocab_size = c.padded_vocab_size, out->rope_base = c.rope_base;
  std::snprintf(pattern, static_cast<std::size_t>(pattern_capacity), "%s", c.window_pattern.c_str());
  out->window_pattern = pattern;
  out->value_embedding = c.value_embedding ? 1 : 0;
  return NANOCHAT_STATUS_OK;
}

// The training-run plan (horizon, batch, learning-rate and weight-decay scaling) of a depth as JSON with the keys
// `counts`, `flops_per_token`, `config`, `inputs`, `plan`. Negative `total_batch_size` asks for the predicted optimum.
int64_t ncb_train_plan_json(int depth, int aspect_ratio, int head_dim, int seq_len, int vocab_size,
                            int device_batch_size, const char* window_pattern, int64_t total_batch_size,
                            int64_t num_iterations, double target_flops, int target_param_data_ratio, char* out,
                            int64_t capacity) {
  ncb::TrainPlanInputs in;
  in.depth = depth, in.aspect_ratio = aspect_ratio, in.head_dim = head_dim, in.seq_len = seq_len;
  in.vocab_size = vocab_size, in.device_batch_size = device_batch_size;
  if (window_pattern != nullptr) in.window_pattern = window_pattern;
  in.total_batch_size = total_batch_size, in.num_iterations = num_iterations, in.target_flops = target_flops;
  in.target_param_data_ratio = target_param_data_ratio;
  ncb::TrainPlan plan;
  std::string err;
  if (!ncb::ComputeTrainPlan(in, &plan, &err)) {
    ncb_set_error("ncb_train_plan_json: " + err);
    return -1;
  }
  return CopyOut(ncb::TrainPlanJson(in, plan), out, capacity);
}

double ncb_muon_flops_per_step(const nanochat_config* config, int ns_steps) {
  ncb::EngineConfig c;
  return ToEngine(config, &c, "ncb_muon_flops_per_step") ? ncb::MuonFlopsPerStep(c, ns_steps) : 0.0;
}
double ncb_prefill_flops(const nanochat_config* config, int prompt_tokens) {
  ncb::EngineConfig c;
  return ToEngine(config, &c, "ncb_prefill_flops") ? ncb::PrefillFlops(c, prompt_tokens) : 0.0;
}
double ncb_decode_flops_per_token(const nanochat_config* config, int context_tokens) {
  ncb::EngineConfig c;
  return ToEngine(config, &c, "ncb_decode_flops_per_token") ? ncb::DecodeFlopsPerToken(c, context_tokens) : 0.0;
}

// --- collectives over TCP for multi-process CPU jobs (the ports travel through the caller) ------------------
struct ncb_tcp {
  std::unique_ptr<ncb::TcpTransport> t;
};
ncb_tcp* ncb_tcp_create(int rank, int world) {
  auto* h = new ncb_tcp();
  h->t = std::make_unique<ncb::TcpTransport>(rank, world);
  if (h->t->port() == 0) {
    ncb_set_error("ncb_tcp_create: " + h->t->error());
    delete h;
    return nullptr;
  }
  return h;
}
int ncb_tcp_port(ncb_tcp* h) { return h ? h->t->port() : 0; }
nanochat_status ncb_tcp_connect(ncb_tcp* h, const int* ports, int count, int timeout_ms) {
  if (h == nullptr || ports == nullptr) return NANOCHAT_STATUS_ERROR;
  if (!h->t->Connect(std::vector<int>(ports, ports + count), timeout_ms)) {
    ncb_set_error("ncb_tcp_connect: " + h->t->error());
    return NANOCHAT_STATUS_ERROR;
  }
  return NANOCHAT_STATUS_OK;
}
nanochat_status ncb_tcp_all_reduce_sum(ncb_tcp* h, float* data, int64_t count, int timeout_ms) {
  if (h == nullptr || data == nullptr || count < 0) return NANOCHAT_STATUS_ERROR;
  if (!ncb::RingAllReduceSum(h->t.get(), data, static_cast<std::size_t>(count), timeout_ms)) {
    ncb_set_error("ncb_tcp_all_reduce_sum: " + h->t->error());
    return NANOCHAT_STATUS_ERROR;
  }
  return NANOCHAT_STATUS_OK;
}
void ncb_tcp_free(ncb_tcp* h) { delete h; }

// In-process check of the ring over the mailbox transport: `world` threads reduce their rows of data[world][count].
nanochat_status ncb_memory_ring_all_reduce(float* data, int world, int64_t count, int drop_from, int timeout_ms) {
  if (data == nullptr || world < 1 || count < 0) return NANOCHAT_STATUS_ERROR;
  ncb::MemoryHub hub(world);
  if (drop_from >= 0 && world > 1) hub.DropNext(drop_from, (drop_from + 1) % world, 1);
  std::vector<char> ok(world, 1);
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r)
    threads.emplace_back([&, r] {
      auto link = hub.Endpoint(r);
      ok[r] = ncb::RingAllReduceSum(link.get(), data + static_cast<std::size_t>(r) * count,
                                    static_cast<std::size_t>(count), timeout_ms);
    });
  for (auto& t : threads) t.join();
  for (int r = 0; r < world; ++r)
    if (!ok[r]) {
      ncb_set_error("ncb_memory_ring_all_reduce: rank " + std::to_string(r) + " lost a peer");
      return NANOCHAT_STATUS_ERROR;
    }
  return NANOCHAT_STATUS_OK;
}

}  // extern "C"
