// C ABI of the CPU engine: model, optimizer, scoring, generation, evaluation (reference
// include/nanochat/capi.h:377-439, 571-617). Errors are reported through nanochat_last_error(); functions that
// return a value return NaN / 0 / null on failure.
#include <cmath>
#include <cstring>
#include <limits>
#include <stdexcept>

#include "capi_internal.h"
#include "engine.h"

struct nanochat_model {
  std::unique_ptr<ncb::CpuModel> model;       // the CPU engine, or
  std::unique_ptr<ncb::DeviceEngine> gpu;     // the engine of the selected CUDA device (exactly one of the two is set)
  const ncb::EngineConfig& config() const { return gpu ? gpu->config() : model->config(); }
  // storage that results handed to the caller point into; valid until the next call on the same model
  std::vector<std::vector<float>> score_nll, score_focus;
  std::vector<std::vector<int>> score_argmax;
  std::vector<int> seq_tokens, seq_lengths, seq_offsets;
  std::vector<std::uint8_t> seq_mask;
};
struct nanochat_optim {
  std::unique_ptr<ncb::CpuOptimizer> opt;   // null for a model on a CUDA device: its engine holds the optimizer
  nanochat_model* model = nullptr;
  int steps_done = 0;  // for nanochat_train_step, which does not take a step number
};

namespace {

const float kNaN = std::numeric_limits<float>::quiet_NaN();

template <typename F>
auto Guard(F&& f, decltype(f()) fallback) -> decltype(f()) {
  try {
    return f();
  } catch (const std::exception& e) {
    ncb_set_error(e.what());
    return fallback;
  }
}

void FillSequences(nanochat_model* m, const std::vector<ncb::GeneratedRow>& rows, nanochat_sequences* out) {
  m->seq_tokens.clear(), m->seq_mask.clear(), m->seq_lengths.clear(), m->seq_offsets.clear();
  for (const auto& r : rows) {
    m->seq_offsets.push_back(static_cast<int>(m->seq_tokens.size()));
    m->seq_lengths.push_back(static_cast<int>(r.tokens.size()));
    m->seq_tokens.insert(m->seq_tokens.end(), r.tokens.begin(), r.tokens.end());
    m->seq_mask.insert(m->seq_mask.end(), r.mask.begin(), r.mask.end());
  }
  out->count = static_cast<int>(rows.size());
  out->tokens = m->seq_tokens.data();
  out->mask = m->seq_mask.data();
  out->lengths = m->seq_lengths.data();
  out->offsets = m->seq_offsets.data();
}

// Weights between a host model and a device engine, parameter by parameter (both register the same names).
void CopyWeights(ncb::CpuModel* host, ncb::DeviceEngine* dev, bool to_device) {
  const auto& dp = dev->params();
  for (std::size_t i = 0; i < dp.size(); ++i) {
    const ncb::CpuParam* hp = host->Find(dp[i].name);
    if (hp == nullptr || hp->count != dp[i].count) throw std::runtime_error("parameter tables disagree at " + dp[i].name);
    if (to_device) {
      dev->WriteParam(i, false, 0, static_cast<std::int64_t>(hp->count), host->value(*hp));
    } else {
      dev->ReadParam(i, false, 0, static_cast<std::int64_t>(hp->count), host->value(*hp));
    }
  }
}

ncb::GenerateOptions ToOptions(const nanochat_generate_params& p) {
  ncb::GenerateOptions o;
  o.num_samples = p.num_samples > 0 ? p.num_samples : 1;
  o.max_tokens = p.max_tokens;
  o.temperature = p.temperature;
  o.top_k = p.top_k;
  o.seed = p.seed;
  o.stop_id = p.stop_id;
  o.bos_id = p.bos_id;
  if (p.stop_ids != nullptr) o.stop_ids.assign(p.stop_ids, p.stop_ids + o.num_samples);
  return o;
}

}  // namespace

extern "C" {

nanochat_model* nanochat_model_create(const nanochat_config* config, uint64_t seed) {
  if (config == nullptr) {
    ncb_set_error("nanochat_model_create: config is null");
    return nullptr;
  }
  ncb::EngineConfig cfg;
  static_cast<ncb::ModelConfig&>(cfg) = ncb_to_model_config(*config);
  cfg.short_window_override = ncb_short_window_override();
  std::string err;
  if (!cfg.Validate(&err)) {
    ncb_set_error("nanochat_model_create: " + err);
    return nullptr;
  }
  return Guard([&]() {
    auto m = std::make_unique<nanochat_model>();
    const int cuda = ncb_selected_cuda_device();
    if (cuda >= 0) {
      const ncb_gpu_library* lib = ncb_gpu();
      char err_text[512] = {0};
      ncb::DeviceEngine* e = lib != nullptr ? lib->create(&cfg, cuda, err_text, sizeof(err_text)) : nullptr;
      if (e == nullptr) throw std::runtime_error(std::string("nanochat_model_create: ") + (err_text[0] ? err_text : "no GPU engine"));
      m->gpu.reset(e);
      // the same initial weights as the CPU engine: drawn on the host from the seed, then uploaded
      ncb::CpuModel host(cfg);
      host.InitWeights(seed);
      CopyWeights(&host, m->gpu.get(), /*to_device=*/true);
    } else {
      m->model = std::make_unique<ncb::CpuModel>(cfg);
      m->model->InitWeights(seed);
    }
    return m.release();
  }, static_cast<nanochat_model*>(nullptr));
}
void nanochat_model_free(nanochat_model* model) { delete model; }

float nanochat_forward_loss(nanochat_model* model, const int* tokens, const int* targets, int batch, int seq) {
  if (model == nullptr || tokens == nullptr || targets == nullptr || batch <= 0 || seq <= 0) return kNaN;
  return Guard([&]() {
    return model->gpu ? model->gpu->ForwardLoss(tokens, targets, batch, seq, false)
                      : model->model->ForwardLoss(tokens, targets, batch, seq);
  }, kNaN);
}
namespace {
void BackwardOn(nanochat_model* model, float scale, const float* row_weights) {
  if (model == nullptr) return;
  Guard([&]() {
    if (model->gpu) model->gpu->Backward(scale, row_weights, 0.0); else model->model->Backward(scale, row_weights);
    return 0;
  }, 0);
}
}  // namespace
void nanochat_backward(nanochat_model* model) { BackwardOn(model, 1.0f, nullptr); }
void nanochat_backward_accumulate(nanochat_model* model, float scale) { BackwardOn(model, scale, nullptr); }
void nanochat_backward_weighted(nanochat_model* model, const float* row_weights, float scale) {
  BackwardOn(model, scale, row_weights);
}
void nanochat_zero_grad(nanochat_model* model) {
  if (model == nullptr) return;
  Guard([&]() {
    if (model->gpu) model->gpu->ZeroGrad(); else model->model->ZeroGrad();
    return 0;
  }, 0);
}
float nanochat_train_step(nanochat_model* model, nanochat_optim* optimizer, const int* tokens, const int* targets,
                          int batch, int seq) {
  if (model == nullptr) return kNaN;
  return Guard([&]() {
    if (model->gpu) {
      model->gpu->ZeroGrad();
      const float loss = model->gpu->ForwardBackward(tokens, targets, batch, seq, 1.0f);
      if (optimizer != nullptr) model->gpu->OptimStep(++optimizer->steps_done);
      return loss;
    }
    model->model->ZeroGrad();
    const float loss = model->model->ForwardLoss(tokens, targets, batch, seq);
    model->model->Backward(1.0f);
    if (optimizer != nullptr) optimizer->opt->Step(++optimizer->steps_done);
    return loss;
  }, kNaN);
}
// Forward and backward of one micro-batch in one call, gradients accumulated with `scale` (no zeroing, no optimizer
// step): on a CUDA device the LM head's forward and backward are fused per row chunk, which a separate
// nanochat_forward_loss + nanochat_backward_accumulate pair has to run twice. Returns the micro-batch loss.
float ncb_forward_backward(nanochat_model* model, const int* tokens, const int* targets, int batch, int seq, float scale) {
  if (model == nullptr || tokens == nullptr || targets == nullptr || batch <= 0 || seq <= 0) return kNaN;
  return Guard([&]() {
    if (model->gpu) return model->gpu->ForwardBackward(tokens, targets, batch, seq, scale);
    const float loss = model->model->ForwardLoss(tokens, targets, batch, seq);
    model->model->Backward(scale);
    return loss;
  }, kNaN);
}
float nanochat_rl_step(nanochat_model* model, nanochat_optim* optimizer, const int* tokens, const int* targets,
                       const float* advantages, int batch, int seq, int num_passes, int examples_per_rank, int step) {
  if (model == nullptr || tokens == nullptr || targets == nullptr || advantages == nullptr || batch <= 0 || seq <= 0 ||
      num_passes <= 0 || examples_per_rank <= 0) {
    ncb_set_error("nanochat_rl_step: invalid argument");
    return kNaN;
  }
  return Guard([&]() {
    if (model->gpu) {
      ncb::DeviceModelView view{model->gpu.get()};
      ncb::DeviceOptimView opt{model->gpu.get()};
      return ncb::RlStepOn(&view, optimizer ? &opt : static_cast<ncb::DeviceOptimView*>(nullptr), tokens, targets,
                           advantages, batch, seq, num_passes, examples_per_rank, step);
    }
    return ncb::RlStep(model->model.get(), optimizer ? optimizer->opt.get() : nullptr, tokens, targets, advantages, batch,
                       seq, num_passes, examples_per_rank, step);
  }, kNaN);
}

namespace {
const std::vector<ncb::CpuParam>& ParamsOf(nanochat_model* model) {
  return model->gpu ? model->gpu->params() : model->model->params();
}
}  // namespace

int nanochat_param_count(nanochat_model* model) {
  return model == nullptr ? 0 : static_cast<int>(ParamsOf(model).size());
}
// On a CUDA device `value` and `grad` are null: the weights live in device memory and are reached through
// nanochat_param_read / nanochat_param_write.
int nanochat_param_info(nanochat_model* model, int index, nanochat_param* out) {
  if (model == nullptr || out == nullptr || index < 0 || index >= nanochat_param_count(model)) return 0;
  const ncb::CpuParam& p = ParamsOf(model)[static_cast<std::size_t>(index)];
  out->name = p.name.c_str();
  out->value = model->gpu ? nullptr : model->model->value(p);
  out->grad = model->gpu ? nullptr : model->model->grad(p);
  out->count = static_cast<int64_t>(p.count);
  out->rows = p.rows, out->cols = p.cols;
  return 1;
}
int64_t nanochat_param_read(nanochat_model* model, int index, int grad, int64_t offset, int64_t count, void* data) {
  if (model == nullptr || data == nullptr || index < 0 || index >= nanochat_param_count(model)) return 0;
  const ncb::CpuParam& p = ParamsOf(model)[static_cast<std::size_t>(index)];
  if (offset < 0 || offset >= static_cast<int64_t>(p.count)) return 0;
  const int64_t n = std::min<int64_t>(count, static_cast<int64_t>(p.count) - offset);
  if (model->gpu) {
    return Guard([&]() {
      model->gpu->ReadParam(static_cast<std::size_t>(index), grad != 0, offset, n, static_cast<float*>(data));
      return n;
    }, static_cast<int64_t>(0));
  }
  const float* src = (grad ? model->model->grad(p) : model->model->value(p)) + offset;
  std::memcpy(data, src, static_cast<std::size_t>(n) * sizeof(float));
  return n;
}
int64_t nanochat_param_write(nanochat_model* model, int index, int grad, int64_t offset, int64_t count,
                             const void* data) {
  if (model == nullptr || data == nullptr || index < 0 || index >= nanochat_param_count(model)) return 0;
  const ncb::CpuParam& p = ParamsOf(model)[static_cast<std::size_t>(index)];
  if (offset < 0 || offset >= static_cast<int64_t>(p.count)) return 0;
  const int64_t n = std::min<int64_t>(count, static_cast<int64_t>(p.count) - offset);
  if (model->gpu) {
    return Guard([&]() {
      model->gpu->WriteParam(static_cast<std::size_t>(index), grad != 0, offset, n, static_cast<const float*>(data));
      return n;
    }, static_cast<int64_t>(0));
  }
  float* dst = (grad ? model->model->grad(p) : model->model->value(p)) + offset;
  std::memcpy(dst, data, static_cast<std::size_t>(n) * sizeof(float));
  return n;
}
// A model on a CUDA device is saved and loaded through a host copy of its weights (the same container either way).
void nanochat_save(nanochat_model* model, const char* path) {
  std::string err;
  if (model == nullptr || path == nullptr) {
    ncb_set_error("nanochat_save: null argument");
    return;
  }
  Guard([&]() {
    if (model->gpu) {
      ncb::CpuModel host(model->gpu->config());
      CopyWeights(&host, model->gpu.get(), false);
      if (!host.Save(path, &err)) ncb_set_error("nanochat_save: " + err);
    } else if (!model->model->Save(path, &err)) {
      ncb_set_error("nanochat_save: " + err);
    }
    return 0;
  }, 0);
}
void nanochat_load(nanochat_model* model, const char* path) {
  std::string err;
  if (model == nullptr || path == nullptr) {
    ncb_set_error("nanochat_load: null argument");
    return;
  }
  Guard([&]() {
    if (model->gpu) {
      ncb::CpuModel host(model->gpu->config());
      if (!host.Load(path, &err)) {
        ncb_set_error("nanochat_load: " + err);
      } else {
        CopyWeights(&host, model->gpu.get(), true);
      }
    } else if (!model->model->Load(path, &err)) {
      ncb_set_error("nanochat_load: " + err);
    }
    return 0;
  }, 0);
}

nanochat_optim* nanochat_optim_create(nanochat_model* model, const nanochat_optim_config* c) {
  if (model == nullptr || c == nullptr) return nullptr;
  ncb::OptimConfig o;
  o.unembedding_lr = c->unembedding_lr, o.embedding_lr = c->embedding_lr, o.matrix_lr = c->matrix_lr;
  o.scalar_lr = c->scalar_lr, o.weight_decay = c->weight_decay, o.muon_ns_steps = c->muon_ns_steps;
  o.muon_beta2 = c->muon_beta2, o.adam_eps = c->adam_eps, o.clip = c->clip;
  o.num_iterations = c->num_iterations, o.warmup_steps = c->warmup_steps, o.warmdown_ratio = c->warmdown_ratio;
  o.final_lr_frac = c->final_lr_frac, o.weight_decay_base = c->weight_decay_base;
  o.muon_momentum_warmup_steps = c->muon_momentum_warmup_steps, o.muon_momentum_start = c->muon_momentum_start;
  o.muon_momentum_peak = c->muon_momentum_peak, o.muon_momentum_final = c->muon_momentum_final;
  return Guard([&]() {
    auto h = std::make_unique<nanochat_optim>();
    if (model->gpu) {
      model->gpu->OptimInit(o);
    } else {
      h->opt = std::make_unique<ncb::CpuOptimizer>(model->model.get(), o);
    }
    h->model = model;
    return h.release();
  }, static_cast<nanochat_optim*>(nullptr));
}
void nanochat_optim_step(nanochat_optim* optimizer, int step) {
  if (optimizer == nullptr) return;
  Guard([&]() {
    if (optimizer->opt) optimizer->opt->Step(step); else optimizer->model->gpu->OptimStep(step);
    return 0;
  }, 0);
  optimizer->steps_done = step;
}
float nanochat_optim_grad_norm(nanochat_optim* optimizer) {
  if (optimizer == nullptr) return 0.0f;
  return optimizer->opt ? optimizer->opt->grad_norm() : optimizer->model->gpu->grad_norm();
}
void nanochat_optim_free(nanochat_optim* optimizer) { delete optimizer; }

void nanochat_score_batch(nanochat_model* model, const int* tokens, int batch, int seq, const int* lengths,
                          const nanochat_focus* focus, nanochat_score_result* out) {
  if (model == nullptr || tokens == nullptr || out == nullptr || batch <= 0 || seq <= 0) return;
  Guard([&]() {
    std::vector<ncb::FocusRequest> req;
    if (focus != nullptr) {
      req.resize(static_cast<std::size_t>(batch));
      for (int b = 0; b < batch; ++b) {
        req[b].position = focus[b].position;
        if (focus[b].ids != nullptr && focus[b].count > 0) req[b].ids.assign(focus[b].ids, focus[b].ids + focus[b].count);
        if (req[b].ids.empty()) req[b].position = -1;
      }
    }
    ncb::DeviceModelView view{model->gpu.get()};
    auto rows = model->gpu ? ncb::ScoreBatchOn(&view, tokens, batch, seq, lengths, focus ? req.data() : nullptr)
                           : ncb::ScoreBatch(model->model.get(), tokens, batch, seq, lengths, focus ? req.data() : nullptr);
    model->score_nll.resize(rows.size()), model->score_argmax.resize(rows.size()), model->score_focus.resize(rows.size());
    for (std::size_t b = 0; b < rows.size(); ++b) {
      model->score_nll[b] = std::move(rows[b].nll);
      model->score_argmax[b] = std::move(rows[b].argmax);
      model->score_focus[b] = std::move(rows[b].focus_logits);
      out[b].nll = model->score_nll[b].data();
      out[b].argmax = model->score_argmax[b].data();
      out[b].focus_logits = model->score_focus[b].empty() ? nullptr : model->score_focus[b].data();
    }
    return 0;
  }, 0);
}

void nanochat_generate(nanochat_model* model, const int* prompt, int length, const nanochat_generate_params* params,
                       nanochat_sequences* out) {
  if (model == nullptr || prompt == nullptr || params == nullptr || out == nullptr || length <= 0) return;
  Guard([&]() {
    ncb::DeviceModelView view{model->gpu.get()};
    FillSequences(model, model->gpu ? ncb::GenerateBatchOn(&view, prompt, length, ToOptions(*params))
                                    : ncb::GenerateBatch(model->model.get(), prompt, length, ToOptions(*params)), out);
    return 0;
  }, 0);
}

void nanochat_generate_multi(nanochat_model* model, const int* prompts, const nanochat_generate_multi_params* params,
                             nanochat_sequences* out) {
  if (model == nullptr || prompts == nullptr || params == nullptr || out == nullptr || params->num_prompts <= 0 ||
      params->prompt_len <= 0)
    return;
  Guard([&]() {
    std::vector<ncb::GeneratedRow> all;
    ncb::GenerateOptions base = ToOptions(params->params);
    const int S = base.num_samples;
    for (int p = 0; p < params->num_prompts; ++p) {
      ncb::GenerateOptions o = base;
      if (params->row_stops != nullptr) o.stop_ids.assign(params->row_stops + p * S, params->row_stops + (p + 1) * S);
      ncb::DeviceModelView view{model->gpu.get()};
      const int* prompt = prompts + static_cast<std::size_t>(p) * params->prompt_len;
      auto rows = model->gpu ? ncb::GenerateBatchOn(&view, prompt, params->prompt_len, o, p * S)
                             : ncb::GenerateBatch(model->model.get(), prompt, params->prompt_len, o, p * S);
      for (auto& r : rows) all.push_back(std::move(r));
    }
    FillSequences(model, all, out);
    return 0;
  }, 0);
}

// First bounded-wait failure recorded by a kernel of the model's device (0 = none, always 0 on the CPU), and the
// number of kernel launches the model's engine has issued so far.
int ncb_model_device_status(nanochat_model* model) {
  if (model == nullptr || !model->gpu) return 0;
  return Guard([&]() { return model->gpu->Status(); }, -1);
}
int64_t ncb_model_launch_count(nanochat_model* model) {
  return model != nullptr && model->gpu ? model->gpu->LaunchCount() : 0;
}

// An activation of the model's last forward on a CUDA device, widened to fp32 (see DeviceEngine::ReadActivation).
// Returns the element count (the copy is truncated to `capacity`), or -1 for an unknown name or a CPU model.
int64_t ncb_model_read_activation(nanochat_model* model, const char* name, int layer, float* dst, int64_t capacity) {
  if (model == nullptr || !model->gpu || name == nullptr) return -1;
  return Guard([&]() {
    std::vector<float> v;
    if (!model->gpu->ReadActivation(name, layer, &v)) return static_cast<int64_t>(-1);
    if (dst != nullptr && capacity > 0)
      std::memcpy(dst, v.data(), static_cast<std::size_t>(std::min<int64_t>(capacity, static_cast<int64_t>(v.size()))) * sizeof(float));
    return static_cast<int64_t>(v.size());
  }, static_cast<int64_t>(-1));
}

float nanochat_eval_bpb(nanochat_model* model, nanochat_loader* loader, int steps) {
  const float inf = std::numeric_limits<float>::infinity();
  if (model == nullptr || loader == nullptr || steps <= 0 || loader->batch <= 0 || loader->seq <= 0) return inf;
  return Guard([&]() {
    const std::size_t rows = static_cast<std::size_t>(loader->batch) * loader->seq;
    std::vector<int> tokens(rows), targets(rows);
    int vocab = 0;
    const uint8_t* bytes = nanochat_loader_token_bytes(loader, &vocab);
    double nats = 0.0;
    long long total = 0;
    for (int s = 0; s < steps; ++s) {
      if (!nanochat_loader_next(loader, tokens.data(), targets.data())) break;
      if (model->gpu) {
        model->gpu->ForwardLoss(tokens.data(), targets.data(), loader->batch, loader->seq, false);
      } else {
        model->model->ForwardLoss(tokens.data(), targets.data(), loader->batch, loader->seq);
      }
      const std::vector<float>& losses = model->gpu ? model->gpu->losses() : model->model->losses();
      for (std::size_t i = 0; i < rows; ++i) {
        const int t = targets[i];
        if (t < 0) continue;
        const int b = bytes != nullptr ? (t < vocab ? bytes[t] : 0) : 1;
        if (b <= 0) continue;
        nats += losses[i];
        total += b;
      }
    }
    return total == 0 ? inf : static_cast<float>(nats / (std::log(2.0) * static_cast<double>(total)));
  }, inf);
}

}  // extern "C"
