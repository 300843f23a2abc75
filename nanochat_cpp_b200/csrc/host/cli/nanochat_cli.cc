// nanochat_cli: a native command line over the C ABI (include/nanochat/capi.h) for hosts without Python or a GPU.
// It runs the CPU engine: `train` (the in-process mesh driver), `generate`, `eval` (bits per byte), `score` and `rl_step`
// (fixtures), `tok_train`, `params`, `roofline`. Flag names follow the Python entry point (`python -m nanochat_cpp_b200.cli`), which follows the
// reference's `nanochat_cli` (src/train_command.cc:27-61, src/generate_command.cc:37-50, src/eval_command.cc:42-54).
// The GPU path is driven from Python; this binary links only libnanochat_core.
//
// Environment contract of the reference's binaries (include/nanochat/sandbox.h): they refuse to start outside their
// sandbox. Here the check is opt-in: with NANOCHAT_SANDBOX_ENFORCE=1 the binary exits unless NANOCHAT_SANDBOX names
// a profile; otherwise the variable is only echoed in `--version`.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <ctime>
#include <cstdlib>
#include <cstring>
#include <csignal>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include <sys/wait.h>
#include <unistd.h>

#include "nanochat/capi.h"

namespace {

struct Args {
  std::map<std::string, std::vector<std::string>> values;
  bool Has(const std::string& k) const { return values.count(k) != 0; }
  std::string Str(const std::string& k, const std::string& d = "") const {
    auto it = values.find(k);
    return it == values.end() || it->second.empty() ? d : it->second.back();
  }
  long long Int(const std::string& k, long long d) const { return Has(k) ? std::atoll(Str(k).c_str()) : d; }
  double Num(const std::string& k, double d) const { return Has(k) ? std::atof(Str(k).c_str()) : d; }
  const std::vector<std::string>& All(const std::string& k) const {
    static const std::vector<std::string> none;
    auto it = values.find(k);
    return it == values.end() ? none : it->second;
  }
};

// `--key value`, `--key=value`, bare `--flag` (value "1"); a key may repeat.
Args Parse(int argc, char** argv, int first) {
  Args a;
  for (int i = first; i < argc; ++i) {
    std::string s = argv[i];
    if (s.rfind("--", 0) != 0) {
      a.values["_"].push_back(s);
      continue;
    }
    s = s.substr(2);
    const auto eq = s.find('=');
    if (eq != std::string::npos) {
      a.values[s.substr(0, eq)].push_back(s.substr(eq + 1));
    } else if (i + 1 < argc && std::strncmp(argv[i + 1], "--", 2) != 0) {
      a.values[s].push_back(argv[++i]);
    } else {
      a.values[s].push_back("1");
    }
  }
  return a;
}

int Fail(const char* what) {
  const char* e = nanochat_last_error();
  std::fprintf(stderr, "nanochat_cli: %s%s%s\n", what, e && *e ? ": " : "", e ? e : "");
  return 1;
}

// Model flags; `--preset-model` picks a named shape, `--depth N` derives hidden = 64 N rounded up to 128 per head.
std::string g_pattern;
nanochat_config ModelFromArgs(const Args& a) {
  nanochat_config c{};
  c.num_layers = 12, c.num_heads = 6, c.hidden_dim = 768, c.seq_len = 2048, c.vocab_size = 32768;
  const std::string preset = a.Str("preset-model");
  if (preset == "tiny") c.num_layers = 2, c.num_heads = 2, c.hidden_dim = 64, c.seq_len = 64, c.vocab_size = 512;
  else if (preset == "d12") c.num_layers = 12, c.num_heads = 6, c.hidden_dim = 768, c.vocab_size = 32768;
  else if (preset == "d20") c.num_layers = 20, c.num_heads = 10, c.hidden_dim = 1280, c.vocab_size = 65536;
  else if (preset == "d26") c.num_layers = 26, c.num_heads = 13, c.hidden_dim = 1664, c.vocab_size = 65536;
  if (a.Has("depth")) {
    const int d = static_cast<int>(a.Int("depth", 12));
    c.num_layers = d;
    c.hidden_dim = (d * 64 + 127) / 128 * 128;
    c.num_heads = c.hidden_dim / 128;
  }
  c.num_layers = static_cast<int>(a.Int("layers", c.num_layers));
  c.num_heads = static_cast<int>(a.Int("heads", c.num_heads));
  c.hidden_dim = static_cast<int>(a.Int("hidden", c.hidden_dim));
  c.seq_len = static_cast<int>(a.Int("seq", c.seq_len));
  c.vocab_size = static_cast<int>(a.Int("vocab", c.vocab_size));
  c.num_kv_heads = static_cast<int>(a.Int("kv-heads", 0));
  if (c.num_kv_heads <= 0) c.num_kv_heads = c.num_heads;
  c.padded_vocab_size = static_cast<int>(a.Int("padded-vocab", 0));
  if (c.padded_vocab_size <= 0) c.padded_vocab_size = (c.vocab_size + 63) / 64 * 64;
  c.rope_base = static_cast<float>(a.Num("rope-base", 100000.0));
  g_pattern = a.Str("window-pattern", "SSSL");
  c.window_pattern = g_pattern.c_str();
  c.value_embedding = a.Has("no-value-embedding") ? 0 : 1;
  // the d12/d20/d26 presets are the benchmark shapes: 1024-token sliding window at seq 2048
  const bool bench_shape = preset == "d12" || preset == "d20" || preset == "d26";
  ncb_set_short_window(static_cast<int>(a.Int("short-window", bench_shape ? 1024 : 0)));
  return c;
}

// Shape of the model stored in a checkpoint (its metadata block), for commands that continue from one: explicit
// model flags still win. Returns false when the file has no readable metadata.
bool ConfigFromCheckpoint(const std::string& path, nanochat_config* c) {
  nanochat_checkpoint* owner = nullptr;
  nanochat_checkpoint_metadata meta{};
  if (nanochat_checkpoint_metadata_read(path.c_str(), &owner, &meta) != NANOCHAT_STATUS_OK) return false;
  const char* js = nanochat_checkpoint_metadata_config_json(&meta);
  const std::string j = js != nullptr ? js : "";
  auto num = [&](const char* key, double d) {
    const auto k = j.find(std::string("\"") + key + "\":");
    return k == std::string::npos ? d : std::atof(j.c_str() + k + std::strlen(key) + 3);
  };
  c->num_layers = static_cast<int>(num("num_layers", c->num_layers));
  c->num_heads = static_cast<int>(num("num_heads", c->num_heads));
  c->num_kv_heads = static_cast<int>(num("num_kv_heads", c->num_kv_heads));
  c->hidden_dim = static_cast<int>(num("hidden_dim", c->hidden_dim));
  c->seq_len = static_cast<int>(num("seq_len", c->seq_len));
  c->vocab_size = static_cast<int>(num("vocab_size", c->vocab_size));
  c->padded_vocab_size = static_cast<int>(num("padded_vocab_size", c->padded_vocab_size));
  c->rope_base = static_cast<float>(num("rope_base", c->rope_base));
  const auto w = j.find("\"window_pattern\": \"");
  if (w != std::string::npos) {
    const auto b = w + std::strlen("\"window_pattern\": \"");
    g_pattern = j.substr(b, j.find('"', b) - b);
    c->window_pattern = g_pattern.c_str();
  }
  c->value_embedding = j.find("\"value_embedding\": false") == std::string::npos ? 1 : 0;
  nanochat_checkpoint_free(owner);
  // Files written through the plain C ABI carry default metadata: when the tensor shapes disagree with it, the shapes win.
  owner = nullptr;
  const nanochat_record* recs = nullptr;
  int64_t n = 0;
  if (nanochat_checkpoint_read(path.c_str(), &owner, &recs, &n, nullptr, nullptr) == NANOCHAT_STATUS_OK) {
    auto find = [&](const std::string& name) -> const nanochat_record* {
      for (int64_t i = 0; i < n; ++i)
        if (name == recs[i].name) return &recs[i];
      return nullptr;
    };
    auto ends_with = [](const std::string& v, const char* suffix) {
      const size_t k = std::strlen(suffix);
      return v.size() >= k && v.compare(v.size() - k, k, suffix) == 0;
    };
    const nanochat_record* lm = find("lm_head.weight");
    const nanochat_record* cq = find("transformer.h.0.attn.c_q.weight");
    const nanochat_record* ck = find("transformer.h.0.attn.c_k.weight");
    if (lm != nullptr && cq != nullptr && ck != nullptr && lm->ndim == 2) {
      int layers = 0;
      const nanochat_record* gate = nullptr;
      for (int64_t i = 0; i < n; ++i) {
        if (ends_with(recs[i].name, "attn.c_q.weight")) ++layers;
        if (gate == nullptr && ends_with(recs[i].name, "attn.ve_gate.weight")) gate = &recs[i];
      }
      const int padded = static_cast<int>(lm->dims[0]), hidden = static_cast<int>(lm->dims[1]);
      const int q_dim = static_cast<int>(cq->dims[0]), kv_dim = static_cast<int>(ck->dims[0]);
      const int base_head = c->num_heads > 0 ? c->hidden_dim / c->num_heads : 128;
      const bool consistent = c->hidden_dim == hidden && c->padded_vocab_size == padded && c->num_layers == layers &&
                              c->num_heads * base_head == q_dim && c->num_kv_heads * base_head == kv_dim;
      if (!consistent) {
        int kv_heads, head_dim;
        if (gate != nullptr) {
          kv_heads = static_cast<int>(gate->dims[0]);
          head_dim = kv_dim / kv_heads;
        } else {
          head_dim = q_dim % 128 == 0 ? 128 : q_dim % 64 == 0 ? 64 : base_head;
          kv_heads = kv_dim / head_dim;
        }
        if (!(c->vocab_size <= padded && c->padded_vocab_size == padded)) c->vocab_size = padded;
        c->num_layers = layers, c->num_heads = q_dim / head_dim, c->num_kv_heads = kv_heads, c->hidden_dim = hidden;
        c->padded_vocab_size = padded, c->value_embedding = gate != nullptr ? 1 : 0;
      }
    }
    nanochat_checkpoint_free(owner);
  }
  return c->num_layers > 0 && c->hidden_dim > 0;
}

bool OptimFromArgs(const Args& a, nanochat_optim_config* o, const char* default_preset = "default") {
  if (nanochat_optim_config_preset(a.Str("preset", default_preset).c_str(), o) != NANOCHAT_STATUS_OK) return false;
  o->embedding_lr = static_cast<float>(a.Num("embedding-lr", o->embedding_lr));
  o->unembedding_lr = static_cast<float>(a.Num("unembedding-lr", o->unembedding_lr));
  o->matrix_lr = static_cast<float>(a.Num("matrix-lr", o->matrix_lr));
  o->scalar_lr = static_cast<float>(a.Num("scalar-lr", o->scalar_lr));
  o->weight_decay = static_cast<float>(a.Num("weight-decay", o->weight_decay));
  o->weight_decay_base = static_cast<float>(a.Num("weight-decay-base", o->weight_decay_base));
  o->clip = static_cast<float>(a.Num("clip", o->clip));
  o->adam_eps = static_cast<float>(a.Num("adam-eps", o->adam_eps));
  o->muon_ns_steps = static_cast<int>(a.Int("muon-ns-steps", o->muon_ns_steps));
  o->muon_beta2 = static_cast<float>(a.Num("muon-beta2", o->muon_beta2));
  o->warmup_steps = static_cast<int>(a.Int("warmup-steps", o->warmup_steps));
  o->warmdown_ratio = static_cast<float>(a.Num("warmdown-ratio", o->warmdown_ratio));
  o->final_lr_frac = static_cast<float>(a.Num("final-lr-frac", o->final_lr_frac));
  o->muon_momentum_warmup_steps = static_cast<float>(a.Num("muon-momentum-warmup-steps", o->muon_momentum_warmup_steps));
  o->muon_momentum_start = static_cast<float>(a.Num("muon-momentum-start", o->muon_momentum_start));
  o->muon_momentum_peak = static_cast<float>(a.Num("muon-momentum-peak", o->muon_momentum_peak));
  o->muon_momentum_final = static_cast<float>(a.Num("muon-momentum-final", o->muon_momentum_final));
  o->num_iterations = static_cast<int>(a.Int("num-iterations", 100));
  return true;
}

int CmdTrain(const Args& a, const char* default_preset = "default") {
  nanochat_mesh_train_config c{};
  c.model = ModelFromArgs(a);
  // continuing from a checkpoint without naming a shape: take the shape the checkpoint records
  const bool shape_given = a.Has("preset-model") || a.Has("depth") || a.Has("layers") || a.Has("hidden") || a.Has("heads");
  if (!shape_given && a.Has("warm-start")) ConfigFromCheckpoint(a.Str("warm-start"), &c.model);
  nanochat_optim_config optim;
  if (!OptimFromArgs(a, &optim, default_preset)) return Fail("train");
  c.optimizer = &optim;
  nanochat_mesh* mesh = nanochat_mesh_create(nullptr, static_cast<int>(a.Int("mesh", 1)));
  c.mesh = mesh;
  std::vector<const char*> parquet;
  for (const std::string& p : a.All("train-parquet")) parquet.push_back(p.c_str());
  c.data.parquet = parquet.data();
  c.data.parquet_count = static_cast<int>(parquet.size());
  const std::string tok = a.Str("tokenizer"), rows = a.Str("rows"), warm = a.Str("warm-start");
  const std::string out_dir = a.Str("out-dir", "."), ckpt = a.Str("checkpoint");
  c.data.tokenizer_path = tok.c_str();
  c.data.packed_rows_path = rows.c_str();
  c.warm_start_path = warm.c_str();
  c.run.batch = static_cast<int>(a.Int("batch", 8));
  c.run.grad_accum = static_cast<int>(a.Int("grad-accum", 1));
  c.run.seq = static_cast<int>(a.Int("train-seq", 0));
  if (c.run.seq == 0 && !rows.empty()) {   // packed rows fix the row length: take it from the shard
    ncb_record_file* shard = nullptr;
    const nanochat_record* srecs = nullptr;
    int64_t sn = 0;
    char smagic[9];
    if (ncb_record_file_read(rows.c_str(), &shard, smagic, &srecs, &sn) == NANOCHAT_STATUS_OK) {
      for (int64_t i = 0; i < sn; ++i)
        if (std::strcmp(srecs[i].name, "tokens") == 0 && srecs[i].ndim == 2) c.run.seq = static_cast<int>(srecs[i].dims[1]);
      ncb_record_file_free(shard);
    }
  }
  c.run.seed = static_cast<uint64_t>(a.Int("seed", 42));
  c.run.num_iterations = static_cast<int>(a.Int("num-iterations", 100));
  c.run.log_every = static_cast<int>(a.Int("log-every", 10));
  c.run.save_every = static_cast<int>(a.Int("save-every", 0));
  c.run.resume = a.Has("resume") ? 1 : 0;
  c.peak_flops = a.Num("peak-flops", 0.0);
  c.output.out_dir = out_dir.c_str();
  c.output.checkpoint_path = ckpt.c_str();
  nanochat_mesh_train_summary s{};
  // multi-process data parallelism: flags or the launcher's environment (NANOCHAT_RANK / _WORLD_SIZE / _MASTER_PORT)
  auto env_int = [](const char* name, long long d) {
    const char* v = std::getenv(name);
    return v != nullptr && *v ? std::atoll(v) : d;
  };
  const int world = static_cast<int>(a.Int("world-size", env_int("NANOCHAT_WORLD_SIZE", 1)));
  const int rank = static_cast<int>(a.Int("rank", env_int("NANOCHAT_RANK", 0)));
  const int port = static_cast<int>(a.Int("port", env_int("NANOCHAT_MASTER_PORT", 29500)));
  const float last = world > 1 ? ncb_dist_train_run(&c, rank, world, port, static_cast<int>(a.Int("timeout-ms", 0)), &s)
                               : nanochat_mesh_train_run(&c, &s);
  nanochat_mesh_free(mesh);
  if (world > 1 && rank != 0) return (s.steps == 0 && last == 0.0f) ? Fail("train") : 0;
  if (s.steps == 0 && last == 0.0f) return Fail("train");
  std::printf("[nanochat] %d steps%s, mean loss %.6f, last loss %.6f, checkpoint %s\n", s.steps,
              s.interrupted ? " (interrupted)" : "", s.mean_loss, last, s.checkpoint);
  return 0;
}

// `train --device cuda:N`: the training loop on the C++ GPU engine through the C ABI (one process, one GPU). Data:
// `--train-parquet ... --tokenizer T`, or `--synthetic-zipf S` (Zipf(S) token ids, no files). Each step runs
// `--grad-accum` micro-batches of `--batch` rows; every `--log-every` steps it prints the reference's log line
// (src/train.cc:74-101: step | loss | lr | grad_norm | tok/s | mfu | ... | step_ms | ...).
int CmdTrainDevice(const Args& a) {
  nanochat_config cfg = ModelFromArgs(a);
  nanochat_optim_config optim;
  if (!OptimFromArgs(a, &optim, "default")) return Fail("train");
  const int batch = static_cast<int>(a.Int("batch", 8)), accum = std::max(1, static_cast<int>(a.Int("grad-accum", 1)));
  const int seq = static_cast<int>(a.Int("train-seq", cfg.seq_len)), iters = static_cast<int>(a.Int("num-iterations", 100));
  const int log_every = static_cast<int>(a.Int("log-every", 10));
  optim.num_iterations = optim.num_iterations > 0 ? optim.num_iterations : iters;
  nanochat_tokenizer* tok = nullptr;
  nanochat_loader* loader = nullptr;
  if (a.Has("synthetic-zipf")) {
    loader = ncb_loader_zipf(cfg.vocab_size, seq, a.Num("synthetic-zipf", 1.1), static_cast<uint64_t>(a.Int("seed", 42)),
                             batch, seq, static_cast<size_t>(a.Int("buffer-docs", 1000)));
  } else {
    tok = nanochat_tokenizer_load(a.Str("tokenizer").c_str());
    if (tok == nullptr) return Fail("train: tokenizer");
    std::vector<const char*> parquet;
    for (const std::string& p : a.All("train-parquet")) parquet.push_back(p.c_str());
    loader = nanochat_loader_create(parquet.data(), static_cast<int>(parquet.size()), a.Str("text-column", "text").c_str(),
                                    tok, batch, seq, static_cast<uint64_t>(a.Int("seed", 42)),
                                    static_cast<int>(a.Int("tokenizer-threads", 4)),
                                    static_cast<size_t>(a.Int("buffer-docs", 1000)));
  }
  if (loader == nullptr) return Fail("train: loader");
  nanochat_model* m = nanochat_model_create(&cfg, static_cast<uint64_t>(a.Int("seed", 42)));
  if (m == nullptr) return Fail("train: model");
  if (a.Has("warm-start")) nanochat_load(m, a.Str("warm-start").c_str());
  nanochat_optim* opt = nanochat_optim_create(m, &optim);
  if (opt == nullptr) return Fail("train: optimizer");
  nanochat_params counts{};
  nanochat_params_get(&cfg, &counts);
  const double peak = a.Num("peak-flops", 0.0);
  std::vector<int> tokens(static_cast<std::size_t>(batch) * seq), targets(tokens.size());
  double window_s = 0.0, loss_sum = 0.0, last = 0.0;
  int window_steps = 0;
  for (int step = 1; step <= iters; ++step) {
    const auto t0 = std::chrono::steady_clock::now();
    double loss = 0.0;
    nanochat_zero_grad(m);
    for (int k = 0; k < accum; ++k) {
      if (!nanochat_loader_next(loader, tokens.data(), targets.data())) break;
      loss += ncb_forward_backward(m, tokens.data(), targets.data(), batch, seq, 1.0f / static_cast<float>(accum)) / accum;
    }
    nanochat_optim_step(opt, step);
    if (!(loss == loss)) return Fail("train: the loss is not a number");
    window_s += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    ++window_steps;
    loss_sum += loss;
    last = loss;
    if ((log_every > 0 && step % log_every == 0) || step == iters) {
      const double step_s = window_s / window_steps, tok_s = static_cast<double>(batch) * seq * accum / step_s;
      std::printf("step %06d | loss %.6f | lr %.6g | grad_norm %.6g | tok/s %.3f | mfu %.2f%% | model_tflops %.3f | "
                  "optim_tflops %.3f | step_ms %.3f | data_ms 0.000 | fwd_ms 0.000 | bwd_ms 0.000 | sync_ms 0.000 | "
                  "opt_ms 0.000 | eval_ms 0.000\n",
                  step, loss, static_cast<double>(optim.matrix_lr), static_cast<double>(nanochat_optim_grad_norm(opt)),
                  tok_s, peak > 0 ? 100.0 * tok_s * counts.flops_per_token / peak : 0.0,
                  tok_s * counts.flops_per_token / 1e12,
                  ncb_muon_flops_per_step(&cfg, optim.muon_ns_steps) / step_s / 1e12, step_s * 1e3);
      std::fflush(stdout);
      window_s = 0.0, window_steps = 0;
    }
  }
  const int status = ncb_model_device_status(m);
  if (status != 0) {
    std::fprintf(stderr, "nanochat_cli train: a kernel gave up waiting (status %d); not saving\n", status);
    return 1;
  }
  if (a.Has("checkpoint")) nanochat_save(m, a.Str("checkpoint").c_str());
  std::printf("[nanochat] %d steps on %s, mean loss %.6f, last loss %.6f, kernel launches %lld\n", iters,
              nanochat_backend(), loss_sum / std::max(1, iters), last, static_cast<long long>(ncb_model_launch_count(m)));
  nanochat_optim_free(opt);
  nanochat_model_free(m);
  nanochat_loader_free(loader);
  if (tok != nullptr) nanochat_tokenizer_free(tok);
  return 0;
}

nanochat_model* LoadModel(const Args& a, nanochat_config* cfg) {
  *cfg = ModelFromArgs(a);
  nanochat_model* m = nanochat_model_create(cfg, static_cast<uint64_t>(a.Int("seed", 42)));
  if (m != nullptr && a.Has("model")) {
    nanochat_load(m, a.Str("model").c_str());
    const char* e = nanochat_last_error();
    if (e != nullptr && *e) {
      nanochat_model_free(m);
      return nullptr;
    }
  }
  return m;
}

int CmdGenerate(const Args& a) {
  nanochat_config cfg;
  nanochat_model* m = LoadModel(a, &cfg);
  if (m == nullptr) return Fail("generate");
  nanochat_tokenizer* tok = a.Has("tokenizer") ? nanochat_tokenizer_load(a.Str("tokenizer").c_str()) : nullptr;
  std::vector<int> prompt;
  if (a.Has("tokens")) {
    const std::string s = a.Str("tokens");
    for (std::size_t i = 0; i < s.size();) {
      std::size_t j = s.find(',', i);
      if (j == std::string::npos) j = s.size();
      prompt.push_back(std::atoi(s.substr(i, j - i).c_str()));
      i = j + 1;
    }
  } else if (tok != nullptr) {
    const std::string text = a.Str("prompt");
    prompt.resize(text.size() + 8);
    const int n = nanochat_encode(tok, text.c_str(), prompt.data(), static_cast<int>(prompt.size()));
    prompt.resize(static_cast<std::size_t>(n > 0 ? n : 0));
    const int bos = ncb_tokenizer_special_id(tok, "<|bos|>");
    if (bos >= 0) prompt.insert(prompt.begin(), bos);
  }
  if (prompt.empty()) {
    std::fprintf(stderr, "nanochat_cli generate: give --tokens a,b,c or --tokenizer with --prompt\n");
    return 2;
  }
  nanochat_generate_params p{};
  p.num_samples = static_cast<int>(a.Int("num-samples", 1));
  p.max_tokens = static_cast<int>(a.Int("max-tokens", 32));
  p.temperature = static_cast<float>(a.Num("temperature", 0.0));
  p.top_k = static_cast<int>(a.Int("top-k", 0));
  p.seed = static_cast<uint64_t>(a.Int("seed", 42));
  p.stop_id = static_cast<int>(a.Int("stop-id", -1));
  p.bos_id = static_cast<int>(a.Int("bos-id", -1));
  nanochat_sequences out{};
  nanochat_generate(m, prompt.data(), static_cast<int>(prompt.size()), &p, &out);
  for (int r = 0; r < out.count; ++r) {
    const int* row = out.tokens + out.offsets[r];
    const int len = out.lengths[r];
    if (tok != nullptr) {
      std::vector<char> text(static_cast<std::size_t>(len) * 16 + 16);
      const int n = nanochat_decode(tok, row, len, text.data(), static_cast<int>(text.size()));
      std::printf("%.*s\n", n > 0 ? n : 0, text.data());
    } else {
      for (int i = 0; i < len; ++i) std::printf("%s%d", i ? "," : "", row[i]);
      std::printf("\n");
    }
  }
  if (tok) nanochat_tokenizer_free(tok);
  nanochat_model_free(m);
  return 0;
}

int CmdEval(const Args& a) {
  nanochat_config cfg;
  nanochat_model* m = LoadModel(a, &cfg);
  if (m == nullptr) return Fail("eval");
  nanochat_tokenizer* tok = nanochat_tokenizer_load(a.Str("tokenizer").c_str());
  if (tok == nullptr) return Fail("eval: tokenizer");
  std::vector<const char*> parquet;
  for (const std::string& p : a.All("val-parquet")) parquet.push_back(p.c_str());
  const int batch = static_cast<int>(a.Int("batch", 8)), seq = static_cast<int>(a.Int("eval-seq", cfg.seq_len));
  nanochat_loader* loader = nanochat_loader_create(parquet.data(), static_cast<int>(parquet.size()),
                                                   a.Str("text-column", "text").c_str(), tok, batch, seq, 0, 1,
                                                   static_cast<size_t>(a.Int("buffer-docs", 1000)));
  if (loader == nullptr) return Fail("eval: loader");
  const float bpb = nanochat_eval_bpb(m, loader, static_cast<int>(a.Int("steps", 10)));
  std::printf("val_bpb %.6f\n", bpb);
  nanochat_loader_free(loader);
  nanochat_tokenizer_free(tok);
  nanochat_model_free(m);
  return 0;
}

// score: per-position nll / argmax and the logits of focus ids over a NANOEVL1 fixture (input/tokens [B, T] int32,
// input/lengths [B], optional input/focus_positions / focus_offsets / focus_ids). The model is `--model CKPT`, or the
// one the fixture carries (config/* and param/* records), or a fresh one from the model flags. Results are printed
// per row, or written as a NANOEVL1 record file with `--out` (reference: src/score_command.cc).
const nanochat_record* FindRecord(const nanochat_record* recs, int64_t n, const std::string& name) {
  for (int64_t i = 0; i < n; ++i)
    if (name == recs[i].name) return &recs[i];
  return nullptr;
}

long long RecordInt(const nanochat_record* recs, int64_t n, const std::string& name, long long d) {
  const nanochat_record* r = FindRecord(recs, n, name);
  if (r == nullptr || r->bytes < 4) return d;
  return r->dtype == 3 ? static_cast<long long>(*static_cast<const int64_t*>(r->data))
                       : static_cast<long long>(*static_cast<const int32_t*>(r->data));
}
double RecordNum(const nanochat_record* recs, int64_t n, const std::string& name, double d) {
  const nanochat_record* r = FindRecord(recs, n, name);
  if (r == nullptr || r->bytes < 4) return d;
  if (r->dtype == 0) return *static_cast<const float*>(r->data);
  if (r->dtype == 2) return *static_cast<const double*>(r->data);
  return static_cast<double>(RecordInt(recs, n, name, 0));
}

// The model a fixture carries: config/* records give the shape, param/<name> records (fp32) the weights.
nanochat_model* ModelFromFixture(const nanochat_record* recs, int64_t n) {
  static std::string pattern;
  nanochat_config cfg{};
  cfg.num_layers = static_cast<int>(RecordInt(recs, n, "config/layers", 0));
  cfg.num_heads = static_cast<int>(RecordInt(recs, n, "config/heads", 0));
  cfg.num_kv_heads = static_cast<int>(RecordInt(recs, n, "config/kv_heads", cfg.num_heads));
  cfg.hidden_dim = static_cast<int>(RecordInt(recs, n, "config/embd", 0));
  cfg.seq_len = static_cast<int>(RecordInt(recs, n, "config/seq", 0));
  cfg.vocab_size = static_cast<int>(RecordInt(recs, n, "config/vocab", 0));
  cfg.padded_vocab_size = static_cast<int>(RecordInt(recs, n, "config/padded_vocab", cfg.vocab_size));
  cfg.rope_base = 100000.0f;
  pattern = "SSSL";
  if (const nanochat_record* wp = FindRecord(recs, n, "config/window_pattern"))
    if (wp->bytes > 0) pattern.assign(static_cast<const char*>(wp->data), static_cast<size_t>(wp->bytes));
  cfg.window_pattern = pattern.c_str();
  cfg.value_embedding = 1;
  ncb_set_short_window(0);
  nanochat_model* m = nanochat_model_create(&cfg, 0);
  if (m == nullptr) {
    Fail("fixture model");
    return nullptr;
  }
  const int count = nanochat_param_count(m);
  for (int i = 0; i < count; ++i) {
    nanochat_param info{};
    nanochat_param_info(m, i, &info);
    const nanochat_record* r = FindRecord(recs, n, std::string("param/") + info.name);
    if (r == nullptr || r->dtype != 0 || r->bytes != info.count * 4) {
      std::fprintf(stderr, "nanochat_cli: the fixture has no fp32 record param/%s of %lld values\n", info.name,
                   static_cast<long long>(info.count));
      nanochat_model_free(m);
      return nullptr;
    }
    nanochat_param_write(m, i, 0, 0, info.count, r->data);
  }
  return m;
}

int CmdScore(const Args& a) {
  if (!a.Has("fixture")) {
    std::fprintf(stderr, "nanochat_cli score: --fixture is required\n");
    return 2;
  }
  ncb_record_file* owner = nullptr;
  const nanochat_record* recs = nullptr;
  int64_t n = 0;
  char magic[9];
  if (ncb_record_file_read(a.Str("fixture").c_str(), &owner, magic, &recs, &n) != NANOCHAT_STATUS_OK) return Fail("score");
  nanochat_model* m = nullptr;
  if (!a.Has("model") && FindRecord(recs, n, "config/layers") != nullptr) {
    m = ModelFromFixture(recs, n);
    if (m == nullptr) return 1;
  } else {
    nanochat_config cfg;
    m = LoadModel(a, &cfg);
    if (m == nullptr) return Fail("score: model");
  }
  const nanochat_record* tok = FindRecord(recs, n, "input/tokens");
  const nanochat_record* len = FindRecord(recs, n, "input/lengths");
  if (tok == nullptr || len == nullptr || tok->ndim != 2 || tok->dtype != 1 || len->dtype != 1) {
    std::fprintf(stderr, "nanochat_cli score: input/tokens [B, T] and input/lengths [B] (int32) are required\n");
    return 1;
  }
  const int B = static_cast<int>(tok->dims[0]), T = static_cast<int>(tok->dims[1]);
  const int* lengths = static_cast<const int*>(len->data);
  std::vector<nanochat_focus> focus;
  const nanochat_record* fp = FindRecord(recs, n, "input/focus_positions");
  const nanochat_record* fo = FindRecord(recs, n, "input/focus_offsets");
  const nanochat_record* fi = FindRecord(recs, n, "input/focus_ids");
  if (fp != nullptr && fo != nullptr && fi != nullptr) {
    const int* pos = static_cast<const int*>(fp->data);
    const int* off = static_cast<const int*>(fo->data);
    const int* ids = static_cast<const int*>(fi->data);
    focus.resize(static_cast<size_t>(B));
    for (int b = 0; b < B; ++b) {
      focus[b].position = pos[b];
      focus[b].ids = ids + off[b];
      focus[b].count = pos[b] >= 0 ? off[b + 1] - off[b] : 0;
    }
  }
  std::vector<nanochat_score_result> res(static_cast<size_t>(B));
  nanochat_score_batch(m, static_cast<const int*>(tok->data), B, T, lengths, focus.empty() ? nullptr : focus.data(),
                       res.data());
  const char* e = nanochat_last_error();
  if (e != nullptr && *e) return Fail("score");
  std::vector<float> nll(static_cast<size_t>(B) * T), flog;
  std::vector<int32_t> amax(static_cast<size_t>(B) * T), offs(1, 0);
  for (int b = 0; b < B; ++b) {
    for (int t = 0; t < T; ++t) nll[static_cast<size_t>(b) * T + t] = res[b].nll[t], amax[static_cast<size_t>(b) * T + t] = res[b].argmax[t];
    const int fc = focus.empty() ? 0 : focus[b].count;
    for (int j = 0; j < fc; ++j) flog.push_back(res[b].focus_logits[j]);
    offs.push_back(static_cast<int32_t>(flog.size()));
  }
  if (a.Has("out")) {
    const int64_t d_bt[2] = {B, T}, d_off[1] = {B + 1}, d_f[1] = {static_cast<int64_t>(flog.size())};
    nanochat_record out[4] = {};
    out[0].name = "result/nll", out[0].dtype = 0, out[0].ndim = 2, out[0].dims = d_bt, out[0].data = nll.data(),
    out[0].bytes = static_cast<int64_t>(nll.size() * 4);
    out[1].name = "result/argmax", out[1].dtype = 1, out[1].ndim = 2, out[1].dims = d_bt, out[1].data = amax.data(),
    out[1].bytes = static_cast<int64_t>(amax.size() * 4);
    out[2].name = "result/focus_offsets", out[2].dtype = 1, out[2].ndim = 1, out[2].dims = d_off, out[2].data = offs.data(),
    out[2].bytes = static_cast<int64_t>(offs.size() * 4);
    out[3].name = "result/focus_logits", out[3].dtype = 0, out[3].ndim = 1, out[3].dims = d_f, out[3].data = flog.data(),
    out[3].bytes = static_cast<int64_t>(flog.size() * 4);
    if (ncb_record_file_write(a.Str("out").c_str(), "NANOEVL1", out, 4) != NANOCHAT_STATUS_OK) return Fail("score: out");
  } else {
    for (int b = 0; b < B; ++b) {
      const int cnt = lengths[b] - 1;
      double mean = 0.0;
      for (int t = 0; t < cnt; ++t) mean += res[b].nll[t];
      std::printf("row %d: mean nll %.6f focus [", b, cnt > 0 ? mean / cnt : 0.0);
      for (int j = offs[b]; j < offs[b + 1]; ++j) std::printf("%s%.6f", j > offs[b] ? ", " : "", flog[j]);
      std::printf("]\n");
    }
  }
  nanochat_model_free(m);
  ncb_record_file_free(owner);
  return 0;
}

// rl_step: replay the policy-gradient steps of a NANOORC1 fixture (model and optimizer settings carried by the
// fixture; rollout/<k>/tokens, targets [B, T] int32 and advantages [B] fp32 per step) and print, or write with --out,
// each step's loss and gradient norm and the final parameters (reference: src/rl_step_command.cc).
int CmdRlStep(const Args& a) {
  if (!a.Has("fixture")) {
    std::fprintf(stderr, "nanochat_cli rl_step: --fixture is required\n");
    return 2;
  }
  ncb_record_file* owner = nullptr;
  const nanochat_record* recs = nullptr;
  int64_t n = 0;
  char magic[9];
  if (ncb_record_file_read(a.Str("fixture").c_str(), &owner, magic, &recs, &n) != NANOCHAT_STATUS_OK) return Fail("rl_step");
  nanochat_model* m = ModelFromFixture(recs, n);
  if (m == nullptr) return 1;
  nanochat_optim_config oc{};
  auto o = [&](const char* k, double d) { return static_cast<float>(RecordNum(recs, n, std::string("config/opt/") + k, d)); };
  auto sc = [&](const char* k, double d) { return static_cast<float>(RecordNum(recs, n, std::string("config/sched/") + k, d)); };
  oc.unembedding_lr = o("unembedding_lr", .004), oc.embedding_lr = o("embedding_lr", .2), oc.matrix_lr = o("matrix_lr", .02);
  oc.scalar_lr = o("scalar_lr", .5), oc.weight_decay = o("weight_decay", 0.0), oc.clip = o("clip", 0.0);
  oc.adam_eps = o("adam_eps", 1e-10), oc.muon_ns_steps = static_cast<int>(o("muon_ns_steps", 5)), oc.muon_beta2 = o("muon_beta2", .9);
  oc.num_iterations = static_cast<int>(sc("num_iterations", 0)), oc.warmup_steps = static_cast<int>(sc("warmup_steps", 0));
  oc.warmdown_ratio = sc("warmdown_ratio", 0.0), oc.final_lr_frac = sc("final_lr_frac", 0.0);
  oc.weight_decay_base = sc("weight_decay_base", 0.0), oc.muon_momentum_warmup_steps = sc("muon_momentum_warmup_steps", 0.0);
  oc.muon_momentum_start = sc("muon_momentum_start", .95), oc.muon_momentum_peak = sc("muon_momentum_peak", .95);
  oc.muon_momentum_final = sc("muon_momentum_final", .95);
  nanochat_optim* opt = nanochat_optim_create(m, &oc);
  if (opt == nullptr) return Fail("rl_step: optimizer");
  const int steps = static_cast<int>(a.Int("steps", RecordInt(recs, n, "config/steps", 0)));
  const int passes = static_cast<int>(RecordInt(recs, n, "config/num_passes", 1));
  const int per = static_cast<int>(RecordInt(recs, n, "config/examples_per_rank", 1));
  std::vector<float> losses, norms;
  for (int k = 0; k < steps; ++k) {
    const std::string base = "rollout/" + std::to_string(k) + "/";
    const nanochat_record* tok = FindRecord(recs, n, base + "tokens");
    const nanochat_record* tgt = FindRecord(recs, n, base + "targets");
    const nanochat_record* adv = FindRecord(recs, n, base + "advantages");
    if (tok == nullptr || tgt == nullptr || adv == nullptr || tok->ndim != 2) {
      std::fprintf(stderr, "nanochat_cli rl_step: step %d is missing from the fixture\n", k);
      return 1;
    }
    const float loss = nanochat_rl_step(m, opt, static_cast<const int*>(tok->data), static_cast<const int*>(tgt->data),
                                        static_cast<const float*>(adv->data), static_cast<int>(tok->dims[0]),
                                        static_cast<int>(tok->dims[1]), passes, per, k + 1);
    const char* e = nanochat_last_error();
    if (e != nullptr && *e) return Fail("rl_step");
    losses.push_back(loss);
    norms.push_back(nanochat_optim_grad_norm(opt));
    std::fprintf(stderr, "rl: step %d loss %.6f grad_norm %.6f\n", k + 1, loss, norms.back());
  }
  if (a.Has("out")) {
    const int count = nanochat_param_count(m);
    std::vector<std::string> names;
    std::vector<std::vector<float>> values(static_cast<size_t>(count));
    std::vector<std::vector<int64_t>> dims;
    std::vector<nanochat_record> out;
    names.reserve(static_cast<size_t>(2 * steps + count));
    dims.reserve(static_cast<size_t>(2 * steps + count));
    auto push = [&](std::string name, const float* data, std::vector<int64_t> d, int64_t cnt) {
      names.push_back(std::move(name));
      dims.push_back(std::move(d));
      nanochat_record r{};
      r.name = names.back().c_str(), r.dtype = 0, r.ndim = static_cast<int32_t>(dims.back().size());
      r.dims = dims.back().data(), r.data = data, r.bytes = cnt * 4;
      out.push_back(r);
    };
    for (int k = 0; k < steps; ++k) {
      push("step/" + std::to_string(k) + "/loss", &losses[k], {1}, 1);
      push("step/" + std::to_string(k) + "/grad_norm", &norms[k], {1}, 1);
    }
    for (int i = 0; i < count; ++i) {
      nanochat_param info{};
      nanochat_param_info(m, i, &info);
      values[i].resize(static_cast<size_t>(info.count));
      nanochat_param_read(m, i, 0, 0, info.count, values[i].data());
      std::vector<int64_t> d = info.cols > 0 ? std::vector<int64_t>{info.rows, info.cols} : std::vector<int64_t>{info.count};
      push(std::string("param/") + info.name, values[i].data(), d, info.count);
    }
    if (ncb_record_file_write(a.Str("out").c_str(), "NANOORC1", out.data(), static_cast<int64_t>(out.size())) !=
        NANOCHAT_STATUS_OK)
      return Fail("rl_step: out");
  }
  nanochat_optim_free(opt);
  nanochat_model_free(m);
  ncb_record_file_free(owner);
  return 0;
}

// eval_bench: time the evaluation forward (loss over one batch) of the CPU engine and print a `nanochat.bench.v3`
// document (reference: src/eval_bench_command.cc). Tokens are xorshift-random in [0, vocab).
// rl_worker: the persistent policy worker of the RL loop (reference src/rl_worker_command.cc:197-205, protocol
// src/rl_worker.h). With `--fixture` it replays a recorded run like `rl_step`. Otherwise it loads `--checkpoint`
// (or builds a model from the model flags), then answers one request per line on stdin with one reply line on stdout:
//   ping                                                         -> pong ok=1
//   rollout prompts=<ids,> num_prompts= prompt_len= [num_samples= max_tokens= temperature= top_k= seed= stop_id=
//           stop_ids=<ids,> bos_id=]                              -> rollout ok=1 ... rows= lengths= masks= tokens=
//   advantage tokens=<ids,> targets=<ids,> advantages=<floats,> batch= seq= num_passes= examples_per_rank=
//                                                                -> advantage ok=1 step= loss= grad_norm= valid_targets=
//   save path=<file>                                             -> save ok=1
//   quit                                                         -> quit ok=1   (and the worker exits)
// A request that fails is answered `<kind> ok=0 error=<words_joined_by_underscores>` and the worker stays alive.
// The same lines are spoken by the Python worker, so the Python RL loop can drive either.
namespace rlw {
std::map<std::string, std::string> Fields(const std::vector<std::string>& words) {
  std::map<std::string, std::string> f;
  for (std::size_t i = 1; i < words.size(); ++i) {
    const std::size_t eq = words[i].find('=');
    if (eq != std::string::npos) f[words[i].substr(0, eq)] = words[i].substr(eq + 1);
  }
  return f;
}
template <typename T, typename Conv>
std::vector<T> List(const std::string& text, Conv conv) {
  std::vector<T> out;
  std::size_t a = 0;
  while (a < text.size()) {
    std::size_t b = text.find(',', a);
    if (b == std::string::npos) b = text.size();
    if (b > a) out.push_back(conv(text.substr(a, b - a)));
    a = b + 1;
  }
  return out;
}
std::vector<int> Ints(const std::string& t) { return List<int>(t, [](const std::string& w) { return std::atoi(w.c_str()); }); }
std::vector<float> Floats(const std::string& t) {
  return List<float>(t, [](const std::string& w) { return static_cast<float>(std::atof(w.c_str())); });
}
std::string Need(const std::map<std::string, std::string>& f, const char* key) {
  const auto it = f.find(key);
  if (it == f.end()) throw std::runtime_error(std::string("missing ") + key + "=");
  return it->second;
}
std::string Get(const std::map<std::string, std::string>& f, const char* key, const char* fallback) {
  const auto it = f.find(key);
  return it == f.end() ? fallback : it->second;
}
}  // namespace rlw

int CmdRlStep(const Args& a);

int CmdRlWorker(const Args& a) {
  if (a.Has("fixture")) return CmdRlStep(a);
  nanochat_config cfg;
  nanochat_model* m = nullptr;
  {
    Args with_model = a;
    if (a.Has("checkpoint")) {
      cfg = ModelFromArgs(a);
      const bool shape_given = a.Has("preset-model") || a.Has("layers") || a.Has("hidden") || a.Has("heads");
      if (!shape_given) ConfigFromCheckpoint(a.Str("checkpoint"), &cfg);
      m = nanochat_model_create(&cfg, static_cast<uint64_t>(a.Int("seed", 0)));
      if (m != nullptr) nanochat_load(m, a.Str("checkpoint").c_str());
    } else {
      m = LoadModel(a, &cfg);
    }
  }
  if (m == nullptr) return Fail("rl_worker: model");
  nanochat_optim_config oc;
  if (!OptimFromArgs(a, &oc, "default")) return Fail("rl_worker");
  nanochat_optim* opt = nanochat_optim_create(m, &oc);
  if (opt == nullptr) return Fail("rl_worker: optimizer");
  int step = 0;
  std::string line;
  char buf[1 << 16];
  while (std::fgets(buf, sizeof(buf), stdin) != nullptr) {
    line = buf;
    while (!line.empty() && line.back() != '\n' && std::fgets(buf, sizeof(buf), stdin) != nullptr) line += buf;   // long lines
    while (!line.empty() && (line.back() == '\n' || line.back() == '\r')) line.pop_back();
    if (line.empty()) continue;
    std::vector<std::string> words;
    for (std::size_t i = 0; i < line.size();) {
      std::size_t j = line.find(' ', i);
      if (j == std::string::npos) j = line.size();
      if (j > i) words.push_back(line.substr(i, j - i));
      i = j + 1;
    }
    const std::string kind = words.empty() ? "unknown" : words[0];
    std::string reply;
    try {
      const auto f = rlw::Fields(words);
      if (kind == "ping") {
        reply = "pong ok=1";
      } else if (kind == "quit") {
        reply = "quit ok=1";
      } else if (kind == "save") {
        nanochat_save(m, rlw::Need(f, "path").c_str());
        reply = "save ok=1";
      } else if (kind == "advantage") {
        const int batch = std::atoi(rlw::Need(f, "batch").c_str()), seq = std::atoi(rlw::Need(f, "seq").c_str());
        const std::vector<int> tokens = rlw::Ints(rlw::Get(f, "tokens", "")), targets = rlw::Ints(rlw::Get(f, "targets", ""));
        const std::vector<float> adv = rlw::Floats(rlw::Get(f, "advantages", ""));
        const std::size_t n = static_cast<std::size_t>(std::max(batch, 0)) * static_cast<std::size_t>(std::max(seq, 0));
        if (batch <= 0 || seq <= 0) throw std::runtime_error("batch and seq must be positive");
        if (tokens.size() != n || targets.size() != n || adv.size() != n)
          throw std::runtime_error("every list must hold batch*seq = " + std::to_string(n) + " entries");
        int valid = 0;
        for (int t : targets) valid += t != -1 ? 1 : 0;
        const float loss = nanochat_rl_step(m, opt, tokens.data(), targets.data(), adv.data(), batch, seq,
                                            std::atoi(rlw::Need(f, "num_passes").c_str()),
                                            std::atoi(rlw::Need(f, "examples_per_rank").c_str()), step + 1);
        if (!(loss == loss)) throw std::runtime_error(nanochat_last_error());
        if (valid > 0) ++step;
        char out[256];
        std::snprintf(out, sizeof(out), "advantage ok=1 step=%d loss=%.9g grad_norm=%.9g valid_targets=%d", step,
                      static_cast<double>(loss), valid > 0 ? static_cast<double>(nanochat_optim_grad_norm(opt)) : 0.0, valid);
        reply = out;
      } else if (kind == "rollout") {
        nanochat_generate_multi_params gp{};
        gp.num_prompts = std::atoi(rlw::Need(f, "num_prompts").c_str());
        gp.prompt_len = std::atoi(rlw::Need(f, "prompt_len").c_str());
        const std::vector<int> prompts = rlw::Ints(rlw::Get(f, "prompts", ""));
        if (gp.num_prompts <= 0 || gp.prompt_len <= 0 ||
            prompts.size() != static_cast<std::size_t>(gp.num_prompts) * static_cast<std::size_t>(gp.prompt_len))
          throw std::runtime_error("prompts must hold num_prompts * prompt_len ids");
        gp.params.num_samples = std::atoi(rlw::Get(f, "num_samples", "1").c_str());
        gp.params.max_tokens = std::atoi(rlw::Need(f, "max_tokens").c_str());
        gp.params.temperature = static_cast<float>(std::atof(rlw::Get(f, "temperature", "1.0").c_str()));
        gp.params.top_k = std::atoi(rlw::Get(f, "top_k", "0").c_str());
        gp.params.seed = std::strtoull(rlw::Get(f, "seed", "0").c_str(), nullptr, 10);
        gp.params.stop_id = std::atoi(rlw::Get(f, "stop_id", "-1").c_str());
        gp.params.bos_id = std::atoi(rlw::Get(f, "bos_id", "-1").c_str());
        nanochat_sequences seqs{};
        nanochat_generate_multi(m, prompts.data(), &gp, &seqs);
        std::string lengths, masks, toks;
        for (int r = 0; r < seqs.count; ++r) {
          lengths += (r ? "," : "") + std::to_string(seqs.lengths[r]);
          for (int k = 0; k < seqs.lengths[r]; ++k) {
            const int at = seqs.offsets[r] + k;
            masks += (masks.empty() ? "" : ",") + std::to_string(static_cast<int>(seqs.mask[at]));
            toks += (toks.empty() ? "" : ",") + std::to_string(seqs.tokens[at]);
          }
        }
        reply = "rollout ok=1 num_prompts=" + std::to_string(gp.num_prompts) + " num_samples=" +
                std::to_string(gp.params.num_samples) + " rows=" + std::to_string(seqs.count) + " lengths=" + lengths +
                " masks=" + masks + " tokens=" + toks;
      } else {
        throw std::runtime_error("unknown message type " + kind);
      }
    } catch (const std::exception& e) {
      std::string msg = e.what();
      for (char& c : msg)
        if (c == ' ' || c == '\n' || c == '\t') c = '_';
      reply = kind + " ok=0 error=" + (msg.empty() ? "error" : msg);
    }
    std::printf("%s\n", reply.c_str());
    std::fflush(stdout);
    if (reply.rfind("quit ok=1", 0) == 0) break;
  }
  if (a.Has("save")) nanochat_save(m, a.Str("save").c_str());
  nanochat_optim_free(opt);
  nanochat_model_free(m);
  return 0;
}

int CmdEvalBench(const Args& a) {
  nanochat_config cfg;
  nanochat_model* m = LoadModel(a, &cfg);
  if (m == nullptr) return Fail("eval_bench");
  const int batch = static_cast<int>(a.Int("batch", 8)), seq = static_cast<int>(a.Int("eval-seq", cfg.seq_len));
  const int iters = static_cast<int>(a.Int("iters", 10)), warmup = static_cast<int>(a.Int("warmup", 3));
  std::vector<int> tok(static_cast<size_t>(batch) * seq), tgt(tok.size());
  unsigned long long x = 0x9E3779B97F4A7C15ull ^ static_cast<unsigned long long>(a.Int("seed", 0));
  for (size_t i = 0; i < tok.size(); ++i) {
    x ^= x << 13, x ^= x >> 7, x ^= x << 17;
    tok[i] = static_cast<int>(x % static_cast<unsigned long long>(cfg.vocab_size));
  }
  for (size_t i = 0; i < tok.size(); ++i) tgt[i] = (i + 1) % seq == 0 ? -1 : tok[i + 1];
  float loss = 0.0f;
  for (int i = 0; i < warmup; ++i) loss = nanochat_forward_loss(m, tok.data(), tgt.data(), batch, seq);
  std::vector<double> ms;
  for (int i = 0; i < iters; ++i) {
    timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    loss = nanochat_forward_loss(m, tok.data(), tgt.data(), batch, seq);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    ms.push_back((t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6);
  }
  const char* e = nanochat_last_error();
  if (e != nullptr && *e) return Fail("eval_bench");
  std::sort(ms.begin(), ms.end());
  const double med = ms.empty() ? 0.0 : ms[ms.size() / 2];
  nanochat_params counts{};
  nanochat_params_get(&cfg, &counts);
  const double flops = counts.flops_per_token / 3.0 * batch * seq;   // forward = a third of forward + backward
  std::printf("{\"schema\":\"nanochat.bench.v3\",\"device\":\"cpu\",\"precision\":\"fp32\",\"rows\":[{\"name\":"
              "\"eval_forward\",\"family\":\"eval_forward\",\"phase\":\"fwd\",\"precision\":\"fp32\",\"shape\":\"B=%d T=%d "
              "L=%d C=%d V=%d\",\"ms\":%.6f,\"gflops\":%.3f,\"work_ratio\":0,\"mfu\":0,\"iterations\":%d}],\"loss\":%.6f,"
              "\"tokens_per_second\":%.1f}\n",
              batch, seq, cfg.num_layers, cfg.hidden_dim, cfg.vocab_size, med, med > 0 ? flops / med / 1e6 : 0.0, iters, loss,
              med > 0 ? batch * seq / med * 1e3 : 0.0);
  nanochat_model_free(m);
  return 0;
}

int CmdTokTrain(const Args& a) {
  nanochat_tokenizer* tok = ncb_tokenizer_train(a.Has("text") ? a.Str("text").c_str() : nullptr,
                                                a.Has("parquet") ? a.Str("parquet").c_str() : nullptr,
                                                a.Str("text-column", "text").c_str(),
                                                static_cast<int>(a.Int("vocab", 32768)), a.Int("doc-cap", 10000),
                                                a.Int("max-chars", 10000000000ll));
  if (tok == nullptr) return Fail("tok_train");
  const nanochat_status st = ncb_tokenizer_save(tok, a.Str("out", "tokenizer.nctoken").c_str());
  std::printf("vocab %d -> %s\n", ncb_tokenizer_vocab_size(tok), a.Str("out", "tokenizer.nctoken").c_str());
  nanochat_tokenizer_free(tok);
  return st == NANOCHAT_STATUS_OK ? 0 : Fail("tok_train: save");
}

int CmdParams(const Args& a) {
  nanochat_config cfg = ModelFromArgs(a);
  nanochat_params p{};
  if (nanochat_params_get(&cfg, &p) != NANOCHAT_STATUS_OK) return Fail("params");
  std::printf("{\"total\": %lld, \"transformer_matrices\": %lld, \"lm_head\": %lld, \"embeddings\": %lld, "
              "\"scalars\": %lld, \"flops_per_token\": %.0f}\n",
              static_cast<long long>(p.total), static_cast<long long>(p.transformer_matrices),
              static_cast<long long>(p.lm_head), static_cast<long long>(p.embeddings),
              static_cast<long long>(p.scalars), p.flops_per_token);
  return 0;
}

int CmdRoofline(const Args& a) {
  nanochat_config cfg = ModelFromArgs(a);
  std::vector<char> text(1 << 16);
  const int64_t n = ncb_roofline(&cfg, a.Str("device", "b200").c_str(), a.Str("precision", "bf16").c_str(),
                                 static_cast<int>(a.Int("batch", 32)), static_cast<int>(a.Int("grad-accum", 1)),
                                 static_cast<int>(a.Int("devices", 1)), a.Int("tokens", 0), a.Num("link-gbps", 0.0),
                                 a.Num("latency-us", 5.0), a.Num("overlap", 0.0),
                                 static_cast<int>(a.Int("muon-ns-steps", 5)), a.Num("bf16-tflops", 0.0),
                                 a.Num("hbm-gbs", 0.0), a.Has("json") ? 0 : 1, text.data(),
                                 static_cast<int64_t>(text.size()));
  if (n < 0) return Fail("roofline");
  std::printf("%s%s", text.data(), a.Has("json") ? "\n" : "");
  return 0;
}

// `plan --spec <spec.json> --caps <device.json> [--precision bf16] [--graph train]`: the operator plan as JSON.
int CmdPlan(const Args& a) {
  std::vector<char> text(1 << 16);
  const int64_t n = ncb_plan_json(a.Str("spec", "").c_str(), a.Str("caps", "").c_str(), a.Str("precision", "bf16").c_str(),
                                  a.Str("graph", "train").c_str(), text.data(), static_cast<int64_t>(text.size()));
  if (n < 0) return Fail("plan");
  std::printf("%s\n", text.data());
  return 0;
}

// `train_plan --depth D --vocab V --device-batch B [--seq T] [--total-batch N] [--num-iterations K] ...`
int CmdTrainPlan(const Args& a) {
  std::vector<char> text(1 << 14);
  const int64_t n = ncb_train_plan_json(
      static_cast<int>(a.Int("depth", 12)), static_cast<int>(a.Int("aspect-ratio", 64)),
      static_cast<int>(a.Int("head-dim", 128)), static_cast<int>(a.Int("seq", 2048)),
      static_cast<int>(a.Int("vocab", 32768)), static_cast<int>(a.Int("device-batch", 32)),
      a.Str("window-pattern", "SSSL").c_str(), a.Int("total-batch", -1), a.Int("num-iterations", 0),
      a.Num("target-flops", 0.0), static_cast<int>(a.Int("param-data-ratio", 12)), text.data(),
      static_cast<int64_t>(text.size()));
  if (n < 0) return Fail("train_plan");
  std::printf("%s\n", text.data());
  return 0;
}

// `dist --world-size N [--port P] -- <command> [flags]`: one child process per rank with NANOCHAT_RANK,
// NANOCHAT_WORLD_SIZE, NANOCHAT_MASTER_ADDR and NANOCHAT_MASTER_PORT set (the reference launcher's contract,
// python/nanochat_cpp/cli.py:827-945), rank 0 first. If a rank fails the others are terminated.
int CmdDist(int argc, char** argv) {
  int split = -1;
  for (int i = 2; i < argc; ++i)
    if (std::strcmp(argv[i], "--") == 0) {
      split = i;
      break;
    }
  if (split < 0 || split + 1 >= argc) {
    std::fprintf(stderr, "nanochat_cli dist: usage: dist --world-size N [--port P] -- <command> [flags]\n");
    return 2;
  }
  const Args a = Parse(split, argv, 2);
  const int world = static_cast<int>(a.Int("world-size", 2));
  const std::string port = a.Str("port", "29500");
  std::vector<pid_t> kids;
  for (int r = 0; r < world; ++r) {
    const pid_t pid = ::fork();
    if (pid == 0) {
      ::setenv("NANOCHAT_RANK", std::to_string(r).c_str(), 1);
      ::setenv("NANOCHAT_WORLD_SIZE", std::to_string(world).c_str(), 1);
      ::setenv("NANOCHAT_MASTER_ADDR", "127.0.0.1", 1);
      ::setenv("NANOCHAT_MASTER_PORT", port.c_str(), 1);
      std::vector<char*> child = {argv[0]};
      for (int i = split + 1; i < argc; ++i) child.push_back(argv[i]);
      child.push_back(nullptr);
      ::execv("/proc/self/exe", child.data());
      std::perror("nanochat_cli dist: exec");
      ::_exit(127);
    }
    if (pid < 0) return Fail("dist: fork");
    kids.push_back(pid);
    if (r == 0) ::usleep(200000);  // rank 0 opens the rendezvous port first
  }
  int worst = 0;
  for (std::size_t left = kids.size(); left > 0; --left) {
    int status = 0;
    const pid_t done = ::wait(&status);
    if (done < 0) break;
    const int rc = WIFEXITED(status) ? WEXITSTATUS(status) : 128 + WTERMSIG(status);
    if (rc != 0 && worst == 0) {
      worst = rc;
      for (pid_t k : kids)
        if (k != done) ::kill(k, SIGTERM);  // exact PIDs of the children this launcher started
    }
  }
  return worst;
}

void Usage() {
  std::printf(
      "nanochat_cli <command> [--flag value ...] [--device cpu|cuda|cuda:N]\n"
      "  (native engines: C++ on the CPU, or the sm_100a kernels driven from C++ on a CUDA device; no Python in either)\n"
      "  train --device cuda:N also takes --synthetic-zipf S (synthetic token ids instead of parquet + tokenizer)\n"
      "  train      --train-parquet P.. --tokenizer T | --rows shard.nchsft   [--mesh N (replicas in this process) | --rank R\n"
      "             --world-size W --port P (one process per rank; or `dist`)] [--batch B --grad-accum A\n"
      "             --num-iterations K --log-every L --save-every S --out-dir D --checkpoint C --resume --warm-start W\n"
      "             --preset track3 + optimizer / schedule / model flags]\n"
      "  sft        --rows shard.nchsft --warm-start base.ckpt [train flags]   fine-tuning over packed rows\n"
      "  generate   --model C [--tokenizer T --prompt TEXT | --tokens a,b,c] --max-tokens N --num-samples S\n"
      "             --temperature X --top-k K --seed Z --stop-id I\n"
      "  eval       --model C --val-parquet P.. --tokenizer T --steps N --batch B\n"
      "  score      --fixture F.bin [--model C] [--out results.bin]   nll / argmax / focus logits over a NANOEVL1 fixture\n"
      "  rl_step    --fixture F.bin [--steps N] [--out results.bin]  replay the policy-gradient steps of a NANOORC1 fixture\n"
      "  eval_bench model flags --batch B --iters N --warmup W     evaluation forward time as a nanochat.bench.v3 document\n"
      "  tok_train  --text F | --parquet P  --vocab V --out tokenizer.nctoken\n"
      "  dist       --world-size N [--port P] -- train ...      one process per rank over the TCP ring\n"
      "  params     model flags -> parameter counts and FLOPs per token (JSON)\n"
      "  plan       --spec model.json --caps device.json [--precision bf16] [--graph train|prefill|decode|generate|eval]\n"
      "  train_plan --depth D --vocab V --device-batch B [--seq T --total-batch N --num-iterations K --target-flops F]\n"
      "  roofline   --device b200|h100|t4|cpu --precision bf16|fp8|fp32 --batch B --grad-accum A --devices N --tokens T\n"
      "             --link-gbps G --latency-us U --overlap F --muon-ns-steps K [--bf16-tflops X --hbm-gbs Y] [--json]\n"
      "model flags: --preset-model tiny|d12|d20|d26 | --depth N | --layers --heads --kv-heads --hidden --seq --vocab\n"
      "             --padded-vocab --rope-base --window-pattern --short-window --no-value-embedding\n");
}

}  // namespace

int main(int argc, char** argv) {
  const char* sandbox = std::getenv("NANOCHAT_SANDBOX");
  const char* enforce = std::getenv("NANOCHAT_SANDBOX_ENFORCE");
  if (enforce != nullptr && std::strcmp(enforce, "1") == 0 && (sandbox == nullptr || !*sandbox)) {
    std::fprintf(stderr, "nanochat_cli: NANOCHAT_SANDBOX is not set and NANOCHAT_SANDBOX_ENFORCE=1; refusing to start\n");
    return 3;
  }
  if (argc < 2 || std::strcmp(argv[1], "help") == 0 || std::strcmp(argv[1], "--help") == 0) {
    Usage();
    return argc < 2 ? 2 : 0;
  }
  const std::string cmd = argv[1];
  if (cmd == "--version" || cmd == "version") {
    std::printf("nanochat_cli %s (backend %s, sandbox %s)\n", nanochat_version(), nanochat_backend(),
                sandbox != nullptr && *sandbox ? sandbox : "none");
    return 0;
  }
  if (cmd == "dist") return CmdDist(argc, argv);
  if (nanochat_init() != NANOCHAT_STATUS_OK) return Fail("init");
  const Args a = Parse(argc, argv, 2);
  // `--device cpu|cuda|cuda:N` on any command: models live in that engine (NANOCHAT_DEVICE is the default)
  // (`roofline --device` names a device *profile* instead and is left alone)
  const bool runs_a_model = cmd == "train" || cmd == "sft" || cmd == "generate" || cmd == "eval" || cmd == "score" ||
                            cmd == "rl_step" || cmd == "rl_worker" || cmd == "eval_bench";
  if (runs_a_model && a.Has("device") && nanochat_select_device(a.Str("device").c_str()) != NANOCHAT_STATUS_OK)
    return Fail("--device");
  if (cmd == "train" && std::strcmp(nanochat_backend(), "cuda") == 0) return CmdTrainDevice(a);
  if (cmd == "train") return CmdTrain(a);
  if (cmd == "sft") {   // supervised fine-tuning = the training driver over a packed NCSFT001 shard, from a base model
    if (!a.Has("rows") || !(a.Has("warm-start") || a.Has("resume"))) {
      std::fprintf(stderr, "nanochat_cli sft: --rows shard.nchsft and --warm-start base.ckpt (or --resume) are required\n");
      return 2;
    }
    return CmdTrain(a, "sft");   // the fine-tuning optimizer and schedule unless --preset says otherwise
  }
  if (cmd == "generate") return CmdGenerate(a);
  if (cmd == "eval") return CmdEval(a);
  if (cmd == "score") return CmdScore(a);
  if (cmd == "rl_step") return CmdRlStep(a);
  if (cmd == "rl_worker") return CmdRlWorker(a);
  if (cmd == "eval_bench") return CmdEvalBench(a);
  if (cmd == "tok_train") return CmdTokTrain(a);
  if (cmd == "params") return CmdParams(a);
  if (cmd == "roofline") return CmdRoofline(a);
  if (cmd == "plan") return CmdPlan(a);
  if (cmd == "train_plan") return CmdTrainPlan(a);
  std::fprintf(stderr, "nanochat_cli: unknown command '%s'\n", cmd.c_str());
  Usage();
  return 2;
}
