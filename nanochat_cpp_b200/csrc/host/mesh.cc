#include "mesh.h"

#include "perf.h"

#include <glob.h>
#include <sys/stat.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <csignal>
#include <cstdio>
#include <cstring>
#include <thread>

namespace ncb {

// ------------------------------------------------------------------------------------------------ runtime
MeshRuntime::MeshRuntime(const MeshSpec& mesh, const EngineConfig& cfg, const OptimConfig& optim, int batch,
                         int grad_accum, int seq, std::uint64_t seed, std::string* error)
    : batch_(batch), accum_(std::max(1, grad_accum)), seq_(seq > 0 ? seq : cfg.seq_len) {
  const int world = std::max(1, mesh.size());
  if (batch <= 0 || batch % (world * accum_) != 0) {
    if (error) *error = "the global batch must be a positive multiple of world * grad_accum";
    return;
  }
  if (seq_ > cfg.seq_len) {
    if (error) *error = "seq exceeds the model's seq_len";
    return;
  }
  hub_ = std::make_unique<MemoryHub>(world);
  replicas_.resize(world);
  for (int r = 0; r < world; ++r) {
    replicas_[r].model = std::make_unique<CpuModel>(cfg);
    replicas_[r].model->InitWeights(seed);  // the same seed: replicas start identical
    replicas_[r].optim = std::make_unique<CpuOptimizer>(replicas_[r].model.get(), optim);
    replicas_[r].link = hub_->Endpoint(r);
  }
  metrics_.loss.assign(world, 0.0f);
  ok_ = true;
}

MeshRuntime::~MeshRuntime() = default;

void MeshRuntime::InjectDrop(int from) {
  const int n = world();
  if (n > 1 && from >= 0 && from < n) hub_->DropNext(from, (from + 1) % n, 1);
}

float MeshRuntime::TrainStep(const int* tokens, const int* targets, std::string* error) {
  if (!ok_) return 0.0f;
  const auto t0 = std::chrono::steady_clock::now();
  const int world = this->world();
  const int per_replica = batch_ / world, micro = per_replica / accum_;
  const float scale = 1.0f / static_cast<float>(accum_ * world);
  const int step = step_ + 1;
  std::vector<std::string> errors(world);
  std::vector<char> failed(world, 0);
  auto work = [&](int r) {
    Replica& rep = replicas_[r];
    rep.model->ZeroGrad();
    double loss = 0.0;
    for (int m = 0; m < accum_; ++m) {
      const std::size_t row0 = static_cast<std::size_t>(r) * per_replica + static_cast<std::size_t>(m) * micro;
      loss += rep.model->ForwardLoss(tokens + row0 * seq_, targets + row0 * seq_, micro, seq_);
      rep.model->Backward(scale);
    }
    metrics_.loss[r] = static_cast<float>(loss / accum_);
    if (world > 1) {
      std::vector<float>& g = rep.model->grads();
      if (!RingAllReduceSum(rep.link.get(), g.data(), g.size(), timeout_ms_)) {
        failed[r] = 1;
        errors[r] = "replica " + std::to_string(r) + ": " + rep.link->error();
        return;  // no optimizer step on a failed reduce: the weights stay at the previous step
      }
    }
    rep.optim->Step(step);
  };
  if (world == 1) {
    work(0);
  } else {
    std::vector<std::thread> threads;
    for (int r = 0; r < world; ++r) threads.emplace_back(work, r);
    for (auto& t : threads) t.join();
  }
  for (int r = 0; r < world; ++r)
    if (failed[r]) {
      if (error) *error = "gradient reduce failed (" + errors[r] + ")";
      ok_ = false;  // replicas may have diverged: the runtime must be reloaded from a checkpoint
      return 0.0f;
    }
  step_ = step;
  metrics_.grad_norm = replicas_[0].optim->grad_norm();
  double mean = 0.0;
  for (float l : metrics_.loss) mean += l;
  metrics_.step_seconds = std::chrono::duration<float>(std::chrono::steady_clock::now() - t0).count();
  return static_cast<float>(mean / world);
}

std::uint64_t MeshRuntime::ParamDigest(int replica) const {
  std::uint64_t h = 0xCBF29CE484222325ull;
  if (replica < 0 || replica >= static_cast<int>(replicas_.size())) return 0;
  CpuModel* m = replicas_[replica].model.get();
  for (const CpuParam& p : m->params()) {
    const auto* bytes = reinterpret_cast<const std::uint8_t*>(m->value(p));
    for (std::size_t i = 0; i < p.count * 4; ++i) h = (h ^ bytes[i]) * 0x100000001B3ull;
  }
  return h;
}

bool MeshRuntime::Save(const std::string& path, std::string* error) const {
  if (replicas_.empty()) return false;
  return replicas_[0].model->SaveWithOptimizer(path, *replicas_[0].optim, static_cast<std::uint64_t>(step_),
                                               static_cast<std::uint32_t>(replicas_.size()), error);
}

bool MeshRuntime::Load(const std::string& path, std::string* error) {
  std::uint64_t step = 0;
  for (auto& rep : replicas_)
    if (!rep.model->LoadWithOptimizer(path, rep.optim.get(), &step, error)) return false;
  step_ = static_cast<int>(step);
  ok_ = true;
  return true;
}

bool MeshRuntime::LoadWeights(const std::string& path, std::string* error) {
  for (auto& rep : replicas_)
    if (!rep.model->Load(path, error)) return false;
  return true;
}

// ------------------------------------------------------------------------------------------------ driver
double EstimateFlopsPerToken(const EngineConfig& cfg) { return FlopsPerToken(cfg); }

namespace {

std::atomic<int> g_interrupted{0};
extern "C" void OnSigint(int) { g_interrupted = 1; }

std::vector<std::string> ExpandGlobs(const std::vector<std::string>& patterns) {
  std::vector<std::string> out;
  for (const std::string& pat : patterns) {
    glob_t g{};
    if (::glob(pat.c_str(), 0, nullptr, &g) == 0)
      for (std::size_t i = 0; i < g.gl_pathc; ++i) out.emplace_back(g.gl_pathv[i]);
    ::globfree(&g);
  }
  std::sort(out.begin(), out.end());
  return out;
}

// Batches of the run: either the document loader over parquet text, or rows of a packed shard in file order.
class BatchSource {
 public:
  // `rows`: sequences this process consumes per step; with `world` > 1 the documents (parquet) are dealt to the
  // ranks round-robin and packed rows are dealt in blocks of `rows` per rank inside each global step.
  bool Open(const MeshTrainConfig& c, int seq, int rows, int rank, int world, std::string* error) {
    batch_ = rows, seq_ = seq, rank_ = rank, world_ = world;
    if (!c.packed_rows_path.empty()) {
      std::string magic;
      std::vector<FixtureRecord> recs;
      if (!ReadRecordFile(c.packed_rows_path, &magic, &recs, error)) return false;
      const FixtureRecord *tok = nullptr, *tgt = nullptr;
      for (const auto& r : recs) {
        if (r.name == "tokens") tok = &r;
        if (r.name == "targets") tgt = &r;
      }
      if (magic != "NCSFT001" || !tok || !tgt || tok->dtype != 1 || tgt->dtype != 1 || tok->dims.size() != 2 ||
          tok->dims != tgt->dims || static_cast<int>(tok->dims[1]) != seq) {
        if (error) *error = "packed rows: expected an NCSFT001 shard with int32 tokens/targets of the run's row length";
        return false;
      }
      rows_ = static_cast<std::size_t>(tok->dims[0]);
      tokens_.resize(rows_ * seq), targets_.resize(rows_ * seq);
      std::memcpy(tokens_.data(), tok->data.data(), tokens_.size() * 4);
      std::memcpy(targets_.data(), tgt->data.data(), targets_.size() * 4);
      return rows_ > 0;
    }
    tokenizer_ = Tokenizer::Load(c.tokenizer_path, error);
    if (!tokenizer_) return false;
    std::vector<std::vector<int>> docs;
    for (const std::string& path : ExpandGlobs(c.parquet)) {
      std::vector<std::string> text;
      if (!ReadParquetStrings(path, "text", &text, error)) return false;
      for (const std::string& d : text) docs.push_back(tokenizer_->Encode(d, tokenizer_->bos_id()));
    }
    if (docs.empty()) {
      if (error) *error = "no documents: check the parquet paths";
      return false;
    }
    std::unique_ptr<DocumentSource> src = VectorSource(std::move(docs));
    if (world > 1) src = ShardSource(std::move(src), rank, world);
    loader_ = std::make_unique<DataLoader>(std::move(src), rows, seq, 1000, 2, 1);
    return true;
  }
  void Next(int* tokens, int* targets) {
    if (loader_) {
      loader_->Next(tokens, targets);
      return;
    }
    for (int b = 0; b < batch_; ++b) {
      const std::size_t row = (cursor_ + static_cast<std::size_t>(rank_) * batch_ + b) % rows_;
      std::memcpy(tokens + static_cast<std::size_t>(b) * seq_, tokens_.data() + row * seq_, seq_ * 4);
      std::memcpy(targets + static_cast<std::size_t>(b) * seq_, targets_.data() + row * seq_, seq_ * 4);
    }
    cursor_ = (cursor_ + static_cast<std::size_t>(world_) * batch_) % rows_;
  }
  void Skip(int steps) {  // a resume replays the loader to the stored step
    if (loader_) {
      std::vector<int> a(static_cast<std::size_t>(batch_) * seq_), b(a.size());
      for (int i = 0; i < steps; ++i) loader_->Next(a.data(), b.data());
    } else if (rows_) {
      cursor_ = (static_cast<std::size_t>(steps) * batch_ * world_) % rows_;
    }
  }

 private:
  int batch_ = 0, seq_ = 0, rank_ = 0, world_ = 1;
  std::unique_ptr<Tokenizer> tokenizer_;
  std::unique_ptr<DataLoader> loader_;
  std::vector<int> tokens_, targets_;
  std::size_t rows_ = 0, cursor_ = 0;
};

bool FileExists(const std::string& path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0;
}

}  // namespace

float RunMeshTrain(const MeshTrainConfig& c, MeshTrainSummary* out, std::string* error) {
  const int seq = c.seq > 0 ? c.seq : c.model.seq_len;
  std::string out_dir = c.out_dir.empty() ? "." : c.out_dir;
  ::mkdir(out_dir.c_str(), 0755);
  const std::string ckpt = c.checkpoint_path.empty() ? out_dir + "/checkpoint.ckpt" : c.checkpoint_path;
  OptimConfig optim = c.optim;
  if (optim.num_iterations == 0) optim.num_iterations = c.num_iterations;
  MeshRuntime rt(c.mesh, c.model, optim, c.batch, c.grad_accum, seq, c.seed, error);
  if (!rt.ok()) return 0.0f;
  if (!c.warm_start_path.empty() && !rt.LoadWeights(c.warm_start_path, error)) return 0.0f;
  BatchSource data;
  if (!data.Open(c, seq, c.batch, 0, 1, error)) return 0.0f;
  if (c.resume && FileExists(ckpt)) {
    if (!rt.Load(ckpt, error)) return 0.0f;
    data.Skip(rt.step());
  }
  std::FILE* metrics = std::fopen((out_dir + "/metrics.jsonl").c_str(), c.resume ? "a" : "w");
  const double fpt = c.flops_per_token > 0 ? c.flops_per_token : EstimateFlopsPerToken(c.model);
  const double tokens_per_step = static_cast<double>(c.batch) * seq;
  g_interrupted = 0;
  auto previous = std::signal(SIGINT, OnSigint);
  std::vector<int> tokens(static_cast<std::size_t>(c.batch) * seq), targets(tokens.size());
  const int first = rt.step() + 1;
  double loss_sum = 0.0, mfu_sum = 0.0;
  int steps = 0, mfu_steps = 0;
  float last = 0.0f;
  bool failed = false;
  for (int step = first; step <= c.num_iterations; ++step) {
    data.Next(tokens.data(), targets.data());
    last = rt.TrainStep(tokens.data(), targets.data(), error);
    if (!rt.ok()) {
      failed = true;
      break;
    }
    const MeshMetrics& m = rt.metrics();
    const double tok_s = tokens_per_step / std::max(1e-9f, m.step_seconds);
    const double mfu = c.peak_flops > 0 ? tok_s * fpt / (c.peak_flops * rt.world()) : 0.0;
    ++steps;
    loss_sum += last;
    if (step > first) {  // the first step of a run carries one-time costs
      mfu_sum += mfu;
      ++mfu_steps;
    }
    if (metrics) {
      std::fprintf(metrics, "{\"step\": %d, \"loss\": %.6f, \"grad_norm\": %.6f, \"step_seconds\": %.6f, \"tok_s\": %.1f, \"mfu\": %.6f}\n",
                   step, last, m.grad_norm, m.step_seconds, tok_s, mfu);
      std::fflush(metrics);
    }
    const bool log_now = step == first || step == c.num_iterations || (c.log_every > 0 && step % c.log_every == 0);
    if (log_now)
      std::printf("step %6d | loss %.6f | grad_norm %.4f | tok/s %.0f | mfu %.4f | step_ms %.2f\n", step, last,
                  m.grad_norm, tok_s, mfu, m.step_seconds * 1e3);
    if (g_interrupted) break;
    if (c.save_every > 0 && step % c.save_every == 0 && step != c.num_iterations && !rt.Save(ckpt, error)) {
      failed = true;
      break;
    }
  }
  std::signal(SIGINT, previous);
  if (metrics) std::fclose(metrics);
  if (failed) return 0.0f;
  if (!rt.Save(ckpt, error)) return 0.0f;
  MeshTrainSummary s;
  s.steps = steps;
  s.interrupted = g_interrupted != 0 && rt.step() < c.num_iterations;
  s.mean_loss = steps ? loss_sum / steps : 0.0;
  s.steady_mfu = mfu_steps ? mfu_sum / mfu_steps : 0.0;
  s.checkpoint = ckpt;
  if (std::FILE* f = std::fopen((out_dir + "/summary.json").c_str(), "w")) {
    std::fprintf(f, "{\"steps\": %d, \"final_step\": %d, \"interrupted\": %s, \"mean_loss\": %.6f, \"final_loss\": %.6f, "
                    "\"steady_mfu\": %.6f, \"world_size\": %d, \"tokens_per_step\": %.0f, \"checkpoint\": \"%s\"}\n",
                 s.steps, rt.step(), s.interrupted ? "true" : "false", s.mean_loss, last, s.steady_mfu, rt.world(),
                 tokens_per_step, ckpt.c_str());
    std::fclose(f);
  }
  if (out) *out = s;
  return last;
}

float RunDistributedTrain(const MeshTrainConfig& c, const DistConfig& d, MeshTrainSummary* out, std::string* error) {
  const int seq = c.seq > 0 ? c.seq : c.model.seq_len;
  const int world = std::max(1, d.world), accum = std::max(1, c.grad_accum);
  if (d.rank < 0 || d.rank >= world || c.batch <= 0 || seq > c.model.seq_len) {
    if (error) *error = "bad rank, batch or sequence length";
    return 0.0f;
  }
  const bool writer = d.rank == 0;
  std::string out_dir = c.out_dir.empty() ? "." : c.out_dir;
  if (writer) ::mkdir(out_dir.c_str(), 0755);
  const std::string ckpt = c.checkpoint_path.empty() ? out_dir + "/checkpoint.ckpt" : c.checkpoint_path;
  TcpTransport link(d.rank, world);
  if (!RendezvousAndConnect(&link, d.port, d.timeout_ms)) {
    if (error) *error = link.error();
    return 0.0f;
  }
  OptimConfig optim = c.optim;
  if (optim.num_iterations == 0) optim.num_iterations = c.num_iterations;
  CpuModel model(c.model);
  model.InitWeights(c.seed);
  CpuOptimizer opt(&model, optim);
  if (!c.warm_start_path.empty() && !model.Load(c.warm_start_path, error)) return 0.0f;
  BatchSource data;
  if (!data.Open(c, seq, c.batch * accum, d.rank, world, error)) return 0.0f;
  int step0 = 0;
  if (c.resume && FileExists(ckpt)) {  // every rank reads the one canonical file
    std::uint64_t st = 0;
    if (!model.LoadWithOptimizer(ckpt, &opt, &st, error)) return 0.0f;
    step0 = static_cast<int>(st);
    data.Skip(step0);
  }
  std::FILE* metrics = writer ? std::fopen((out_dir + "/metrics.jsonl").c_str(), c.resume ? "a" : "w") : nullptr;
  const double fpt = c.flops_per_token > 0 ? c.flops_per_token : EstimateFlopsPerToken(c.model);
  const double tokens_per_step = static_cast<double>(c.batch) * accum * world * seq;
  const float scale = 1.0f / static_cast<float>(accum * world);
  g_interrupted = 0;
  auto previous = std::signal(SIGINT, OnSigint);
  std::vector<int> tokens(static_cast<std::size_t>(c.batch) * accum * seq), targets(tokens.size());
  double loss_sum = 0.0, mfu_sum = 0.0;
  int steps = 0, mfu_steps = 0, step = step0;
  float last = 0.0f;
  bool failed = false;
  while (step < c.num_iterations && !failed) {
    const auto t0 = std::chrono::steady_clock::now();
    data.Next(tokens.data(), targets.data());
    model.ZeroGrad();
    double loss = 0.0;
    for (int m = 0; m < accum; ++m) {
      const std::size_t off = static_cast<std::size_t>(m) * c.batch * seq;
      loss += model.ForwardLoss(tokens.data() + off, targets.data() + off, c.batch, seq);
      model.Backward(scale);
    }
    // the loss and the stop request travel with the gradients: two extra floats at the end of the reduced vector
    std::vector<float>& g = model.grads();
    const std::size_t n = g.size();
    g.push_back(static_cast<float>(loss / accum));
    g.push_back(g_interrupted ? 1.0f : 0.0f);
    const bool reduced = RingAllReduceSum(&link, g.data(), g.size(), d.timeout_ms);
    const float mean_loss = g[n] / world;
    const bool stop = g[n + 1] > 0.0f;
    g.resize(n);
    if (!reduced) {
      if (error) *error = "watchdog: rank " + std::to_string(d.rank) + ": " + link.error();
      failed = true;
      break;
    }
    ++step;
    opt.Step(step);
    last = mean_loss;
    const float secs = std::chrono::duration<float>(std::chrono::steady_clock::now() - t0).count();
    const double tok_s = tokens_per_step / std::max(1e-9f, secs);
    const double mfu = c.peak_flops > 0 ? tok_s * fpt / (c.peak_flops * world) : 0.0;
    ++steps;
    loss_sum += last;
    if (steps > 1) mfu_sum += mfu, ++mfu_steps;
    if (metrics) {
      std::fprintf(metrics, "{\"step\": %d, \"loss\": %.6f, \"grad_norm\": %.6f, \"step_seconds\": %.6f, \"tok_s\": %.1f, \"mfu\": %.6f}\n",
                   step, last, opt.grad_norm(), secs, tok_s, mfu);
      std::fflush(metrics);
    }
    if (writer && (steps == 1 || step == c.num_iterations || (c.log_every > 0 && step % c.log_every == 0)))
      std::printf("step %6d | loss %.6f | grad_norm %.4f | tok/s %.0f | mfu %.4f | step_ms %.2f\n", step, last,
                  opt.grad_norm(), tok_s, mfu, secs * 1e3);
    if (stop) break;  // every rank saw the same flag, so all leave after the same step
    if (writer && c.save_every > 0 && step % c.save_every == 0 && step != c.num_iterations &&
        !model.SaveWithOptimizer(ckpt, opt, static_cast<std::uint64_t>(step), static_cast<std::uint32_t>(world), error))
      failed = true;
  }
  std::signal(SIGINT, previous);
  if (metrics) std::fclose(metrics);
  if (failed) return 0.0f;
  if (writer && !model.SaveWithOptimizer(ckpt, opt, static_cast<std::uint64_t>(step), static_cast<std::uint32_t>(world), error))
    return 0.0f;
  MeshTrainSummary s;
  s.steps = steps;
  s.interrupted = step < c.num_iterations;
  s.mean_loss = steps ? loss_sum / steps : 0.0;
  s.steady_mfu = mfu_steps ? mfu_sum / mfu_steps : 0.0;
  s.checkpoint = ckpt;
  if (writer) {
    if (std::FILE* f = std::fopen((out_dir + "/summary.json").c_str(), "w")) {
      std::fprintf(f, "{\"steps\": %d, \"final_step\": %d, \"interrupted\": %s, \"mean_loss\": %.6f, \"final_loss\": %.6f, "
                      "\"steady_mfu\": %.6f, \"world_size\": %d, \"tokens_per_step\": %.0f, \"checkpoint\": \"%s\"}\n",
                   s.steps, step, s.interrupted ? "true" : "false", s.mean_loss, last, s.steady_mfu, world,
                   tokens_per_step, ckpt.c_str());
      std::fclose(f);
    }
  }
  if (out) *out = s;
  return last;
}

}  // namespace ncb
