// Benchmark harness around the unmodified reference (ming6ao/nanochat.cpp).
//
// `ref_train train ...` does what the reference's own `nanochat_cli train` does
// (src/train_command.cc:65-179 of the reference: environment contract NANOCHAT_RANK / WORLD_SIZE /
// MASTER_ADDR / MASTER_PORT, the same flags, `TrainLoop loop(config); loop.Run();`) with one difference:
// the documents come from an in-memory synthetic source plugged into `TrainConfig::train_source`
// (src/train.h:78-81), the hook the reference provides for running without its parquet reader.
// Everything below that hook is the reference's stock path: its DataLoader tokenizes and best-fit packs
// the documents on its producer thread, its Model / Optimizer / GradientSync run the step, and its Logger
// prints the per-step line this harness's caller parses.
//
// The synthetic corpus: every document is `--doc-tokens` words, every word is one space and one to three
// ASCII letters, and `ref_train make-tokenizer` writes an NCTOKEN1 artifact (through the reference's own
// `SaveTokenizer`) whose merges make each such word exactly one token. Word ranks are drawn Zipf(s) and
// scattered over the vocabulary by a fixed multiplicative permutation, so the token stream the model sees
// is Zipf(s) over (vocab - 256 byte tokens - 9 specials) ids with a BOS at the start of every row.
//
// `ref_train generate ...` times the reference's own `GenerateBatch` path for the decode benchmark.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "nanochat/config.h"
#include "nanochat/dataloader.h"
#include "nanochat/kernels.h"
#include "nanochat/mesh.h"
#include "nanochat/model.h"
#include "nanochat/tokenizer.h"
#include "src/cli.h"
#include "src/tokenizer/split_pattern.h"
#include "src/tokenizer/tokenizer_internal.h"
#include "src/train.h"

namespace {

constexpr int kLetters = 52;
constexpr int kByteTokens = 256;
constexpr int kSpecials = 9;

char Letter(int i) { return static_cast<char>(i < 26 ? 'a' + i : 'A' + (i - 26)); }

// Merge index m (0-based; token id 256 + m) -> the word that encodes to it.
//   level 1: " x"   m in [0, 52)            level 2: " xy"  m in [52, 52 + 52^2)
//   level 3: " xyz" m in [52 + 52^2, ...)
std::string WordOfMerge(int m) {
  std::string w = " ";
  if (m < kLetters) {
    w.push_back(Letter(m));
    return w;
  }
  m -= kLetters;
  if (m < kLetters * kLetters) {
    w.push_back(Letter(m / kLetters));
    w.push_back(Letter(m % kLetters));
    return w;
  }
  m -= kLetters * kLetters;
  w.push_back(Letter(m / (kLetters * kLetters)));
  w.push_back(Letter((m / kLetters) % kLetters));
  w.push_back(Letter(m % kLetters));
  return w;
}

int MakeTokenizer(const std::string& path, int vocab) {
  const int merges = vocab - kByteTokens - kSpecials;
  if (merges < kLetters + kLetters * kLetters || merges > kLetters + kLetters * kLetters + kLetters * kLetters * kLetters) {
    std::fprintf(stderr, "make-tokenizer: vocab %d out of range for the three-letter scheme\n", vocab);
    return 2;
  }
  std::vector<std::pair<std::uint32_t, std::uint32_t>> pairs;
  pairs.reserve(merges);
  for (int m = 0; m < merges; ++m) {
    if (m < kLetters) {
      pairs.emplace_back(static_cast<std::uint32_t>(' '), static_cast<std::uint32_t>(Letter(m)));
    } else if (m < kLetters + kLetters * kLetters) {
      const int r = m - kLetters;
      pairs.emplace_back(static_cast<std::uint32_t>(kByteTokens + r / kLetters),
                         static_cast<std::uint32_t>(Letter(r % kLetters)));
    } else {
      const int r = m - kLetters - kLetters * kLetters;
      pairs.emplace_back(static_cast<std::uint32_t>(kByteTokens + kLetters + r / kLetters),
                         static_cast<std::uint32_t>(Letter(r % kLetters)));
    }
  }
  static const char* kNames[kSpecials] = {"<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>",
                                          "<|assistant_end|>", "<|python_start|>", "<|python_end|>",
                                          "<|output_start|>", "<|output_end|>"};
  std::vector<std::pair<std::string, std::uint32_t>> specials;
  for (int i = 0; i < kSpecials; ++i) {
    specials.emplace_back(kNames[i], static_cast<std::uint32_t>(kByteTokens + merges + i));
  }
  if (!nanochat::SaveTokenizer(path, nanochat::NanochatSplitPattern(), pairs, specials)) {
    std::fprintf(stderr, "make-tokenizer: cannot write %s\n", path.c_str());
    return 1;
  }
  // Self-check through the reference's own loader and encoder.
  auto tok = nanochat::LoadTokenizer(path);
  if (tok == nullptr || tok->vocab_size() != vocab) {
    std::fprintf(stderr, "make-tokenizer: artifact does not load back with vocab %d\n", vocab);
    return 1;
  }
  for (int m : {0, 51, 52, 52 + 2703, 52 + 2704, merges - 1}) {
    const std::vector<int> ids = tok->Encode(WordOfMerge(m) + WordOfMerge((m * 7 + 3) % merges));
    if (ids.size() != 2 || ids[0] != kByteTokens + m) {
      std::fprintf(stderr, "make-tokenizer: word of merge %d encodes to %zu ids (first %d)\n", m, ids.size(),
                   ids.empty() ? -1 : ids[0]);
      return 1;
    }
  }
  std::printf("make-tokenizer: %s vocab %d merges %d bos %d\n", path.c_str(), vocab, merges, tok->bos_id());
  return 0;
}

// splitmix64: one stream per document index, so every rank regenerates the same corpus.
inline std::uint64_t Mix(std::uint64_t& s) {
  s += 0x9E3779B97F4A7C15ull;
  std::uint64_t z = s;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

class ZipfSource : public nanochat::DocumentSource {
 public:
  ZipfSource(int merges, int doc_tokens, double s, std::uint64_t seed)
      : merges_(merges), doc_tokens_(doc_tokens), seed_(seed) {
    cdf_.resize(merges);
    double total = 0.0;
    for (int k = 0; k < merges; ++k) {
      total += 1.0 / std::pow(static_cast<double>(k + 1), s);
      cdf_[k] = total;
    }
    for (double& c : cdf_) c /= total;
    words_.resize(merges);
    for (int m = 0; m < merges; ++m) words_[m] = WordOfMerge(m);
    multiplier_ = 40503;
    auto gcd = [](std::uint64_t a, std::uint64_t b) {
      while (b != 0) {
        const std::uint64_t t = a % b;
        a = b;
        b = t;
      }
      return a;
    };
    while (gcd(multiplier_, static_cast<std::uint64_t>(merges)) != 1) ++multiplier_;
  }

  bool Next(std::vector<std::string>* documents, std::string* error) override {
    if (error != nullptr) error->clear();
    documents->clear();
    for (int d = 0; d < 8; ++d) {
      std::uint64_t state = seed_ ^ (0xD1B54A32D192ED03ull * static_cast<std::uint64_t>(position_ + 1));
      std::string doc;
      doc.reserve(static_cast<std::size_t>(doc_tokens_) * 4);
      for (int t = 0; t < doc_tokens_; ++t) {
        const double u = static_cast<double>(Mix(state) >> 11) * (1.0 / 9007199254740992.0);
        const int rank = static_cast<int>(std::lower_bound(cdf_.begin(), cdf_.end(), u) - cdf_.begin());
        // fixed permutation of ranks over the merge ids (multiplier coprime to the count): hot tokens land
        // on scattered embedding rows, as in a trained vocabulary
        const std::uint64_t id = (static_cast<std::uint64_t>(std::min(rank, merges_ - 1)) * multiplier_ + 12345ull) %
                                 static_cast<std::uint64_t>(merges_);
        doc += words_[static_cast<std::size_t>(id)];
      }
      documents->push_back(std::move(doc));
      ++position_;
    }
    return true;
  }

  std::int64_t position() const override { return position_; }

 private:
  int merges_;
  int doc_tokens_;
  std::uint64_t seed_;
  std::uint64_t multiplier_ = 1;
  std::int64_t position_ = 0;
  std::vector<double> cdf_;
  std::vector<std::string> words_;
};

int RunTrainHarness(int argc, char** argv) {
  using namespace nanochat;
  TrainConfig config;
  config.rank = cli::EnvInt("NANOCHAT_RANK", config.rank);
  config.world_size = cli::EnvInt("NANOCHAT_WORLD_SIZE", config.world_size);
  config.master = cli::EnvString("NANOCHAT_MASTER_ADDR", config.master);
  config.port = cli::EnvInt("NANOCHAT_MASTER_PORT", config.port);
  float zipf_s = 1.1f;
  int doc_tokens = 0;
  int device_index = -1;

  cli::FlagParser flags("ref_train train");
  flags.AddString("--tokenizer", &config.tokenizer_path);
  flags.AddInt("--tokenizer-threads", &config.tokenizer_threads);
  flags.AddInt("--buffer-docs", &config.document_buffer);
  flags.AddInt("--batch", &config.batch);
  flags.AddInt("--grad-accum", &config.grad_accum);
  flags.AddInt("--num-iterations", &config.num_iterations);
  flags.AddInt("--log-every", &config.log_every);
  flags.AddU64("--seed", &config.seed);
  flags.AddString("--log", &config.log_path);
  flags.AddString("--device", &config.device_name);
  flags.AddValue("--hw-check", [&config](std::string_view value) { return ParseHwCheck(value, &config.hw_check); });
  flags.AddInt("--rank", &config.rank);
  flags.AddInt("--world-size", &config.world_size);
  flags.AddString("--master", &config.master);
  flags.AddInt("--port", &config.port);
  flags.AddInt("--muon-ns-steps", &config.optimizer.muon_ns_steps);
  flags.AddInt("--warmup-steps", &config.scheduler.warmup_steps);
  flags.AddFloat("--zipf", &zipf_s);
  flags.AddInt("--doc-tokens", &doc_tokens);
  flags.AddInt("--device-index", &device_index);
  flags.AddModelFlags(&config.model);
  const int parse_status = flags.Parse(argc, argv);
  if (parse_status != -1) return parse_status;
  if (config.tokenizer_path.empty()) {
    std::fprintf(stderr, "ref_train: --tokenizer is required\n");
    return 2;
  }
  if (doc_tokens <= 0) doc_tokens = config.model.seq_len;
  if (device_index >= 0) SelectDevice(device_index);

  const int merges = config.model.vocab_size - kByteTokens - kSpecials;
  const std::uint64_t seed = config.seed;
  config.train_source = [merges, doc_tokens, zipf_s, seed](std::string* error) -> std::unique_ptr<DocumentSource> {
    if (error != nullptr) error->clear();
    return std::make_unique<ZipfSource>(merges, doc_tokens, static_cast<double>(zipf_s), seed);
  };

  std::setvbuf(stdout, nullptr, _IOLBF, 0);
  const Caps caps = kernels::GetCaps();
  std::printf("[harness] backend device=%d name=%s feature_mask=0x%llx rank=%d world=%d\n", caps.is_device ? 1 : 0,
              config.device_name.c_str(), static_cast<unsigned long long>(caps.feature_mask), config.rank,
              config.world_size);
  const auto t0 = std::chrono::steady_clock::now();
  TrainLoop loop(std::move(config));
  std::printf("[harness] constructed in %.1f s\n",
              std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
  const float loss = loop.Run();
  std::printf("[harness] final loss %.6f at step %d\n", static_cast<double>(loss), loop.last_step());
  return 0;
}

}  // namespace

int RunGenerateHarness(int argc, char** argv);

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: ref_train <make-tokenizer|train|generate> [flags]\n");
    return 2;
  }
  const std::string verb = argv[1];
  if (verb == "make-tokenizer") {
    std::string path;
    int vocab = 65536;
    for (int i = 2; i + 1 < argc; i += 2) {
      if (std::strcmp(argv[i], "--out") == 0) path = argv[i + 1];
      if (std::strcmp(argv[i], "--vocab") == 0) vocab = std::atoi(argv[i + 1]);
    }
    if (path.empty()) {
      std::fprintf(stderr, "make-tokenizer: --out is required\n");
      return 2;
    }
    return MakeTokenizer(path, vocab);
  }
  if (verb == "train") return RunTrainHarness(argc - 1, argv + 1);
  if (verb == "generate") return RunGenerateHarness(argc - 1, argv + 1);
  std::fprintf(stderr, "ref_train: unknown verb %s\n", verb.c_str());
  return 2;
}

// ---------------------------------------------------------------------------------------------------------
// Decode benchmark through the reference's own generation path (src/generate.cc:458-576, `GenerateBatch`):
// random-init weights of the named architecture, `--prompts` prompts of `--prompt-tokens` uniform-random ids,
// greedy decode of `--max-tokens` tokens each. The reference prefills once per prompt at batch 1 and decodes
// row by row; `GenerateMultiPrompt` is its batched-prompt entry. Prints one line with the wall-clock seconds.
// ---------------------------------------------------------------------------------------------------------
int RunGenerateHarness(int argc, char** argv) {
  using namespace nanochat;
  Config model;
  int prompts = 64;
  int prompt_tokens = 512;
  int max_tokens = 256;
  int device_index = -1;
  std::uint64_t seed = 0;
  cli::FlagParser flags("ref_train generate");
  flags.AddInt("--prompts", &prompts);
  flags.AddInt("--prompt-tokens", &prompt_tokens);
  flags.AddInt("--max-tokens", &max_tokens);
  flags.AddInt("--device-index", &device_index);
  flags.AddU64("--seed", &seed);
  flags.AddModelFlags(&model);
  const int parse_status = flags.Parse(argc, argv);
  if (parse_status != -1) return parse_status;
  if (device_index >= 0) SelectDevice(device_index);
  std::setvbuf(stdout, nullptr, _IOLBF, 0);

  std::unique_ptr<Model> m = Model::Create(model);
  if (m == nullptr) {
    std::fprintf(stderr, "generate: cannot create the model\n");
    return 1;
  }
  m->InitWeights(seed);
  std::uint64_t state = seed + 17;
  std::vector<int> all(static_cast<std::size_t>(prompts) * static_cast<std::size_t>(prompt_tokens));
  for (int& t : all) t = static_cast<int>(Mix(state) % static_cast<std::uint64_t>(model.vocab_size));
  GenerateParams params;
  params.max_tokens = max_tokens;
  params.num_samples = 1;
  params.temperature = 0.0f;
  params.top_k = 0;
  params.stop_id = -1;
  params.bos_id = -1;
  params.seed = seed;
  std::int64_t generated = 0;
  // one untimed prompt first: workspaces, cuBLAS handles and plan caches are created on first use
  {
    std::vector<GeneratedSequence> warm;
    GenerateParams wp = params;
    wp.max_tokens = 4;
    GenerateBatch(m.get(), all.data(), prompt_tokens, wp, &warm);
    kernels::Synchronize();
  }
  const auto wall0 = std::chrono::steady_clock::now();
  std::vector<GeneratedSequence> out;
  GenerateMultiPrompt(m.get(), all.data(), prompts, prompt_tokens, params, nullptr, &out);
  kernels::Synchronize();
  for (const GeneratedSequence& s : out) generated += static_cast<std::int64_t>(s.tokens.size()) - prompt_tokens;
  const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - wall0).count();
  std::printf("[harness] generate prompts=%d prompt_tokens=%d new_tokens=%lld wall_s=%.6f\n", prompts,
              prompt_tokens, static_cast<long long>(generated), wall);
  return 0;
}
