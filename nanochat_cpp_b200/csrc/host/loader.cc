// Random numbers, sampling, document sources and the best-fit packing data loader.
#include <algorithm>
#include <cmath>
#include <condition_variable>
#include <deque>
#include <fstream>
#include <limits>
#include <mutex>
#include <thread>

#include "core.h"

namespace ncb {

// ------------------------------------------------------------------ RNG
namespace {
inline std::uint64_t Rotl(std::uint64_t v, int s) { return (v << s) | (v >> (64 - s)); }
inline std::uint64_t SplitMix(std::uint64_t* x) {
  *x += 0x9e3779b97f4a7c15ULL;
  std::uint64_t z = *x;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}
}  // namespace

Rng::Rng(std::uint64_t seed) {
  for (auto& s : s_) s = SplitMix(&seed);
  if ((s_[0] | s_[1] | s_[2] | s_[3]) == 0) s_[0] = 1;
}
std::uint64_t Rng::NextU64() {
  const std::uint64_t result = Rotl(s_[1] * 5, 7) * 9;
  const std::uint64_t t = s_[1] << 17;
  s_[2] ^= s_[0];
  s_[3] ^= s_[1];
  s_[1] ^= s_[2];
  s_[0] ^= s_[3];
  s_[2] ^= t;
  s_[3] = Rotl(s_[3], 45);
  return result;
}
double Rng::NextDouble() { return static_cast<double>(NextU64() >> 11) * 0x1.0p-53; }
std::uint64_t Rng::NextBelow(std::uint64_t n) { return n == 0 ? 0 : NextU64() % n; }
double Rng::NextNormal() {
  if (have_spare_) {
    have_spare_ = false;
    return spare_;
  }
  const double u1 = 1.0 - NextDouble(), u2 = NextDouble();
  const double r = std::sqrt(-2.0 * std::log(u1));
  spare_ = r * std::sin(6.283185307179586 * u2);
  have_spare_ = true;
  return r * std::cos(6.283185307179586 * u2);
}
std::uint64_t MixSeed(std::uint64_t seed, std::uint64_t stream) {
  std::uint64_t x = seed + stream * 0x9e3779b97f4a7c15ULL;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
  return x ^ (x >> 31);
}

// ------------------------------------------------------------------ sampling
int SampleToken(const float* logits, int vocab, float temperature, int top_k, Rng* rng) {
  if (logits == nullptr || vocab <= 0) return -1;
  if (!(temperature > 0.0f)) {
    int best = 0;
    for (int i = 1; i < vocab; ++i)
      if (logits[i] > logits[best]) best = i;
    return best;
  }
  std::vector<float> scores(logits, logits + vocab);
  if (top_k > 0 && top_k < vocab) {
    std::vector<float> sorted(scores);
    std::nth_element(sorted.begin(), sorted.begin() + (top_k - 1), sorted.end(), std::greater<float>());
    const float threshold = sorted[top_k - 1];
    for (float& s : scores)
      if (s < threshold) s = -std::numeric_limits<float>::infinity();
  }
  const float inv_t = 1.0f / temperature;
  float mx = -std::numeric_limits<float>::infinity();
  for (float& s : scores) {
    s *= inv_t;
    mx = std::max(mx, s);
  }
  double sum = 0.0;
  for (float& s : scores) {
    s = std::exp(s - mx);
    sum += s;
  }
  Rng local(0);
  Rng* g = rng != nullptr ? rng : &local;
  const float r = static_cast<float>(g->NextU64() >> 40) * 0x1p-24f * static_cast<float>(sum);
  float cum = 0.0f;
  for (int i = 0; i < vocab; ++i) {
    cum += scores[i];
    if (r <= cum) return i;
  }
  return vocab - 1;
}

// ------------------------------------------------------------------ document sources
namespace {

class VectorDocs final : public DocumentSource {
 public:
  explicit VectorDocs(std::vector<std::vector<int>> docs) : docs_(std::move(docs)) {}
  bool Next(std::vector<int>* tokens) override {
    if (docs_.empty()) return false;
    if (pos_ >= docs_.size()) {
      pos_ = 0;
      return false;
    }
    *tokens = docs_[pos_++];
    return true;
  }
  void Reset() override { pos_ = 0; }

 private:
  std::vector<std::vector<int>> docs_;
  std::size_t pos_ = 0;
};

class Sharded final : public DocumentSource {
 public:
  Sharded(std::unique_ptr<DocumentSource> inner, int rank, int world)
      : inner_(std::move(inner)), rank_(rank), world_(std::max(1, world)) {}
  bool Next(std::vector<int>* tokens) override {
    while (true) {
      std::vector<int> doc;
      if (!inner_->Next(&doc)) {
        index_ = 0;
        return false;
      }
      const bool mine = (index_ % world_) == static_cast<std::uint64_t>(rank_);
      ++index_;
      if (mine) {
        *tokens = std::move(doc);
        return true;
      }
    }
  }
  void Reset() override {
    inner_->Reset();
    index_ = 0;
  }

 private:
  std::unique_ptr<DocumentSource> inner_;
  int rank_, world_;
  std::uint64_t index_ = 0;
};

class ZipfDocs final : public DocumentSource {
 public:
  ZipfDocs(int vocab, int doc_len, double s, std::uint64_t seed)
      : vocab_(vocab), doc_len_(doc_len), seed_(seed), rng_(seed) {
    cdf_.resize(std::max(1, vocab - 1));
    double acc = 0.0;
    for (int r = 1; r < vocab; ++r) {
      acc += std::pow(static_cast<double>(r), -s);
      cdf_[r - 1] = acc;
    }
    for (double& c : cdf_) c /= acc;
  }
  bool Next(std::vector<int>* tokens) override {
    tokens->resize(doc_len_);
    (*tokens)[0] = 0;  // BOS
    for (int i = 1; i < doc_len_; ++i) {
      const double u = rng_.NextDouble();
      const auto it = std::lower_bound(cdf_.begin(), cdf_.end(), u);
      (*tokens)[i] = std::min(vocab_ - 1, static_cast<int>(it - cdf_.begin()) + 1);
    }
    return true;
  }
  void Reset() override { rng_ = Rng(seed_); }

 private:
  int vocab_, doc_len_;
  std::uint64_t seed_;
  Rng rng_;
  std::vector<double> cdf_;
};

class TextLines final : public DocumentSource {
 public:
  TextLines(std::vector<std::string> docs, const Tokenizer* tok) : docs_(std::move(docs)), tok_(tok) {}
  bool Next(std::vector<int>* tokens) override {
    if (docs_.empty()) return false;
    if (pos_ >= docs_.size()) {
      pos_ = 0;
      return false;
    }
    *tokens = tok_->Encode(docs_[pos_++], tok_->bos_id());
    return true;
  }
  void Reset() override { pos_ = 0; }

 private:
  std::vector<std::string> docs_;
  const Tokenizer* tok_;
  std::size_t pos_ = 0;
};

}  // namespace

std::unique_ptr<DocumentSource> VectorSource(std::vector<std::vector<int>> docs) {
  return std::make_unique<VectorDocs>(std::move(docs));
}
std::unique_ptr<DocumentSource> ShardSource(std::unique_ptr<DocumentSource> inner, int rank, int world) {
  return std::make_unique<Sharded>(std::move(inner), rank, world);
}
std::unique_ptr<DocumentSource> ZipfSource(int vocab, int doc_len, double s, std::uint64_t seed) {
  return std::make_unique<ZipfDocs>(vocab, doc_len, s, seed);
}
std::unique_ptr<DocumentSource> TextFileSource(const std::string& path, const Tokenizer* tok) {
  std::ifstream f(path);
  std::vector<std::string> docs;
  std::string line;
  while (std::getline(f, line))
    if (!line.empty()) docs.push_back(line);
  return std::make_unique<TextLines>(std::move(docs), tok);
}
std::unique_ptr<DocumentSource> ParquetSource(const std::string& path, const std::string& column,
                                              const Tokenizer* tok, std::string* error) {
  std::vector<std::string> docs;
  if (!ReadParquetStrings(path, column, &docs, error)) return nullptr;
  return std::make_unique<TextLines>(std::move(docs), tok);
}

// ------------------------------------------------------------------ data loader
struct DataLoader::Impl {
  std::unique_ptr<DocumentSource> source;
  int batch, seq, buffer_docs, prefetch, source_batch = 1;
  // packing state (owned by the producer thread, or by the caller while the producer is stopped)
  std::vector<std::vector<int>> buffer;
  std::uint64_t epoch = 0, position = 0;
  // hand-off
  struct Batch {
    std::vector<int> rows;  // [batch, seq + 1]
    LoaderState state_after;
  };
  std::deque<Batch> ready;
  LoaderState consumed_state;
  std::mutex mu;
  std::condition_variable cv_ready, cv_space;
  std::thread worker;
  bool stop = false;

  void Refill() {
    int guard = 0;
    while (static_cast<int>(buffer.size()) < buffer_docs && guard < 4) {
      for (int k = 0; k < source_batch && guard < 4;) {
        std::vector<int> doc;
        if (source->Next(&doc)) {
          ++position;
          ++k;
          if (!doc.empty()) buffer.push_back(std::move(doc));
          guard = 0;
        } else {
          ++epoch;
          position = 0;
          ++guard;  // an empty source must not spin forever
        }
      }
    }
  }

  // One row of capacity seq + 1: take the largest buffered document that fits the remaining space; when none
  // fits, crop the shortest document to fill the row exactly.
  void PackRow(int* row) {
    const int cap = seq + 1;
    int filled = 0;
    while (filled < cap) {
      Refill();
      if (buffer.empty()) {  // no data at all: pad with zeros
        std::fill(row + filled, row + cap, 0);
        return;
      }
      const int space = cap - filled;
      int best = -1;
      for (int i = 0; i < static_cast<int>(buffer.size()); ++i) {
        const int len = static_cast<int>(buffer[i].size());
        if (len <= space && (best < 0 || len > static_cast<int>(buffer[best].size()))) best = i;
      }
      if (best >= 0) {
        std::copy(buffer[best].begin(), buffer[best].end(), row + filled);
        filled += static_cast<int>(buffer[best].size());
        buffer.erase(buffer.begin() + best);
      } else {
        int shortest = 0;
        for (int i = 1; i < static_cast<int>(buffer.size()); ++i)
          if (buffer[i].size() < buffer[shortest].size()) shortest = i;
        std::copy(buffer[shortest].begin(), buffer[shortest].begin() + space, row + filled);
        filled += space;
        buffer.erase(buffer.begin() + shortest);
      }
    }
  }

  Batch Produce() {
    Batch b;
    b.rows.resize(static_cast<std::size_t>(batch) * (seq + 1));
    for (int r = 0; r < batch; ++r) PackRow(b.rows.data() + static_cast<std::size_t>(r) * (seq + 1));
    b.state_after.epoch = epoch;
    b.state_after.position = position;
    b.state_after.buffered = buffer;
    return b;
  }

  void Run() {
    while (true) {
      {
        std::unique_lock<std::mutex> lock(mu);
        cv_space.wait(lock, [&] { return stop || static_cast<int>(ready.size()) < prefetch; });
        if (stop) return;
      }
      Batch b = Produce();
      {
        std::lock_guard<std::mutex> lock(mu);
        ready.push_back(std::move(b));
      }
      cv_ready.notify_one();
    }
  }

  void Start() {
    stop = false;
    worker = std::thread([this] { Run(); });
  }
  void Stop() {
    {
      std::lock_guard<std::mutex> lock(mu);
      stop = true;
    }
    cv_space.notify_all();
    if (worker.joinable()) worker.join();
  }
};

DataLoader::DataLoader(std::unique_ptr<DocumentSource> source, int batch, int seq, int buffer_docs, int prefetch,
                       int source_batch)
    : impl_(std::make_unique<Impl>()) {
  impl_->source_batch = std::max(1, source_batch);
  impl_->source = std::move(source);
  impl_->batch = batch;
  impl_->seq = seq;
  impl_->buffer_docs = std::max(1, buffer_docs);
  impl_->prefetch = std::max(1, prefetch);
  impl_->Start();
}
DataLoader::~DataLoader() { impl_->Stop(); }

void DataLoader::Next(int* tokens, int* targets) {
  Impl::Batch b;
  {
    std::unique_lock<std::mutex> lock(impl_->mu);
    impl_->cv_ready.wait(lock, [&] { return !impl_->ready.empty(); });
    b = std::move(impl_->ready.front());
    impl_->ready.pop_front();
    impl_->consumed_state = b.state_after;
  }
  impl_->cv_space.notify_one();
  const int seq = impl_->seq;
  for (int r = 0; r < impl_->batch; ++r) {
    const int* row = b.rows.data() + static_cast<std::size_t>(r) * (seq + 1);
    std::copy(row, row + seq, tokens + static_cast<std::size_t>(r) * seq);
    std::copy(row + 1, row + seq + 1, targets + static_cast<std::size_t>(r) * seq);
  }
}

LoaderState DataLoader::State() const {
  std::lock_guard<std::mutex> lock(impl_->mu);
  return impl_->consumed_state;
}
std::uint64_t DataLoader::epoch() const { return State().epoch; }

void DataLoader::Restore(const LoaderState& state) {
  impl_->Stop();
  impl_->ready.clear();
  // rewind the source to the recorded position of the recorded epoch
  std::vector<int> scratch;
  impl_->source->Reset();
  for (std::uint64_t i = 0; i < state.position; ++i)
    if (!impl_->source->Next(&scratch)) break;
  impl_->epoch = state.epoch;
  impl_->position = state.position;
  impl_->buffer = state.buffered;
  impl_->consumed_state = state;
  impl_->Start();
}

}  // namespace ncb
