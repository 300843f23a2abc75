// Binary formats: fixture record container, NCHKPT01 checkpoints with the metadata word stream, data cursor.
#include <bit>
#include <cmath>
#include <cstring>
#include <fstream>

#include "core.h"

namespace ncb {

namespace {

class Reader {
 public:
  explicit Reader(std::istream& in) : in_(in) {}
  template <typename T>
  bool Get(T* v) {
    in_.read(reinterpret_cast<char*>(v), sizeof(T));
    return static_cast<bool>(in_);
  }
  bool Bytes(void* dst, std::size_t n) {
    if (n == 0) return true;
    in_.read(static_cast<char*>(dst), static_cast<std::streamsize>(n));
    return static_cast<bool>(in_);
  }
  bool AtEnd() { return in_.peek() == std::char_traits<char>::eof(); }

 private:
  std::istream& in_;
};

template <typename T>
void Put(std::ostream& out, T v) {
  out.write(reinterpret_cast<const char*>(&v), sizeof(T));
}

bool Fail(std::string* error, const std::string& msg) {
  if (error != nullptr) *error = msg;
  return false;
}

constexpr std::uint32_t kMaxStringWords = 4096;
constexpr std::uint32_t kMaxVectorEntries = 1024;
constexpr std::size_t kMaxBlockWords = 64 * 1024 / sizeof(std::uint32_t);

// ---- metadata word stream ------------------------------------------------------------------
class WordWriter {
 public:
  void U32(std::uint32_t v) { w_.push_back(v); }
  void I32(std::int32_t v) { w_.push_back(std::bit_cast<std::uint32_t>(v)); }
  void U64(std::uint64_t v) {
    w_.push_back(static_cast<std::uint32_t>(v & 0xffffffffu));
    w_.push_back(static_cast<std::uint32_t>(v >> 32));
  }
  void F32(float v) {
    if (!std::isfinite(v)) ok_ = false;
    w_.push_back(std::bit_cast<std::uint32_t>(v));
  }
  void Str(const std::string& s) {
    if (s.size() > kMaxStringWords * 4) {
      ok_ = false;
      return;
    }
    w_.push_back(static_cast<std::uint32_t>(s.size()));
    const std::size_t start = w_.size();
    w_.resize(start + (s.size() + 3) / 4, 0);
    for (std::size_t i = 0; i < s.size(); ++i)
      w_[start + i / 4] |= static_cast<std::uint32_t>(static_cast<unsigned char>(s[i])) << (8 * (i % 4));
  }
  std::size_t BeginBlock() {
    w_.push_back(0);
    return w_.size() - 1;
  }
  void EndBlock(std::size_t at) { w_[at] = static_cast<std::uint32_t>(w_.size() - at - 1); }
  bool ok() const { return ok_; }
  std::vector<std::uint32_t> Take() { return std::move(w_); }

 private:
  std::vector<std::uint32_t> w_;
  bool ok_ = true;
};

// Reads fields in order; running out of words inside a block keeps the defaults of the remaining fields.
class WordReader {
 public:
  WordReader(const std::vector<std::uint32_t>& w, std::size_t pos, std::size_t end) : w_(&w), pos_(pos), end_(end) {}
  bool Has(std::size_t n = 1) const { return pos_ + n <= end_; }
  bool U32(std::uint32_t* v) {
    if (!Has()) return false;
    *v = (*w_)[pos_++];
    return true;
  }
  bool I32(std::int32_t* v) {
    std::uint32_t u;
    if (!U32(&u)) return false;
    *v = std::bit_cast<std::int32_t>(u);
    return true;
  }
  bool U64(std::uint64_t* v) {
    if (!Has(2)) return false;
    *v = static_cast<std::uint64_t>((*w_)[pos_]) | (static_cast<std::uint64_t>((*w_)[pos_ + 1]) << 32);
    pos_ += 2;
    return true;
  }
  bool F32(float* v) {
    std::uint32_t u;
    if (!U32(&u)) return false;
    const float f = std::bit_cast<float>(u);
    if (!std::isfinite(f)) {
      bad_ = true;
      return false;
    }
    *v = f;
    return true;
  }
  bool Str(std::string* s) {
    std::uint32_t n;
    if (!U32(&n)) return false;
    const std::size_t words = (static_cast<std::size_t>(n) + 3) / 4;
    if (n > kMaxStringWords * 4 || !Has(words)) {
      bad_ = true;
      return false;
    }
    s->assign(n, '\0');
    for (std::uint32_t i = 0; i < n; ++i) (*s)[i] = static_cast<char>(((*w_)[pos_ + i / 4] >> (8 * (i % 4))) & 0xff);
    pos_ += words;
    return true;
  }
  // Enters a nested block: returns a reader over its payload and advances this reader past it.
  bool Block(WordReader* inner) {
    std::uint32_t n;
    if (!U32(&n)) return false;
    if (!Has(n)) {
      bad_ = true;
      return false;
    }
    *inner = WordReader(*w_, pos_, pos_ + n);
    pos_ += n;
    return true;
  }
  std::size_t Remaining() const { return end_ - pos_; }
  bool bad() const { return bad_; }
  void Poison() { bad_ = true; }

 private:
  const std::vector<std::uint32_t>* w_;
  std::size_t pos_, end_;
  bool bad_ = false;
};

}  // namespace

// ------------------------------------------------------------------ small helpers
std::size_t DTypeSize(DType t) {
  switch (t) {
    case DType::kFp32: return 4;
    case DType::kBf16: return 2;
    default: return 1;
  }
}
std::uint16_t FloatToBf16(float v) {
  std::uint32_t u = std::bit_cast<std::uint32_t>(v);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<std::uint16_t>((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<std::uint16_t>(u >> 16);
}
float Bf16ToFloat(std::uint16_t v) { return std::bit_cast<float>(static_cast<std::uint32_t>(v) << 16); }

std::int64_t TensorRecord::NumElements() const {
  std::int64_t n = 1;
  for (std::int64_t d : shape) n *= d;
  return n;
}

bool ModelConfig::Validate(std::string* error) const {
  auto fail = [error](const char* m) {
    if (error != nullptr) *error = m;
    return false;
  };
  if (num_layers <= 0 || num_heads <= 0 || num_kv_heads <= 0 || hidden_dim <= 0 || seq_len <= 0 || vocab_size <= 0 ||
      padded_vocab_size <= 0)
    return fail("model dimensions and vocabulary sizes must be positive");
  if (hidden_dim < 24) return fail("hidden_dim must be at least 24 for the smear and value gates");
  if (hidden_dim % num_heads != 0) return fail("hidden_dim must be divisible by num_heads");
  if (num_heads % num_kv_heads != 0) return fail("num_heads must be divisible by num_kv_heads");
  if ((hidden_dim / num_heads) % 2 != 0) return fail("head_dim must be even for rotary embeddings");
  if (padded_vocab_size < vocab_size) return fail("padded_vocab_size must be >= vocab_size");
  if (!(rope_base > 0.0f) || !std::isfinite(rope_base)) return fail("rope_base must be finite and positive");
  for (char k : window_pattern)
    if (k != 'S' && k != 'L') return fail("window_pattern can contain only 'S' and 'L'");
  return true;
}

// ------------------------------------------------------------------ metadata
std::vector<std::uint32_t> CheckpointMetadata::Write() const {
  WordWriter w;
  w.U32(schema);
  w.U32(stage);
  w.U64(step);
  w.U32(world_size);
  w.U32(precision);
  {
    const std::size_t at = w.BeginBlock();
    w.I32(config.num_layers), w.I32(config.num_heads), w.I32(config.num_kv_heads), w.I32(config.hidden_dim);
    w.I32(config.seq_len), w.I32(config.vocab_size), w.I32(config.padded_vocab_size);
    w.F32(config.rope_base);
    w.Str(config.window_pattern);
    w.U32(config.value_embedding ? 1 : 0);
    w.EndBlock(at);
  }
  w.Str(tokenizer_id), w.Str(git_revision), w.Str(created_utc);
  if (notes.size() > kMaxVectorEntries) return {};
  w.U32(static_cast<std::uint32_t>(notes.size()));
  for (const std::string& n : notes) w.Str(n);
  {
    const std::size_t at = w.BeginBlock();
    const Recipe& r = recipe;
    w.I32(r.device_batch_size), w.I32(r.total_batch_size);
    w.F32(r.embedding_lr), w.F32(r.unembedding_lr), w.F32(r.matrix_lr), w.F32(r.scalar_lr), w.F32(r.adam_eps);
    w.F32(r.init_lr_frac), w.F32(r.warmup_ratio), w.F32(r.warmdown_ratio), w.F32(r.final_lr_frac);
    w.F32(r.muon_momentum_steps), w.F32(r.muon_momentum_start), w.F32(r.muon_momentum_peak);
    w.F32(r.muon_momentum_final);
    w.I32(r.mmlu_epochs), w.I32(r.gsm8k_epochs);
    w.EndBlock(at);
  }
  if (!w.ok()) return {};
  return w.Take();
}

bool CheckpointMetadata::Read(const std::vector<std::uint32_t>& words, std::uint32_t* extra_words,
                              std::string* error) {
  WordReader r(words, 0, words.size());
  std::uint32_t extra = 0;
  bool more = r.U32(&schema) && r.U32(&stage) && r.U64(&step) && r.U32(&world_size) && r.U32(&precision);
  if (more && (stage > 2 || precision > 2)) return Fail(error, "invalid enum in checkpoint metadata");
  if (more) {
    WordReader c(words, 0, 0);
    more = r.Block(&c);
    if (more) {
      std::uint32_t ve = config.value_embedding ? 1 : 0;
      (void)(c.I32(&config.num_layers) && c.I32(&config.num_heads) && c.I32(&config.num_kv_heads) &&
             c.I32(&config.hidden_dim) && c.I32(&config.seq_len) && c.I32(&config.vocab_size) &&
             c.I32(&config.padded_vocab_size) && c.F32(&config.rope_base) && c.Str(&config.window_pattern) &&
             c.U32(&ve));
      if (c.bad() || ve > 1) return Fail(error, "invalid config block in checkpoint metadata");
      config.value_embedding = ve == 1;
      extra += static_cast<std::uint32_t>(c.Remaining());
    }
  }
  more = more && r.Str(&tokenizer_id) && r.Str(&git_revision) && r.Str(&created_utc);
  if (more) {
    std::uint32_t n = 0;
    more = r.U32(&n);
    if (more) {
      if (n > kMaxVectorEntries) return Fail(error, "notes vector too long in checkpoint metadata");
      notes.assign(n, std::string());
      for (std::uint32_t i = 0; i < n && more; ++i) more = r.Str(&notes[i]);
    }
  }
  if (more) {
    WordReader c(words, 0, 0);
    more = r.Block(&c);
    if (more) {
      Recipe& q = recipe;
      (void)(c.I32(&q.device_batch_size) && c.I32(&q.total_batch_size) && c.F32(&q.embedding_lr) &&
             c.F32(&q.unembedding_lr) && c.F32(&q.matrix_lr) && c.F32(&q.scalar_lr) && c.F32(&q.adam_eps) &&
             c.F32(&q.init_lr_frac) && c.F32(&q.warmup_ratio) && c.F32(&q.warmdown_ratio) &&
             c.F32(&q.final_lr_frac) && c.F32(&q.muon_momentum_steps) && c.F32(&q.muon_momentum_start) &&
             c.F32(&q.muon_momentum_peak) && c.F32(&q.muon_momentum_final) && c.I32(&q.mmlu_epochs) &&
             c.I32(&q.gsm8k_epochs));
      if (c.bad()) return Fail(error, "invalid recipe block in checkpoint metadata");
      extra += static_cast<std::uint32_t>(c.Remaining());
    }
  }
  if (r.bad()) return Fail(error, "invalid checkpoint metadata");
  extra += static_cast<std::uint32_t>(r.Remaining());
  if (extra_words != nullptr) *extra_words = extra;
  return true;
}

// ------------------------------------------------------------------ checkpoint container
namespace {

constexpr char kCkptMagic[8] = {'N', 'C', 'H', 'K', 'P', 'T', '0', '1'};

void WriteNameDTypeShape(std::ostream& out, const std::string& name, DType dtype,
                         const std::vector<std::int64_t>& shape) {
  const std::size_t n = std::min<std::size_t>(name.size(), 0xffffu);
  Put<std::uint16_t>(out, static_cast<std::uint16_t>(n));
  out.write(name.data(), static_cast<std::streamsize>(n));
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(dtype));
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(shape.size()));
  for (std::int64_t d : shape) Put<std::int64_t>(out, d);
}
void WritePayload(std::ostream& out, const std::vector<std::uint8_t>& data) {
  Put<std::uint64_t>(out, data.size());
  if (!data.empty()) out.write(reinterpret_cast<const char*>(data.data()), static_cast<std::streamsize>(data.size()));
}
void WriteRecord(std::ostream& out, const TensorRecord& r) {
  WriteNameDTypeShape(out, r.name, r.dtype, r.shape);
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(r.attributes.size()));
  for (const TensorAttribute& a : r.attributes) {
    WriteNameDTypeShape(out, a.name, a.dtype, a.shape);
    WritePayload(out, a.data);
  }
  WritePayload(out, r.data);
}

bool ReadNameDTypeShape(Reader& in, std::string* name, DType* dtype, std::vector<std::int64_t>* shape) {
  std::uint16_t n = 0;
  if (!in.Get(&n)) return false;
  name->assign(n, '\0');
  if (!in.Bytes(name->data(), n)) return false;
  std::uint32_t dt = 0, rank = 0;
  if (!in.Get(&dt) || !in.Get(&rank) || rank > 16) return false;
  *dtype = static_cast<DType>(dt);
  shape->resize(rank);
  for (std::uint32_t i = 0; i < rank; ++i)
    if (!in.Get(&(*shape)[i]) || (*shape)[i] < 0) return false;
  return true;
}
bool ReadPayload(Reader& in, std::vector<std::uint8_t>* data) {
  std::uint64_t n = 0;
  if (!in.Get(&n) || n > (1ull << 40)) return false;
  data->resize(n);
  return in.Bytes(data->data(), n);
}
bool ReadRecord(Reader& in, TensorRecord* r) {
  if (!ReadNameDTypeShape(in, &r->name, &r->dtype, &r->shape)) return false;
  std::uint32_t na = 0;
  if (!in.Get(&na) || na > 4096) return false;
  r->attributes.resize(na);
  for (TensorAttribute& a : r->attributes) {
    if (!ReadNameDTypeShape(in, &a.name, &a.dtype, &a.shape) || !ReadPayload(in, &a.data)) return false;
  }
  if (!ReadPayload(in, &r->data)) return false;
  return static_cast<std::uint64_t>(r->NumElements()) * DTypeSize(r->dtype) == r->data.size();
}

}  // namespace

bool Checkpoint::Save(const std::string& path, std::string* error) const {
  const std::vector<std::uint32_t> words = metadata.Write();
  if (words.empty() || words.size() > kMaxBlockWords) return Fail(error, "checkpoint metadata cannot be written");
  std::string cfg_err;
  if (!metadata.config.Validate(&cfg_err)) return Fail(error, "checkpoint metadata config is invalid (" + cfg_err + ")");
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) return Fail(error, "cannot open " + path);
  out.write(kCkptMagic, 8);
  Put<std::uint32_t>(out, 1);
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(words.size()));
  for (std::uint32_t w : words) Put<std::uint32_t>(out, w);
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(tensors.size()));
  for (const TensorRecord& r : tensors) WriteRecord(out, r);
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(optimizer_state.size()));
  for (const TensorRecord& r : optimizer_state) WriteRecord(out, r);
  return static_cast<bool>(out) ? true : Fail(error, "write failed: " + path);
}

bool Checkpoint::Load(const std::string& path, bool with_optimizer_state, std::string* error) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return Fail(error, "cannot open " + path);
  Reader in(f);
  char magic[8];
  if (!in.Bytes(magic, 8)) return Fail(error, "truncated checkpoint header: " + path);
  if (std::memcmp(magic, kCkptMagic, 8) != 0) return Fail(error, "not an NCHKPT01 container: " + path);
  std::uint32_t ver = 0;
  if (!in.Get(&ver) || ver > 1) return Fail(error, "unsupported checkpoint version: " + path);
  version = ver;
  CheckpointMetadata md;
  if (ver == 1) {
    std::uint32_t nwords = 0;
    if (!in.Get(&nwords)) return Fail(error, "truncated checkpoint metadata header: " + path);
    if (nwords == 0) return Fail(error, "checkpoint metadata section is empty: " + path);
    if (nwords > kMaxBlockWords) return Fail(error, "checkpoint metadata section is too large: " + path);
    std::vector<std::uint32_t> words(nwords);
    for (std::uint32_t& w : words)
      if (!in.Get(&w)) return Fail(error, "truncated checkpoint metadata: " + path);
    std::uint32_t extra = 0;
    std::string why;
    if (!md.Read(words, &extra, &why)) return Fail(error, why + ": " + path);
    if (extra != 0)
      std::fprintf(stderr, "checkpoint: warning: %s carries %u metadata word(s) this build does not know; loading anyway\n",
                   path.c_str(), extra);
    std::string cfg_err;
    if (!md.config.Validate(&cfg_err)) return Fail(error, "checkpoint metadata config is invalid (" + cfg_err + "): " + path);
  }
  std::uint32_t count = 0;
  if (!in.Get(&count)) return Fail(error, "truncated checkpoint header: " + path);
  std::vector<TensorRecord> recs(count);
  for (TensorRecord& r : recs)
    if (!ReadRecord(in, &r)) return Fail(error, "checkpoint record is malformed: " + path);
  std::vector<TensorRecord> opt;
  if (with_optimizer_state && !in.AtEnd()) {
    std::uint32_t n = 0;
    if (!in.Get(&n)) return Fail(error, "truncated checkpoint optimizer-state header: " + path);
    opt.resize(n);
    for (TensorRecord& r : opt)
      if (!ReadRecord(in, &r)) return Fail(error, "checkpoint optimizer state is malformed: " + path);
  }
  tensors = std::move(recs);
  optimizer_state = std::move(opt);
  metadata = std::move(md);
  return true;
}

const TensorRecord* Checkpoint::Find(std::string_view name) const {
  for (const TensorRecord& r : tensors)
    if (r.name == name) return &r;
  return nullptr;
}

// ------------------------------------------------------------------ fixture record container
bool ReadRecordFile(const std::string& path, std::string* magic, std::vector<FixtureRecord>* records,
                    std::string* error) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return Fail(error, "cannot open " + path);
  Reader in(f);
  char m[8];
  std::uint32_t ver = 0, count = 0;
  if (!in.Bytes(m, 8) || !in.Get(&ver) || !in.Get(&count) || ver != 1) return Fail(error, "bad record file header: " + path);
  if (magic != nullptr) magic->assign(m, 8);
  static const std::size_t kSize[5] = {4, 4, 8, 8, 1};
  records->clear();
  records->resize(count);
  for (FixtureRecord& r : *records) {
    std::uint16_t n = 0;
    if (!in.Get(&n)) return Fail(error, "truncated record: " + path);
    r.name.assign(n, '\0');
    std::uint8_t rank = 0;
    if (!in.Bytes(r.name.data(), n) || !in.Get(&r.dtype) || !in.Get(&rank) || r.dtype > 4)
      return Fail(error, "truncated record: " + path);
    r.dims.resize(rank);
    std::uint64_t elems = 1;
    for (std::uint64_t& d : r.dims) {
      if (!in.Get(&d)) return Fail(error, "truncated record: " + path);
      elems *= d;
    }
    r.data.resize(elems * kSize[r.dtype]);
    if (!in.Bytes(r.data.data(), r.data.size())) return Fail(error, "truncated record payload: " + path);
  }
  return true;
}

bool WriteRecordFile(const std::string& path, const std::string& magic, const std::vector<FixtureRecord>& records) {
  if (magic.size() != 8) return false;
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) return false;
  out.write(magic.data(), 8);
  Put<std::uint32_t>(out, 1);
  Put<std::uint32_t>(out, static_cast<std::uint32_t>(records.size()));
  for (const FixtureRecord& r : records) {
    Put<std::uint16_t>(out, static_cast<std::uint16_t>(r.name.size()));
    out.write(r.name.data(), static_cast<std::streamsize>(r.name.size()));
    Put<std::uint8_t>(out, r.dtype);
    Put<std::uint8_t>(out, static_cast<std::uint8_t>(r.dims.size()));
    for (std::uint64_t d : r.dims) Put<std::uint64_t>(out, d);
    out.write(reinterpret_cast<const char*>(r.data.data()), static_cast<std::streamsize>(r.data.size()));
  }
  return static_cast<bool>(out);
}

// ------------------------------------------------------------------ data cursor sidecar
bool SaveCursor(const std::string& path, const LoaderState& s) {
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) return false;
  Put<std::uint64_t>(out, s.epoch);
  Put<std::uint64_t>(out, s.position);
  Put<std::uint64_t>(out, s.buffered.size());
  for (const std::vector<int>& d : s.buffered) {
    Put<std::uint64_t>(out, d.size());
    for (int t : d) Put<std::uint64_t>(out, static_cast<std::uint64_t>(static_cast<std::int64_t>(t)));
  }
  return static_cast<bool>(out);
}
bool LoadCursor(const std::string& path, LoaderState* s) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  Reader in(f);
  std::uint64_t n = 0;
  if (!in.Get(&s->epoch) || !in.Get(&s->position) || !in.Get(&n) || n > (1u << 24)) return false;
  s->buffered.assign(n, {});
  for (std::vector<int>& d : s->buffered) {
    std::uint64_t len = 0;
    if (!in.Get(&len) || len > (1u << 28)) return false;
    d.resize(len);
    for (int& t : d) {
      std::uint64_t v = 0;
      if (!in.Get(&v)) return false;
      t = static_cast<int>(static_cast<std::int64_t>(v));
    }
  }
  return true;
}

}  // namespace ncb
