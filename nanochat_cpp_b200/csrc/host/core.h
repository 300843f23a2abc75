// Host runtime: formats, tokenizer, BPE trainer, data loader, parquet reader, samplers.
// Plain C++20, no CUDA and no PyTorch: the training and inference engines call it through the C ABI
// in capi.cc (ctypes from Python, or directly from C/C++).
//
// Formats follow the reference byte for byte so artefacts are interchangeable:
//   record container  - reference src/record_file.h
//   NCHKPT01          - reference src/data.cc:105-455, metadata words src/fields.cc
//   NCTOKEN1          - reference src/tokenizer/tokenizer.cc:196-300
//   data cursor       - reference src/data_cursor.cc
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace ncb {

// ------------------------------------------------------------------ random numbers
// xoshiro256** seeded through splitmix64 (the generator family of reference include/nanochat/rand.h).
class Rng {
 public:
  explicit Rng(std::uint64_t seed = 0);
  std::uint64_t NextU64();
  double NextDouble();  // [0, 1)
  float NextFloat() { return static_cast<float>(NextDouble()); }
  std::uint64_t NextBelow(std::uint64_t n);
  double NextNormal();

 private:
  std::uint64_t s_[4];
  bool have_spare_ = false;
  double spare_ = 0.0;
};
std::uint64_t MixSeed(std::uint64_t seed, std::uint64_t stream);

// ------------------------------------------------------------------ tensors in files
// dtype codes of the checkpoint container (reference include/nanochat/tensor.h:179-185)
enum class DType : std::uint32_t { kFp32 = 0, kBf16 = 1, kInt8 = 2, kFp8E4M3 = 4, kFp8E5M2 = 5 };
std::size_t DTypeSize(DType t);
std::uint16_t FloatToBf16(float v);  // round to nearest even
float Bf16ToFloat(std::uint16_t v);
// fp8 codecs (fp8.cc): saturating round-to-nearest-even; E4M3 max 448 (no infinities), E5M2 max 57344
std::uint8_t FloatToE4M3(float v);
float E4M3ToFloat(std::uint8_t c);
std::uint8_t FloatToE5M2(float v);
float E5M2ToFloat(std::uint8_t c);

struct TensorAttribute {
  std::string name;
  DType dtype = DType::kFp32;
  std::vector<std::int64_t> shape;
  std::vector<std::uint8_t> data;
};
struct TensorRecord {
  std::string name;
  DType dtype = DType::kFp32;
  std::vector<std::int64_t> shape;
  std::vector<TensorAttribute> attributes;
  std::vector<std::uint8_t> data;
  std::int64_t NumElements() const;
};

// ------------------------------------------------------------------ checkpoint metadata
struct ModelConfig {
  std::int32_t num_layers = 12, num_heads = 6, num_kv_heads = 6, hidden_dim = 768, seq_len = 2048;
  std::int32_t vocab_size = 32768, padded_vocab_size = 32768;
  float rope_base = 100000.0f;
  std::string window_pattern = "SSSL";
  bool value_embedding = true;
  bool Validate(std::string* error) const;
};
struct Recipe {
  std::int32_t device_batch_size = 0, total_batch_size = 0;
  float embedding_lr = 0.2f, unembedding_lr = 0.004f, matrix_lr = 0.02f, scalar_lr = 0.5f, adam_eps = 1e-10f;
  float init_lr_frac = 1.0f, warmup_ratio = 0.0f, warmdown_ratio = 0.65f, final_lr_frac = 0.0f;
  float muon_momentum_steps = 400.0f, muon_momentum_start = 0.85f, muon_momentum_peak = 0.97f,
        muon_momentum_final = 0.90f;
  std::int32_t mmlu_epochs = 3, gsm8k_epochs = 4;
};
struct CheckpointMetadata {
  std::uint32_t schema = 1;
  std::uint32_t stage = 0;  // 0 base, 1 sft, 2 rl
  std::uint64_t step = 0;
  std::uint32_t world_size = 1;
  std::uint32_t precision = 0;  // 0 fp32, 1 bf16, 2 fp8
  ModelConfig config;
  std::string tokenizer_id, git_revision, created_utc;
  std::vector<std::string> notes;
  Recipe recipe;
  // Word stream (u32/i32/float one word; u64 low word first; string = length word + padded bytes;
  // vector = count word; nested block = size word + payload).
  std::vector<std::uint32_t> Write() const;
  // Returns false on an invalid stream. Shorter streams keep defaults; `extra_words` counts words this
  // build does not know (a newer writer).
  bool Read(const std::vector<std::uint32_t>& words, std::uint32_t* extra_words, std::string* error);
};

class Checkpoint {
 public:
  std::vector<TensorRecord> tensors;
  std::vector<TensorRecord> optimizer_state;
  CheckpointMetadata metadata;
  std::uint32_t version = 1;

  bool Save(const std::string& path, std::string* error = nullptr) const;  // always writes version 1
  bool Load(const std::string& path, bool with_optimizer_state, std::string* error = nullptr);
  const TensorRecord* Find(std::string_view name) const;
};

// Fixture record container (magic[8], u32 version = 1, u32 count, records).
struct FixtureRecord {
  std::string name;
  std::uint8_t dtype = 0;  // 0 f32, 1 i32, 2 f64, 3 i64, 4 u8
  std::vector<std::uint64_t> dims;
  std::vector<std::uint8_t> data;
};
bool ReadRecordFile(const std::string& path, std::string* magic, std::vector<FixtureRecord>* records,
                    std::string* error = nullptr);
bool WriteRecordFile(const std::string& path, const std::string& magic, const std::vector<FixtureRecord>& records);

// ------------------------------------------------------------------ tokenizer
std::string NanochatSplitPattern();
std::vector<std::string_view> SplitPattern(std::string_view text);
bool IsUnicodeLetter(std::uint32_t cp);
bool IsUnicodeNumber(std::uint32_t cp);
bool IsUnicodeWhitespace(std::uint32_t cp);

class Tokenizer {
 public:
  // merges[i] = (left, right) creates id 256 + i; specials are (name, id)
  Tokenizer(std::vector<std::pair<std::uint32_t, std::uint32_t>> merges,
            std::vector<std::pair<std::string, std::uint32_t>> specials);
  static std::unique_ptr<Tokenizer> Load(const std::string& path, std::string* error = nullptr);
  bool Save(const std::string& path) const;

  int vocab_size() const { return vocab_size_; }
  int bos_id() const { return SpecialId("<|bos|>"); }
  int SpecialId(std::string_view name) const;
  bool IsSpecial(int id) const;
  std::vector<int> Encode(std::string_view text, int prepend = -1, int append = -1) const;
  std::string Decode(const int* ids, int count) const;  // lossy UTF-8 ("replace")
  bool AppendTokenBytes(int id, std::string* out) const;
  const std::vector<std::uint8_t>& TokenBytes() const { return token_bytes_; }
  const std::vector<std::pair<std::uint32_t, std::uint32_t>>& merges() const { return merges_; }

 private:
  void EncodePiece(std::string_view piece, std::vector<int>* out) const;
  std::vector<std::pair<std::uint32_t, std::uint32_t>> merges_;
  std::vector<std::pair<std::string, std::uint32_t>> specials_;
  std::map<std::uint64_t, std::uint32_t> rank_;  // (left << 32 | right) -> merge index
  std::unordered_map<std::string, std::uint32_t> by_bytes_;  // token bytes -> id (first id wins)
  std::vector<std::string> bytes_of_;            // raw bytes of every ordinary id
  std::vector<std::uint8_t> token_bytes_;
  int vocab_size_ = 0;
};

std::string SanitizeUtf8(std::string_view bytes);  // invalid sequences -> U+FFFD

// The nine chat specials in id order (reference src/tokenizer/tok_train_main.cc:32-37).
const std::vector<std::string>& DefaultSpecialTokens();

struct BpeTrainerConfig {
  int vocab_size = 32768;       // including the specials
  std::int64_t doc_cap = 0;     // bytes per document, 0 = unlimited
  std::int64_t max_chars = 0;   // total bytes, 0 = unlimited
};
// Trains byte-level BPE merges (most frequent pair first, ties to the smaller pair).
std::unique_ptr<Tokenizer> TrainBpe(const std::function<bool(std::string*)>& next_document,
                                    const BpeTrainerConfig& config);

// ------------------------------------------------------------------ data loading
class DocumentSource {
 public:
  virtual ~DocumentSource() = default;
  virtual bool Next(std::vector<int>* tokens) = 0;  // false at end of an epoch (the source then rewinds)
  virtual void Reset() = 0;                         // back to the first document of an epoch
};
// Every `world`-th document starting at `rank` of an underlying source.
std::unique_ptr<DocumentSource> ShardSource(std::unique_ptr<DocumentSource> inner, int rank, int world);
std::unique_ptr<DocumentSource> VectorSource(std::vector<std::vector<int>> docs);
// Zipf(s) ids over [1, vocab) in documents of `doc_len` tokens (benchmark data).
std::unique_ptr<DocumentSource> ZipfSource(int vocab, int doc_len, double s, std::uint64_t seed);
// Text documents (one per line, or parquet rows) tokenised on the fly with BOS prepended.
std::unique_ptr<DocumentSource> TextFileSource(const std::string& path, const Tokenizer* tok);
std::unique_ptr<DocumentSource> ParquetSource(const std::string& path, const std::string& column,
                                              const Tokenizer* tok, std::string* error);

struct LoaderState {
  std::uint64_t epoch = 0, position = 0;
  std::vector<std::vector<int>> buffered;
};

// BOS-aligned best-fit packing (reference src/data.cc:486-748): every row has capacity seq + 1; the largest
// buffered document that fits goes next, and when nothing fits the shortest document is cropped to fill the
// row. Inputs are row[:-1], targets row[1:]. A producer thread keeps `prefetch` batches ready.
class DataLoader {
 public:
  // `source_batch`: documents are pulled from the source in groups of this size whenever fewer than
  // `buffer_docs` are buffered (the upstream loader refills with whole tokenizer batches).
  DataLoader(std::unique_ptr<DocumentSource> source, int batch, int seq, int buffer_docs, int prefetch = 2,
             int source_batch = 1);
  ~DataLoader();
  void Next(int* tokens, int* targets);  // [batch, seq] each
  LoaderState State() const;
  void Restore(const LoaderState& state);
  std::uint64_t epoch() const;

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};
bool SaveCursor(const std::string& path, const LoaderState& state);
bool LoadCursor(const std::string& path, LoaderState* state);

// ------------------------------------------------------------------ parquet
// One OPTIONAL/REQUIRED BYTE_ARRAY column, DATA_PAGE v1, PLAIN encoding, RLE definition levels,
// UNCOMPRESSED pages (ZSTD pages when libzstd can be loaded at run time).
bool ReadParquetStrings(const std::string& path, const std::string& column, std::vector<std::string>* out,
                        std::string* error);

// ------------------------------------------------------------------ sampling
// Temperature / top-k sampling of one row of logits (reference src/generate.cc:614-669). temperature <= 0: argmax.
int SampleToken(const float* logits, int vocab, float temperature, int top_k, Rng* rng);

}  // namespace ncb
