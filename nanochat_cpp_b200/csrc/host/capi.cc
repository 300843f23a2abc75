// C ABI, part 1: process-level calls, tokenizer, loader, checkpoint container, parquet, sampling.
// Error convention of the reference (spec/api-surface.md:72-75): a status code (or a null / negative
// result) plus a thread-local message readable through nanochat_last_error().
#include <cstring>
#include <sstream>

#include <dlfcn.h>

#include <cstdlib>

#include "capi_internal.h"

namespace {
thread_local std::string g_last_error;
}

void ncb_set_error(const std::string& msg) { g_last_error = msg; }

// ---- the GPU engine library, opened on demand ---------------------------------------------------------------------
namespace {
ncb_gpu_library g_gpu;
bool g_gpu_tried = false;
int g_cuda_device = -2;   // -2: not decided yet (NANOCHAT_DEVICE is read on first use), -1: cpu, >= 0: CUDA ordinal
std::string g_gpu_error;

std::string OwnDirectory() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&ncb_set_error), &info) == 0 || info.dli_fname == nullptr) return ".";
  std::string path = info.dli_fname;
  const std::size_t slash = path.rfind('/');
  return slash == std::string::npos ? "." : path.substr(0, slash);
}
}  // namespace

const ncb_gpu_library* ncb_gpu() {
  if (!g_gpu_tried) {
    g_gpu_tried = true;
    const std::string path = OwnDirectory() + "/libnanochat_gpu.so";
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) {
      g_gpu_error = std::string("cannot open ") + path + ": " + dlerror();
    } else {
      g_gpu.device_count = reinterpret_cast<ncb::ncb_gpu_device_count_fn>(dlsym(h, "ncb_gpu_device_count"));
      g_gpu.device_at = reinterpret_cast<ncb::ncb_gpu_device_at_fn>(dlsym(h, "ncb_gpu_device_at"));
      g_gpu.create = reinterpret_cast<ncb::ncb_gpu_engine_create_fn>(dlsym(h, "ncb_gpu_engine_create"));
      if (g_gpu.device_count == nullptr || g_gpu.device_at == nullptr || g_gpu.create == nullptr) {
        g_gpu_error = path + " lacks the engine entry points";
        g_gpu = ncb_gpu_library();
      }
    }
  }
  return g_gpu.create != nullptr ? &g_gpu : nullptr;
}

bool ncb_select_device(const std::string& name, std::string* error) {
  if (name.empty() || name == "cpu") {
    g_cuda_device = -1;
    return true;
  }
  if (name.rfind("cuda", 0) != 0) {
    *error = "unknown device '" + name + "' (cpu, cuda, cuda:N)";
    return false;
  }
  int index = 0;
  if (name.size() > 4) {
    if (name[4] != ':' || name.size() == 5) {
      *error = "unknown device '" + name + "' (cpu, cuda, cuda:N)";
      return false;
    }
    index = std::atoi(name.c_str() + 5);
  }
  const ncb_gpu_library* lib = ncb_gpu();
  if (lib == nullptr) {
    *error = g_gpu_error.empty() ? "the GPU engine library is not available" : g_gpu_error;
    return false;
  }
  const int n = lib->device_count();
  if (index < 0 || index >= n) {
    *error = "CUDA device " + std::to_string(index) + " does not exist (" + std::to_string(n) + " visible)";
    return false;
  }
  g_cuda_device = index;
  return true;
}

int ncb_selected_cuda_device() {
  if (g_cuda_device == -2) {
    g_cuda_device = -1;
    const char* env = std::getenv("NANOCHAT_DEVICE");
    if (env != nullptr && *env) {
      std::string err;
      if (!ncb_select_device(env, &err)) ncb_set_error("NANOCHAT_DEVICE: " + err);
    }
  }
  return g_cuda_device;
}

extern "C" {

size_t nanochat_optim_config_size(void) { return sizeof(nanochat_optim_config); }
nanochat_status nanochat_init(void) { return NANOCHAT_STATUS_OK; }
const char* nanochat_last_error(void) { return g_last_error.c_str(); }
const char* nanochat_version(void) { return "nanochat-b200 0.1.0"; }
const char* nanochat_backend(void) { return ncb_selected_cuda_device() >= 0 ? "cuda" : "cpu"; }
int nanochat_compute_type_size(void) { return ncb_selected_cuda_device() >= 0 ? 2 : 4; }
void nanochat_device_info(nanochat_device* out) { nanochat_device_at(0, out); }

// Device selection. The reference fixes its backend at link time; here one library serves both, so the backend is
// a run-time choice: "cpu" (the default), "cuda" or "cuda:N". The environment variable NANOCHAT_DEVICE gives the
// initial choice. Selecting a CUDA device opens libnanochat_gpu.so (beside this library); models created afterwards
// live on that device.
nanochat_status nanochat_select_device(const char* name) {
  std::string err;
  if (!ncb_select_device(name != nullptr ? name : "cpu", &err)) {
    ncb_set_error("nanochat_select_device: " + err);
    return NANOCHAT_STATUS_ERROR;
  }
  return NANOCHAT_STATUS_OK;
}
int nanochat_device_count(void) {
  if (ncb_selected_cuda_device() < 0) return 1;
  const ncb_gpu_library* lib = ncb_gpu();
  return lib != nullptr ? lib->device_count() : 0;
}
int nanochat_device_at(int ordinal, nanochat_device* out) {
  if (out == nullptr) return 0;
  if (ncb_selected_cuda_device() < 0) {
    if (ordinal != 0) return 0;
    out->device_index = 0;
    out->compute_major = 0;
    out->compute_minor = 0;
    out->total_memory_bytes = 0;
    out->device_name = "cpu";
    return 1;
  }
  const ncb_gpu_library* lib = ncb_gpu();
  static thread_local ncb::DeviceDescription d;
  if (lib == nullptr || !lib->device_at(ordinal, &d)) return 0;
  out->device_index = d.index;
  out->compute_major = d.compute_major;
  out->compute_minor = d.compute_minor;
  out->total_memory_bytes = static_cast<uint64_t>(d.total_memory_bytes);
  out->device_name = d.name;
  return 1;
}

nanochat_status nanochat_optim_config_preset(const char* name, nanochat_optim_config* out) {
  if (out == nullptr) return NANOCHAT_STATUS_ERROR;
  nanochat_optim_config c;
  c.unembedding_lr = 0.004f, c.embedding_lr = 0.2f, c.matrix_lr = 0.02f, c.scalar_lr = 0.5f, c.weight_decay = 0.0f;
  c.muon_ns_steps = 5, c.muon_beta2 = 0.9f, c.adam_eps = 1e-10f, c.clip = 1.0f;
  c.num_iterations = 0, c.warmup_steps = 0, c.warmdown_ratio = 0.65f, c.final_lr_frac = 0.0f, c.weight_decay_base = 0.0f;
  c.muon_momentum_warmup_steps = 400.0f, c.muon_momentum_start = 0.85f, c.muon_momentum_peak = 0.97f;
  c.muon_momentum_final = 0.90f;
  const std::string n = name != nullptr ? name : "default";
  if (n == "track3") {
    // reference src/train.cc:442-473: the Track 3 baseline trains without clipping and with decay 0.28
    c.clip = 0.0f;
    c.weight_decay_base = 0.28f;
    c.warmdown_ratio = 0.5f;
  } else if (n == "sft") {
    // supervised fine-tuning (reference src/sft_command.cc; python/nanochat_cpp/sft.py): higher embedding rate, no
    // clipping, half of the run in warm-down, momentum 0.85 -> 0.95 over 300 steps and held
    c.embedding_lr = 0.3f;
    c.clip = 0.0f;
    c.warmdown_ratio = 0.5f;
    c.muon_momentum_warmup_steps = 300.0f, c.muon_momentum_start = 0.85f, c.muon_momentum_peak = 0.95f;
    c.muon_momentum_final = 0.95f;
  } else if (n != "default" && !n.empty()) {
    ncb_set_error("unknown optimizer preset '" + n + "'");
    return NANOCHAT_STATUS_ERROR;
  }
  *out = c;
  return NANOCHAT_STATUS_OK;
}

// ------------------------------------------------------------------ tokenizer
nanochat_tokenizer* nanochat_tokenizer_load(const char* path) {
  std::string err;
  auto tok = ncb::Tokenizer::Load(path != nullptr ? path : "", &err);
  if (!tok) {
    ncb_set_error(err);
    return nullptr;
  }
  auto* h = new nanochat_tokenizer;
  h->tok = std::move(tok);
  return h;
}
void nanochat_tokenizer_free(nanochat_tokenizer* t) { delete t; }
int nanochat_encode(nanochat_tokenizer* t, const char* text, int* out, int capacity) {
  return ncb_encode_n(t, text, text != nullptr ? static_cast<int64_t>(std::strlen(text)) : 0, -1, -1, out, capacity);
}
int ncb_encode_n(nanochat_tokenizer* t, const char* text, int64_t length, int prepend, int append, int* out,
                 int capacity) {
  if (t == nullptr || text == nullptr) return -1;
  const std::vector<int> ids = t->tok->Encode(std::string_view(text, static_cast<size_t>(length)), prepend, append);
  const int n = static_cast<int>(ids.size());
  if (out != nullptr) std::memcpy(out, ids.data(), sizeof(int) * static_cast<size_t>(std::min(n, capacity)));
  return n;  // the full count, so a caller can size a second call
}
int nanochat_decode(nanochat_tokenizer* t, const int* ids, int count, char* out, int capacity) {
  if (t == nullptr || ids == nullptr) return -1;
  const std::string s = t->tok->Decode(ids, count);
  const int n = static_cast<int>(s.size());
  if (out != nullptr && capacity > 0) {
    const int m = std::min(n, capacity - 1);
    std::memcpy(out, s.data(), static_cast<size_t>(m));
    out[m] = '\0';
  }
  return n;
}
int ncb_tokenizer_vocab_size(nanochat_tokenizer* t) { return t != nullptr ? t->tok->vocab_size() : -1; }
int ncb_tokenizer_special_id(nanochat_tokenizer* t, const char* name) {
  return t != nullptr && name != nullptr ? t->tok->SpecialId(name) : -1;
}
nanochat_status ncb_tokenizer_save(nanochat_tokenizer* t, const char* path) {
  return t != nullptr && path != nullptr && t->tok->Save(path) ? NANOCHAT_STATUS_OK : NANOCHAT_STATUS_ERROR;
}
nanochat_tokenizer* ncb_tokenizer_train(const char* text_path, const char* parquet_path, const char* text_column,
                                        int vocab_size, int64_t doc_cap, int64_t max_chars) {
  std::vector<std::string> docs;
  if (parquet_path != nullptr && parquet_path[0] != '\0') {
    std::string err;
    if (!ncb::ReadParquetStrings(parquet_path, text_column != nullptr ? text_column : "text", &docs, &err)) {
      ncb_set_error(err);
      return nullptr;
    }
  } else if (text_path != nullptr) {
    std::ifstream f(text_path);
    if (!f) {
      ncb_set_error(std::string("cannot open ") + text_path);
      return nullptr;
    }
    std::string line;
    while (std::getline(f, line)) docs.push_back(line + "\n");
  }
  size_t pos = 0;
  ncb::BpeTrainerConfig cfg;
  cfg.vocab_size = vocab_size;
  cfg.doc_cap = doc_cap;
  cfg.max_chars = max_chars;
  auto tok = ncb::TrainBpe(
      [&](std::string* d) {
        if (pos >= docs.size()) return false;
        *d = docs[pos++];
        return true;
      },
      cfg);
  auto* h = new nanochat_tokenizer;
  h->tok = std::move(tok);
  return h;
}
int ncb_split_pattern(const char* text, int64_t length, int64_t* ends, int capacity) {
  if (text == nullptr) return -1;
  const std::string_view view(text, static_cast<size_t>(length));
  const auto pieces = ncb::SplitPattern(view);
  int n = 0;
  for (const auto& p : pieces) {
    if (ends != nullptr && n < capacity) ends[n] = static_cast<int64_t>(p.data() - text) + static_cast<int64_t>(p.size());
    ++n;
  }
  return n;
}

// ------------------------------------------------------------------ loaders
static nanochat_loader* make_loader(std::unique_ptr<ncb::DocumentSource> src, nanochat_tokenizer* tok, int batch,
                                    int seq, size_t buffer, int rank, int world) {
  if (!src) return nullptr;
  if (world > 1) src = ncb::ShardSource(std::move(src), rank, world);
  auto* h = new nanochat_loader;
  h->tok = tok;
  h->batch = batch;
  h->seq = seq;
  int source_batch = 1;
  if (const char* sb = std::getenv("NANOCHAT_SOURCE_BATCH")) source_batch = std::max(1, std::atoi(sb));
  h->loader = std::make_unique<ncb::DataLoader>(std::move(src), batch, seq, static_cast<int>(buffer ? buffer : 1000), 2,
                                                source_batch);
  return h;
}
nanochat_loader* nanochat_loader_create(const char** parquet, int count, const char* text_column,
                                        nanochat_tokenizer* tokenizer, int batch, int seq, uint64_t /*seed*/,
                                        int /*tokenizer_threads*/, size_t document_buffer) {
  if (tokenizer == nullptr || parquet == nullptr || count <= 0) {
    ncb_set_error("loader needs a tokenizer and at least one parquet path");
    return nullptr;
  }
  std::vector<std::string> docs;
  for (int i = 0; i < count; ++i) {
    std::vector<std::string> part;
    std::string err;
    if (!ncb::ReadParquetStrings(parquet[i], text_column != nullptr ? text_column : "text", &part, &err)) {
      ncb_set_error(err);
      return nullptr;
    }
    docs.insert(docs.end(), std::make_move_iterator(part.begin()), std::make_move_iterator(part.end()));
  }
  std::vector<std::vector<int>> tokens;
  tokens.reserve(docs.size());
  for (const std::string& d : docs) tokens.push_back(tokenizer->tok->Encode(d, tokenizer->tok->bos_id()));
  int rank = 0, world = 1;
  if (const char* r = std::getenv("NANOCHAT_RANK")) rank = std::atoi(r);
  if (const char* w = std::getenv("NANOCHAT_WORLD_SIZE")) world = std::max(1, std::atoi(w));
  return make_loader(ncb::VectorSource(std::move(tokens)), tokenizer, batch, seq, document_buffer, rank, world);
}
nanochat_loader* ncb_loader_from_documents(const int* tokens, const int64_t* offsets, int64_t count, int batch,
                                           int seq, size_t document_buffer, int rank, int world) {
  std::vector<std::vector<int>> docs(static_cast<size_t>(count));
  for (int64_t i = 0; i < count; ++i) docs[i].assign(tokens + offsets[i], tokens + offsets[i + 1]);
  return make_loader(ncb::VectorSource(std::move(docs)), nullptr, batch, seq, document_buffer, rank, world);
}
nanochat_loader* ncb_loader_from_text(const char* path, nanochat_tokenizer* tokenizer, int batch, int seq,
                                      size_t document_buffer, int rank, int world) {
  if (tokenizer == nullptr || path == nullptr) return nullptr;
  return make_loader(ncb::TextFileSource(path, tokenizer->tok.get()), tokenizer, batch, seq, document_buffer, rank,
                     world);
}
nanochat_loader* ncb_loader_zipf(int vocab, int doc_len, double s, uint64_t seed, int batch, int seq,
                                 size_t document_buffer) {
  return make_loader(ncb::ZipfSource(vocab, doc_len, s, seed), nullptr, batch, seq, document_buffer, 0, 1);
}
int nanochat_loader_next(nanochat_loader* l, int* tokens, int* targets) {
  if (l == nullptr || tokens == nullptr || targets == nullptr) return 0;
  l->loader->Next(tokens, targets);
  return 1;
}
const uint8_t* nanochat_loader_token_bytes(nanochat_loader* l, int* vocab) {
  if (l == nullptr || l->tok == nullptr) return nullptr;
  if (vocab != nullptr) *vocab = l->tok->tok->vocab_size();
  return l->tok->tok->TokenBytes().data();
}
void nanochat_loader_free(nanochat_loader* l) { delete l; }
nanochat_status ncb_loader_save_cursor(nanochat_loader* l, const char* path) {
  return l != nullptr && ncb::SaveCursor(path, l->loader->State()) ? NANOCHAT_STATUS_OK : NANOCHAT_STATUS_ERROR;
}
nanochat_status ncb_loader_load_cursor(nanochat_loader* l, const char* path) {
  ncb::LoaderState s;
  if (l == nullptr || !ncb::LoadCursor(path, &s)) return NANOCHAT_STATUS_ERROR;
  l->loader->Restore(s);
  return NANOCHAT_STATUS_OK;
}
uint64_t ncb_loader_epoch(nanochat_loader* l) { return l != nullptr ? l->loader->epoch() : 0; }

// ------------------------------------------------------------------ checkpoints
nanochat_status nanochat_checkpoint_dtype(int32_t index, const char** name, int32_t* code, int32_t* size) {
  static const struct { const char* n; int32_t c, s; } k[] = {
      {"float32", 0, 4}, {"bfloat16", 1, 2}, {"int8", 2, 1}, {"float8_e4m3", 4, 1}, {"float8_e5m2", 5, 1}};
  if (index < 0 || index >= 5) return NANOCHAT_STATUS_ERROR;
  if (name != nullptr) *name = k[index].n;
  if (code != nullptr) *code = k[index].c;
  if (size != nullptr) *size = k[index].s;
  return NANOCHAT_STATUS_OK;
}

static void to_records(const nanochat_record* in, int64_t n, std::vector<ncb::TensorRecord>* out) {
  out->resize(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) {
    ncb::TensorRecord& r = (*out)[i];
    r.name = in[i].name != nullptr ? in[i].name : "";
    r.dtype = static_cast<ncb::DType>(in[i].dtype);
    r.shape.assign(in[i].dims, in[i].dims + in[i].ndim);
    r.data.assign(static_cast<const uint8_t*>(in[i].data), static_cast<const uint8_t*>(in[i].data) + in[i].bytes);
    for (int64_t a = 0; a < in[i].attribute_count; ++a) {
      const nanochat_record& ar = in[i].attributes[a];
      ncb::TensorAttribute at;
      at.name = ar.name != nullptr ? ar.name : "";
      at.dtype = static_cast<ncb::DType>(ar.dtype);
      at.shape.assign(ar.dims, ar.dims + ar.ndim);
      at.data.assign(static_cast<const uint8_t*>(ar.data), static_cast<const uint8_t*>(ar.data) + ar.bytes);
      r.attributes.push_back(std::move(at));
    }
  }
}

nanochat_status ncb_checkpoint_write_meta(const char* path, const nanochat_record* records, int64_t record_count,
                                          const nanochat_record* optimizer, int64_t optimizer_count,
                                          const nanochat_config* config, int32_t stage, int64_t step,
                                          int64_t world_size, int32_t precision, const char* tokenizer_id,
                                          const char* notes) {
  ncb::Checkpoint ck;
  to_records(records, record_count, &ck.tensors);
  to_records(optimizer, optimizer_count, &ck.optimizer_state);
  if (config != nullptr) ck.metadata.config = ncb_to_model_config(*config);
  ck.metadata.stage = static_cast<uint32_t>(stage);
  ck.metadata.step = static_cast<uint64_t>(step);
  ck.metadata.world_size = static_cast<uint32_t>(world_size);
  ck.metadata.precision = static_cast<uint32_t>(precision);
  if (tokenizer_id != nullptr) ck.metadata.tokenizer_id = tokenizer_id;
  if (notes != nullptr && notes[0] != '\0') ck.metadata.notes.push_back(notes);
  std::string err;
  if (!ck.Save(path, &err)) {
    ncb_set_error(err);
    return NANOCHAT_STATUS_ERROR;
  }
  return NANOCHAT_STATUS_OK;
}
nanochat_status nanochat_checkpoint_write(const char* path, const nanochat_record* records, int64_t record_count,
                                          const nanochat_record* optimizer, int64_t optimizer_count) {
  return ncb_checkpoint_write_meta(path, records, record_count, optimizer, optimizer_count, nullptr, 0, 0, 1, 0,
                                   nullptr, nullptr);
}

static void export_records(const std::vector<ncb::TensorRecord>& in, std::vector<nanochat_record>* out,
                           std::vector<std::vector<nanochat_record>>* attr_store) {
  out->resize(in.size());
  for (size_t i = 0; i < in.size(); ++i) {
    const ncb::TensorRecord& r = in[i];
    nanochat_record& o = (*out)[i];
    o.name = r.name.c_str();
    o.dtype = static_cast<int32_t>(r.dtype);
    o.ndim = static_cast<int32_t>(r.shape.size());
    o.dims = r.shape.data();
    o.data = r.data.data();
    o.bytes = static_cast<int64_t>(r.data.size());
    attr_store->emplace_back();
    for (const ncb::TensorAttribute& a : r.attributes) {
      nanochat_record ar{};
      ar.name = a.name.c_str();
      ar.dtype = static_cast<int32_t>(a.dtype);
      ar.ndim = static_cast<int32_t>(a.shape.size());
      ar.dims = a.shape.data();
      ar.data = a.data.data();
      ar.bytes = static_cast<int64_t>(a.data.size());
      attr_store->back().push_back(ar);
    }
    o.attribute_count = static_cast<int64_t>(attr_store->back().size());
    o.attributes = attr_store->back().empty() ? nullptr : attr_store->back().data();
  }
}

nanochat_status nanochat_checkpoint_read(const char* path, nanochat_checkpoint** owner,
                                         const nanochat_record** records, int64_t* record_count,
                                         const nanochat_record** optimizer, int64_t* optimizer_count) {
  if (owner == nullptr) return NANOCHAT_STATUS_ERROR;
  auto h = std::make_unique<nanochat_checkpoint>();
  std::string err;
  if (!h->ck.Load(path != nullptr ? path : "", true, &err)) {
    ncb_set_error(err);
    return NANOCHAT_STATUS_ERROR;
  }
  h->attr_store.reserve(h->ck.tensors.size() + h->ck.optimizer_state.size());
  export_records(h->ck.tensors, &h->records, &h->attr_store);
  export_records(h->ck.optimizer_state, &h->optimizer, &h->attr_store);
  if (records != nullptr) *records = h->records.data();
  if (record_count != nullptr) *record_count = static_cast<int64_t>(h->records.size());
  if (optimizer != nullptr) *optimizer = h->optimizer.data();
  if (optimizer_count != nullptr) *optimizer_count = static_cast<int64_t>(h->optimizer.size());
  *owner = h.release();
  return NANOCHAT_STATUS_OK;
}
void nanochat_checkpoint_free(nanochat_checkpoint* owner) { delete owner; }

// ---- record files -------------------------------------------------------------------------------------------
struct ncb_record_file {
  std::vector<ncb::FixtureRecord> recs;
  std::vector<std::vector<int64_t>> dims;
  std::vector<nanochat_record> out;
};

nanochat_status ncb_record_file_read(const char* path, ncb_record_file** owner, char magic[9],
                                     const nanochat_record** records, int64_t* record_count) {
  if (owner == nullptr || path == nullptr) return NANOCHAT_STATUS_ERROR;
  auto h = std::make_unique<ncb_record_file>();
  std::string mg, err;
  if (!ncb::ReadRecordFile(path, &mg, &h->recs, &err)) {
    ncb_set_error(err.empty() ? std::string("cannot read record file ") + path : err);
    return NANOCHAT_STATUS_ERROR;
  }
  if (magic != nullptr) {
    std::memset(magic, 0, 9);
    std::memcpy(magic, mg.data(), mg.size() < 8 ? mg.size() : 8);
  }
  h->dims.resize(h->recs.size());
  h->out.resize(h->recs.size());
  for (size_t i = 0; i < h->recs.size(); ++i) {
    const ncb::FixtureRecord& r = h->recs[i];
    h->dims[i].assign(r.dims.begin(), r.dims.end());
    nanochat_record& o = h->out[i];
    o = nanochat_record{};
    o.name = r.name.c_str();
    o.dtype = r.dtype;
    o.ndim = static_cast<int32_t>(r.dims.size());
    o.dims = h->dims[i].data();
    o.data = r.data.data();
    o.bytes = static_cast<int64_t>(r.data.size());
  }
  if (records != nullptr) *records = h->out.data();
  if (record_count != nullptr) *record_count = static_cast<int64_t>(h->out.size());
  *owner = h.release();
  return NANOCHAT_STATUS_OK;
}
void ncb_record_file_free(ncb_record_file* owner) { delete owner; }

nanochat_status ncb_record_file_write(const char* path, const char* magic, const nanochat_record* records,
                                      int64_t record_count) {
  if (path == nullptr || magic == nullptr || (records == nullptr && record_count > 0)) return NANOCHAT_STATUS_ERROR;
  std::vector<ncb::FixtureRecord> recs(static_cast<size_t>(record_count));
  for (int64_t i = 0; i < record_count; ++i) {
    const nanochat_record& r = records[i];
    recs[i].name = r.name != nullptr ? r.name : "";
    recs[i].dtype = static_cast<std::uint8_t>(r.dtype);
    for (int d = 0; d < r.ndim; ++d) recs[i].dims.push_back(static_cast<std::uint64_t>(r.dims[d]));
    const auto* bytes = static_cast<const std::uint8_t*>(r.data);
    if (bytes != nullptr && r.bytes > 0) recs[i].data.assign(bytes, bytes + r.bytes);
  }
  if (!ncb::WriteRecordFile(path, magic, recs)) {
    ncb_set_error(std::string("cannot write record file ") + path);
    return NANOCHAT_STATUS_ERROR;
  }
  return NANOCHAT_STATUS_OK;
}

nanochat_status nanochat_checkpoint_metadata_read(const char* path, nanochat_checkpoint** owner,
                                                  nanochat_checkpoint_metadata* out) {
  if (owner == nullptr || out == nullptr) return NANOCHAT_STATUS_ERROR;
  auto h = std::make_unique<nanochat_checkpoint>();
  std::string err;
  if (!h->ck.Load(path != nullptr ? path : "", false, &err)) {
    ncb_set_error(err);
    return NANOCHAT_STATUS_ERROR;
  }
  const ncb::CheckpointMetadata& m = h->ck.metadata;
  std::ostringstream js;
  js << "{\"num_layers\": " << m.config.num_layers << ", \"num_heads\": " << m.config.num_heads
     << ", \"num_kv_heads\": " << m.config.num_kv_heads << ", \"hidden_dim\": " << m.config.hidden_dim
     << ", \"seq_len\": " << m.config.seq_len << ", \"vocab_size\": " << m.config.vocab_size
     << ", \"padded_vocab_size\": " << m.config.padded_vocab_size << ", \"rope_base\": " << m.config.rope_base
     << ", \"window_pattern\": \"" << m.config.window_pattern << "\", \"value_embedding\": "
     << (m.config.value_embedding ? "true" : "false") << ", \"container_version\": " << h->ck.version << "}";
  h->config_json = js.str();
  for (const std::string& n : m.notes) h->note_ptrs.push_back(n.c_str());
  out->schema = static_cast<int32_t>(m.schema);
  out->stage = static_cast<int32_t>(m.stage);
  out->step = static_cast<int64_t>(m.step);
  out->world_size = static_cast<int64_t>(m.world_size);
  out->precision = static_cast<int32_t>(m.precision);
  out->config_json = h->config_json.c_str();
  out->tokenizer_id = m.tokenizer_id.c_str();
  out->git_revision = m.git_revision.c_str();
  out->created_utc = m.created_utc.c_str();
  out->notes = h->note_ptrs.empty() ? nullptr : h->note_ptrs.data();
  out->note_count = static_cast<int32_t>(h->note_ptrs.size());
  *owner = h.release();
  return NANOCHAT_STATUS_OK;
}
int32_t nanochat_checkpoint_metadata_stage(const nanochat_checkpoint_metadata* m) { return m ? m->stage : -1; }
int64_t nanochat_checkpoint_metadata_step(const nanochat_checkpoint_metadata* m) { return m ? m->step : -1; }
int64_t nanochat_checkpoint_metadata_world_size(const nanochat_checkpoint_metadata* m) { return m ? m->world_size : -1; }
const char* nanochat_checkpoint_metadata_config_json(const nanochat_checkpoint_metadata* m) {
  return m ? m->config_json : nullptr;
}

// ------------------------------------------------------------------ misc
int64_t ncb_parquet_read(const char* path, const char* column, char* bytes, int64_t byte_capacity, int64_t* offsets,
                         int64_t offset_capacity, int64_t* total_bytes) {
  std::vector<std::string> rows;
  std::string err;
  if (!ncb::ReadParquetStrings(path != nullptr ? path : "", column != nullptr ? column : "text", &rows, &err)) {
    ncb_set_error(err);
    return -1;
  }
  int64_t total = 0;
  for (size_t i = 0; i < rows.size(); ++i) {
    if (offsets != nullptr && static_cast<int64_t>(i) < offset_capacity) offsets[i] = total;
    if (bytes != nullptr && total + static_cast<int64_t>(rows[i].size()) <= byte_capacity)
      std::memcpy(bytes + total, rows[i].data(), rows[i].size());
    total += static_cast<int64_t>(rows[i].size());
  }
  if (offsets != nullptr && static_cast<int64_t>(rows.size()) < offset_capacity) offsets[rows.size()] = total;
  if (total_bytes != nullptr) *total_bytes = total;
  return static_cast<int64_t>(rows.size());
}

// The sampling streams of generation, for engines that keep their logits elsewhere (the GPU engine of the Python
// package): row `row_ids[r]` owns the stream Rng(MixSeed(seed, row_ids[r])) and its `draw_index`-th draw picks the
// token of its `draw_index`-th sampled position, exactly as the native generation loop consumes it
// (engine_drivers.h GenerateBatchOn; reference src/generate.cc:54, 614-669). `logits` is [rows, vocab] fp32,
// soft-capped. out[r] receives the token.
void ncb_sample_rows(const float* logits, int rows, int vocab, float temperature, int top_k, uint64_t seed,
                     const int64_t* row_ids, int64_t draw_index, int* out) {
  if (logits == nullptr || out == nullptr || rows <= 0 || vocab <= 0) return;
#pragma omp parallel for schedule(dynamic, 1)
  for (int r = 0; r < rows; ++r) {
    ncb::Rng rng(ncb::MixSeed(seed, static_cast<uint64_t>(row_ids != nullptr ? row_ids[r] : r)));
    if (temperature > 0.0f)
      for (int64_t k = 0; k < draw_index; ++k) rng.NextU64();
    out[r] = ncb::SampleToken(logits + static_cast<std::size_t>(r) * vocab, vocab, temperature, top_k, &rng);
  }
}

int ncb_sample_token(const float* logits, int vocab, float temperature, int top_k, uint64_t seed, uint64_t row,
                     uint64_t step) {
  ncb::Rng rng(ncb::MixSeed(ncb::MixSeed(seed, row), step));
  return ncb::SampleToken(logits, vocab, temperature, top_k, &rng);
}

}  // extern "C"
