// Native planning layer (see plan.h).
#include "plan.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <set>
#include <sstream>

#include "perf.h"

namespace ncb {

// ---------------------------------------------------------------------------------------------------------------------
// JSON
// ---------------------------------------------------------------------------------------------------------------------
namespace {

struct Reader {
  const std::string& s;
  std::size_t i = 0;
  std::string err;
  explicit Reader(const std::string& text) : s(text) {}
  void Skip() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  bool Fail(const std::string& what) {
    if (err.empty()) err = what + " at byte " + std::to_string(i);
    return false;
  }
  bool String(std::string* out) {
    if (i >= s.size() || s[i] != '"') return Fail("expected a string");
    ++i;
    out->clear();
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c == '\\') {
        if (i >= s.size()) return Fail("unterminated escape");
        const char e = s[i++];
        switch (e) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case '/': case '\\': case '"': out->push_back(e); break;
          case 'u': {
            if (i + 4 > s.size()) return Fail("short \\u escape");
            const unsigned cp = static_cast<unsigned>(std::strtoul(s.substr(i, 4).c_str(), nullptr, 16));
            i += 4;
            if (cp < 0x80) {
              out->push_back(static_cast<char>(cp));
            } else if (cp < 0x800) {
              out->push_back(static_cast<char>(0xC0 | (cp >> 6)));
              out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            } else {
              out->push_back(static_cast<char>(0xE0 | (cp >> 12)));
              out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
              out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            }
            break;
          }
          default: return Fail("unknown escape");
        }
      } else {
        out->push_back(c);
      }
    }
    if (i >= s.size()) return Fail("unterminated string");
    ++i;
    return true;
  }
  bool Value(Json* out, int depth) {
    if (depth > 64) return Fail("nesting too deep");
    Skip();
    if (i >= s.size()) return Fail("unexpected end");
    const char c = s[i];
    if (c == '{') {
      out->kind = Json::kObject;
      ++i;
      Skip();
      if (i < s.size() && s[i] == '}') { ++i; return true; }
      while (true) {
        Skip();
        std::string key;
        if (!String(&key)) return false;
        for (const auto& kv : out->obj)
          if (kv.first == key) return Fail("duplicate key \"" + key + "\"");
        Skip();
        if (i >= s.size() || s[i] != ':') return Fail("expected ':'");
        ++i;
        Json v;
        if (!Value(&v, depth + 1)) return false;
        out->obj.emplace_back(std::move(key), std::move(v));
        Skip();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; return true; }
        return Fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      out->kind = Json::kArray;
      ++i;
      Skip();
      if (i < s.size() && s[i] == ']') { ++i; return true; }
      while (true) {
        Json v;
        if (!Value(&v, depth + 1)) return false;
        out->arr.push_back(std::move(v));
        Skip();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; return true; }
        return Fail("expected ',' or ']'");
      }
    }
    if (c == '"') {
      out->kind = Json::kString;
      return String(&out->str);
    }
    if (s.compare(i, 4, "true") == 0) { out->kind = Json::kBool; out->b = true; i += 4; return true; }
    if (s.compare(i, 5, "false") == 0) { out->kind = Json::kBool; out->b = false; i += 5; return true; }
    if (s.compare(i, 4, "null") == 0) { out->kind = Json::kNull; i += 4; return true; }
    char* end = nullptr;
    const double v = std::strtod(s.c_str() + i, &end);
    if (end == s.c_str() + i) return Fail("unexpected character");
    out->kind = Json::kNumber;
    out->num = v;
    i = static_cast<std::size_t>(end - s.c_str());
    return true;
  }
};

std::string Num(double v) {
  char buf[64];
  if (v == std::floor(v) && std::fabs(v) < 9e15) {
    std::snprintf(buf, sizeof(buf), "%.0f", v);
  } else {
    std::snprintf(buf, sizeof(buf), "%.17g", v);
  }
  return buf;
}

}  // namespace

const Json* Json::Find(const std::string& key) const {
  for (const auto& kv : obj)
    if (kv.first == key) return &kv.second;
  return nullptr;
}

bool ParseJson(const std::string& text, Json* out, std::string* error) {
  Reader r(text);
  if (!r.Value(out, 0)) {
    if (error != nullptr) *error = "json: " + r.err;
    return false;
  }
  r.Skip();
  if (r.i != text.size()) {
    if (error != nullptr) *error = "json: trailing characters at byte " + std::to_string(r.i);
    return false;
  }
  return true;
}

std::string JsonQuote(const std::string& s) {
  std::string o = "\"";
  for (char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\t': o += "\\t"; break;
      default:
        if (static_cast<unsigned char>(c) < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", c);
          o += buf;
        } else {
          o.push_back(c);
        }
    }
  }
  return o + "\"";
}

// ---------------------------------------------------------------------------------------------------------------------
// Model specification
// ---------------------------------------------------------------------------------------------------------------------
namespace {

bool OnlyKeys(const Json& obj, const std::set<std::string>& allowed, const std::string& where, std::string* error) {
  std::string extra;
  for (const auto& kv : obj.obj)
    if (allowed.count(kv.first) == 0) extra += (extra.empty() ? "" : ", ") + kv.first;
  if (!extra.empty()) {
    *error = where + ": unknown keys: " + extra;
    return false;
  }
  return true;
}

bool OneOf(const std::string& value, const std::set<std::string>& allowed, const std::string& where, std::string* error) {
  if (allowed.count(value) != 0) return true;
  std::string list;
  for (const auto& a : allowed) list += (list.empty() ? "" : ", ") + a;
  *error = where + " = \"" + value + "\" is not one of " + list;
  return false;
}

}  // namespace

bool ParseModelSpec(const std::string& json_text, ModelSpec* out, std::string* error) {
  std::string err;
  Json d;
  if (!ParseJson(json_text, &d, &err) || d.kind != Json::kObject) {
    *error = err.empty() ? "spec: not a JSON object" : err;
    return false;
  }
  if (!OnlyKeys(d, {"spec_version", "name", "requires", "dimensions", "blocks", "head", "embedding", "backout_layer"},
                "spec", error))
    return false;
  const Json* ver = d.Find("spec_version");
  if (ver == nullptr || ver->kind != Json::kNumber || ver->num != 1.0) {
    *error = "spec: unsupported spec_version";
    return false;
  }
  for (const char* k : {"name", "dimensions", "blocks"})
    if (!d.Has(k)) {
      *error = std::string("spec lacks \"") + k + "\"";
      return false;
    }
  ModelSpec s;
  s.name = d.Find("name")->str;
  if (const Json* r = d.Find("requires"))
    for (const Json& e : r->arr) s.requires_.push_back(e.str);
  const Json& dm = *d.Find("dimensions");
  if (!OnlyKeys(dm, {"num_heads", "num_kv_heads", "hidden_dim", "seq_len", "rope_base", "vocab_size", "padded_vocab_size"},
                "dimensions", error))
    return false;
  auto geti = [&dm](const char* k, int fallback) {
    const Json* v = dm.Find(k);
    return v != nullptr && v->kind == Json::kNumber ? static_cast<int>(v->num) : fallback;
  };
  if (!dm.Has("num_heads") || !dm.Has("hidden_dim")) {
    *error = "dimensions need num_heads and hidden_dim";
    return false;
  }
  s.num_heads = geti("num_heads", 0);
  s.num_kv_heads = geti("num_kv_heads", s.num_heads);
  s.hidden_dim = geti("hidden_dim", 0);
  s.seq_len = geti("seq_len", 2048);
  s.vocab_size = geti("vocab_size", 32768);
  s.padded_vocab_size = geti("padded_vocab_size", (s.vocab_size + 63) / 64 * 64);
  if (const Json* rb = dm.Find("rope_base")) s.rope_base = rb->num;
  const Json& blocks = *d.Find("blocks");
  if (blocks.kind != Json::kArray || blocks.arr.empty()) {
    *error = "a model needs at least one block";
    return false;
  }
  for (std::size_t i = 0; i < blocks.arr.size(); ++i) {
    const Json& b = blocks.arr[i];
    const std::string where = "block " + std::to_string(i);
    if (!OnlyKeys(b, {"norm", "attention", "attention_variant", "position", "mlp", "residual", "dtype", "value_embedding"},
                  where, error))
      return false;
    BlockSpec bs;
    struct Field {
      const char* key;
      std::string* dst;
      std::set<std::string> allowed;
    } fields[] = {{"norm", &bs.norm, {"rms_norm"}},
                  {"attention", &bs.attention, {"causal", "sliding_window"}},
                  {"attention_variant", &bs.attention_variant, {"mha", "gqa"}},
                  {"position", &bs.position, {"rope"}},
                  {"mlp", &bs.mlp, {"relu_square"}},
                  {"residual", &bs.residual, {"blend"}},
                  {"dtype", &bs.dtype, {"build_default", "fp32", "bf16", "fp8"}}};
    for (auto& f : fields)
      if (const Json* v = b.Find(f.key)) {
        if (!OneOf(v->str, f.allowed, where + ": " + f.key, error)) return false;
        *f.dst = v->str;
      }
    if (const Json* v = b.Find("value_embedding")) bs.value_embedding = v->kind == Json::kBool ? v->b : v->num != 0;
    s.blocks.push_back(bs);
  }
  if (const Json* bl = d.Find("backout_layer"))
    if (bl->kind == Json::kNumber) s.backout_layer = static_cast<int>(bl->num);
  *out = std::move(s);
  return true;
}

bool SpecToConfig(const ModelSpec& spec, EngineConfig* out, std::string* error) {
  std::string pattern;
  for (const BlockSpec& b : spec.blocks) pattern.push_back(b.attention == "sliding_window" ? 'S' : 'L');
  // the last layer is always full context whatever the pattern says; the shortest repeating prefix describes the rest
  std::string body = pattern;
  std::size_t period = body.size();
  for (std::size_t p = 1; p <= body.size(); ++p) {
    bool ok = true;
    for (std::size_t i = 0; i + 1 < body.size() && ok; ++i) ok = body[i] == body[i % p];
    if (ok) {
      period = p;
      break;
    }
  }
  EngineConfig c;
  c.num_layers = static_cast<int>(spec.blocks.size());
  c.num_heads = spec.num_heads;
  c.num_kv_heads = spec.num_kv_heads;
  c.hidden_dim = spec.hidden_dim;
  c.seq_len = spec.seq_len;
  c.vocab_size = spec.vocab_size;
  c.padded_vocab_size = spec.padded_vocab_size;
  c.rope_base = static_cast<float>(spec.rope_base);
  c.window_pattern = body.substr(0, period);
  c.value_embedding = std::any_of(spec.blocks.begin(), spec.blocks.end(), [](const BlockSpec& b) { return b.value_embedding; });
  if (!c.Validate(error)) return false;
  *out = c;
  return true;
}

// ---------------------------------------------------------------------------------------------------------------------
// Device profile
// ---------------------------------------------------------------------------------------------------------------------
bool DeviceProfile::Has(const std::string& feature) const {
  return std::find(features.begin(), features.end(), feature) != features.end();
}

bool ParseDeviceProfile(const std::string& json_text, DeviceProfile* out, std::string* error) {
  Json d;
  if (!ParseJson(json_text, &d, error) || d.kind != Json::kObject) {
    if (error->empty()) *error = "caps: not a JSON object";
    return false;
  }
  const Json* dev = d.Find("device");
  if (dev == nullptr || dev->kind != Json::kString) {
    *error = "caps: no \"device\" name";
    return false;
  }
  DeviceProfile p;
  p.device = dev->str;
  auto strings = [&d](const char* key, std::vector<std::string>* dst) {
    if (const Json* a = d.Find(key))
      for (const Json& e : a->arr)
        if (e.kind == Json::kString) dst->push_back(e.str);
  };
  strings("match", &p.match);
  strings("features", &p.features);
  strings("precisions", &p.precisions);
  if (const Json* pk = d.Find("peaks"))
    for (const auto& kv : pk->obj)
      if (kv.second.kind == Json::kNumber) p.peaks[kv.first] = kv.second.num;
  *out = std::move(p);
  return true;
}

// ---------------------------------------------------------------------------------------------------------------------
// Operator plan
// ---------------------------------------------------------------------------------------------------------------------
namespace {
struct Family {
  const char* family;
  const char* feature;
  const char* kernel;
};
// operation family -> the capability that grants its fused kernel, and what that kernel is
const Family kFamilies[] = {
    {"linear", "fused_gemm_epilogue", "gemm_tcgen05 (pair tiles, fused residual / relu^2 / accumulate epilogues)"},
    {"blend_rms_norm", "fused_blend_rms_norm", "rowops.blend_norm"},
    {"qk_prep", "fused_qk_prep", "rowops.qk_prep (norm + rope + scale, q and k in one launch)"},
    {"attention_forward", "fused_attention_forward", "attention_fwd2 (tcgen05 flash, window-aware)"},
    {"attention_backward", "fused_attention_backward", "attention_bwd (dQ and dK/dV kernels)"},
    {"classifier", "fused_classifier", "rowops.classifier_smem (softcap + CE forward/backward in place)"},
    {"muon", "fused_muon", "optim.muon_* + batched tcgen05 Newton-Schulz"},
    {"adamw", "fused_adamw", "optim.adamw / comm.adamw_push"},
    {"decode_attention", "paged_kv_decode", "decode.paged_decode (split-KV)"},
    {"gradient_sync", "peer_reduce_scatter", "comm.grad_push + grad_reduce_local + update-and-push"},
};
}  // namespace

bool BuildPlan(const ModelSpec& spec, const DeviceProfile& profile, const std::string& precision,
               const std::string& graph, OperatorPlan* out, std::string* error) {
  std::string missing;
  for (const std::string& r : spec.requires_)
    if (!profile.Has(r)) missing += (missing.empty() ? "'" : ", '") + r + "'";
  if (!missing.empty()) {
    *error = "device " + profile.device + " lacks required capabilities [" + missing + "]";
    return false;
  }
  auto runs = [&profile](const std::string& p) {
    return std::find(profile.precisions.begin(), profile.precisions.end(), p) != profile.precisions.end();
  };
  if (!runs(precision) && !(precision == "fp8" && runs("fp8_e4m3"))) {
    *error = "device " + profile.device + " does not run " + precision;
    return false;
  }
  const bool inference = graph == "prefill" || graph == "decode" || graph == "generate" || graph == "eval";
  OperatorPlan plan;
  plan.model = spec.name, plan.device = profile.device, plan.precision = precision, plan.graph = graph;
  for (const Family& f : kFamilies) {
    const std::string fam = f.family;
    if (inference && (fam == "attention_backward" || fam == "muon" || fam == "adamw" || fam == "gradient_sync")) continue;
    if (graph == "train" && fam == "decode_attention") continue;
    if (profile.Has(f.feature)) {
      plan.rows.push_back({fam, "kernel", f.kernel});
    } else {
      plan.rows.push_back({fam, "composition", "PyTorch operators of ops.ref"});
    }
  }
  *out = std::move(plan);
  return true;
}

std::string PlanJson(const OperatorPlan& plan) {
  std::ostringstream o;
  o << "{\"schema\": \"nanochat.plan.v1\", \"model\": " << JsonQuote(plan.model) << ", \"device\": "
    << JsonQuote(plan.device) << ", \"precision\": " << JsonQuote(plan.precision) << ", \"graph\": "
    << JsonQuote(plan.graph) << ", \"rows\": [";
  for (std::size_t i = 0; i < plan.rows.size(); ++i) {
    const PlanRow& r = plan.rows[i];
    o << (i ? ", " : "") << "{\"family\": " << JsonQuote(r.family) << ", \"choice\": " << JsonQuote(r.choice)
      << ", \"detail\": " << JsonQuote(r.detail) << "}";
  }
  o << "]}";
  return o.str();
}

// ---------------------------------------------------------------------------------------------------------------------
// Training-run plan
// ---------------------------------------------------------------------------------------------------------------------
EngineConfig ConfigForDepth(int depth, int aspect_ratio, int head_dim, int seq_len, int vocab_size, int num_kv_heads,
                            const std::string& window_pattern, double rope_base) {
  EngineConfig c;
  const int base = depth * aspect_ratio;
  c.hidden_dim = (base + head_dim - 1) / head_dim * head_dim;
  c.num_layers = depth;
  c.num_heads = c.hidden_dim / head_dim;
  c.num_kv_heads = num_kv_heads > 0 ? num_kv_heads : c.num_heads;
  c.seq_len = seq_len;
  c.vocab_size = vocab_size;
  c.padded_vocab_size = (vocab_size + 63) / 64 * 64;
  c.window_pattern = window_pattern;
  c.rope_base = static_cast<float>(rope_base);
  c.value_embedding = true;
  return c;
}

bool ComputeTrainPlan(const TrainPlanInputs& in, TrainPlan* out, std::string* error) {
  constexpr double kReferenceBatch = 524288.0;  // 2^19 tokens: the batch that is optimal at depth 12
  TrainPlan p;
  p.config = ConfigForDepth(in.depth, in.aspect_ratio, in.head_dim, in.seq_len, in.vocab_size, in.num_kv_heads,
                            in.window_pattern, in.rope_base);
  if (!p.config.Validate(error)) return false;
  const EngineConfig at12 = ConfigForDepth(12, in.aspect_ratio, in.head_dim, in.seq_len, in.vocab_size,
                                           in.num_kv_heads, in.window_pattern, in.rope_base);
  p.counts = CountParams(p.config);
  const ParamCounts ref = CountParams(at12);
  p.num_matmul_params = NumMatmulParams(p.config);
  p.flops_per_token = FlopsPerToken(p.config);
  // the horizon follows the parameters that scale with depth: the block matrices and the LM head
  p.scaling_params = p.counts.transformer_matrices + p.counts.lm_head;
  p.target_tokens = static_cast<std::int64_t>(in.target_param_data_ratio) * p.scaling_params;
  const double tokens_at12 = static_cast<double>(in.target_param_data_ratio) *
                             static_cast<double>(ref.transformer_matrices + ref.lm_head);
  std::int64_t total = in.total_batch_size;
  if (total == -1) {
    const double predicted = kReferenceBatch * std::pow(static_cast<double>(p.target_tokens) / tokens_at12, 0.383);
    total = static_cast<std::int64_t>(std::llround(std::exp2(std::nearbyint(std::log2(predicted)))));
  }
  if (total <= 0) {
    *error = "total_batch_size must be positive (or -1 for the predicted optimum)";
    return false;
  }
  p.total_batch_size = total;
  const double ratio = static_cast<double>(total) / kReferenceBatch;
  p.batch_lr_scale = ratio != 1.0 ? std::sqrt(ratio) : 1.0;
  p.weight_decay = in.weight_decay * std::sqrt(ratio) * (tokens_at12 / static_cast<double>(p.target_tokens));
  if (in.num_iterations > 0) {
    p.num_iterations = in.num_iterations;
  } else if (in.target_flops > 0) {
    p.num_iterations = static_cast<std::int64_t>(std::nearbyint(in.target_flops / (p.flops_per_token * static_cast<double>(total))));
  } else {
    p.num_iterations = p.target_tokens / total;
  }
  const std::int64_t per_micro = static_cast<std::int64_t>(in.device_batch_size) * in.seq_len;
  if (per_micro <= 0) {
    *error = "device_batch_size and seq_len must be positive";
    return false;
  }
  if (total % per_micro != 0) {
    *error = "total_batch_size (" + std::to_string(total) + ") must be a multiple of device_batch_size * seq_len (" +
             std::to_string(per_micro) + ")";
    return false;
  }
  p.grad_accum = total / per_micro;
  p.embedding_lr = in.embedding_lr * p.batch_lr_scale;
  p.unembedding_lr = in.unembedding_lr * p.batch_lr_scale;
  p.matrix_lr = in.matrix_lr * p.batch_lr_scale;
  p.scalar_lr = in.scalar_lr * p.batch_lr_scale;
  p.warmup_steps = in.warmup_steps;
  p.warmdown_ratio = in.warmdown_ratio;
  p.final_lr_frac = in.final_lr_frac;
  *out = p;
  return true;
}

std::string TrainPlanJson(const TrainPlanInputs& in, const TrainPlan& p) {
  std::ostringstream o;
  o << "{\"counts\": {\"embeddings\": " << p.counts.embeddings << ", \"lm_head\": " << p.counts.lm_head
    << ", \"num_matmul_params\": " << p.num_matmul_params << ", \"scalars\": " << p.counts.scalars
    << ", \"total\": " << p.counts.total << ", \"transformer_matrices\": " << p.counts.transformer_matrices << "}, "
    << "\"flops_per_token\": " << Num(p.flops_per_token) << ", "
    << "\"config\": {\"num_layers\": " << p.config.num_layers << ", \"num_heads\": " << p.config.num_heads
    << ", \"num_kv_heads\": " << p.config.num_kv_heads << ", \"hidden_dim\": " << p.config.hidden_dim
    << ", \"seq_len\": " << p.config.seq_len << ", \"vocab_size\": " << p.config.vocab_size
    << ", \"padded_vocab_size\": " << p.config.padded_vocab_size << ", \"window_pattern\": "
    << JsonQuote(p.config.window_pattern) << "}, "
    << "\"inputs\": {\"aspect_ratio\": " << in.aspect_ratio << ", \"depth\": " << in.depth
    << ", \"device_batch_size\": " << in.device_batch_size << ", \"head_dim\": " << in.head_dim
    << ", \"num_iterations\": " << in.num_iterations << ", \"seq_len\": " << in.seq_len << ", \"target_flops\": "
    << Num(in.target_flops) << ", \"target_param_data_ratio\": " << in.target_param_data_ratio
    << ", \"total_batch_size\": " << in.total_batch_size << ", \"vocab_size\": " << in.vocab_size
    << ", \"window_pattern\": " << JsonQuote(in.window_pattern) << "}, "
    << "\"plan\": {\"batch_lr_scale\": " << Num(p.batch_lr_scale) << ", \"grad_accum\": " << p.grad_accum
    << ", \"num_iterations\": " << p.num_iterations << ", \"optimizer\": {\"embedding_lr\": " << Num(p.embedding_lr)
    << ", \"matrix_lr\": " << Num(p.matrix_lr) << ", \"scalar_lr\": " << Num(p.scalar_lr) << ", \"unembedding_lr\": "
    << Num(p.unembedding_lr) << ", \"weight_decay\": " << Num(p.weight_decay) << "}, \"padded_vocab_size\": "
    << p.config.padded_vocab_size << ", \"scaling_params\": " << p.scaling_params << ", \"scheduler\": {\"final_lr_frac\": "
    << Num(p.final_lr_frac) << ", \"warmdown_ratio\": " << Num(p.warmdown_ratio) << ", \"warmup_steps\": "
    << p.warmup_steps << ", \"weight_decay_base\": " << Num(p.weight_decay) << "}, \"target_tokens\": "
    << p.target_tokens << ", \"total_batch_size\": " << p.total_batch_size << "}}";
  return o.str();
}

}  // namespace ncb
