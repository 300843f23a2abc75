// The C++ engine behind the C ABI on a CUDA device: the nanochat graph driven straight through the sm_100a kernel
// launchers of csrc/cuda (no Python, no PyTorch). Same graph and the same kernels as the Python package's model:
//
//     e = rmsnorm(wte[token]);  x = smear(e);  x0 = x
//     per layer: xr = resid*x + x0_lambda*x0; h = rmsnorm(xr); [q|k|v] = h Wqkv^T (one GEMM)
//                v += 3*sigmoid(h[:, :12] Wg^T) * value_embeds[token]        (alternating layers)
//                q, k = 1.2*rope(rmsnorm_head(.)); a = attention(q, k, v)     (causal, windows, GQA)
//                x_mid = xr + a Wo^T; h2 = rmsnorm(x_mid); x = x_mid + relu(h2 Wfc^T)^2 Wproj^T
//     x -= backout * x_{L/2}; logits = rmsnorm(x) Wlm^T in row chunks; loss = CE(15 tanh(logits/15))
//
// with a hand-written backward (weight gradients accumulated by the GEMM epilogue into the flat fp32 gradient, on a
// second stream), Muon on the matrices and AdamW on the rest, and per-sequence inference over a paged KV cache.
// The reference's counterpart is its model / optimizer / generation code linked against its CUDA backend
// (src/model.cc:828-1186, src/optim.cc:154-232, src/generate.cc:266-412).
//
// Memory: parameters live in three flat device buffers (fp32 master, bf16 compute copy, fp32 gradient; 64-element
// aligned offsets so the fused QKV view exists); activations are persistent per-shape buffers (grown on demand,
// never freed inside a step), so a step allocates nothing after the first one of its shape.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "../cuda/attention.h"
#include "../cuda/decode.h"
#include "../cuda/gemm_tcgen05.h"
#include "../cuda/optim.h"
#include "../cuda/rowops.h"
#include "../host/device_engine.h"

namespace ncb {
namespace {

using bf16 = __nv_bfloat16;
constexpr float kRmsEps = 1.1920929e-07f, kSoftcap = 15.0f, kQkScale = 1.2f;
constexpr int kGateCh = 12, kSmearCh = 24, kAlign = 64, kPage = 16;
constexpr double kPolar[5][3] = {{8.156554524902461, -22.48329292557795, 15.878769915207462},
                                 {4.042929935166739, -2.808917465908714, 0.5000178451051316},
                                 {3.8916678022926607, -2.772484153217685, 0.5060648178503393},
                                 {3.285753657755655, -2.3681294933425376, 0.46449024233003106},
                                 {2.3465413258596377, -1.7097828382687081, 0.42323551169305323}};

void Check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void CheckLaunch(const char* err, const char* what) {
  if (err != nullptr) throw std::runtime_error(std::string(what) + ": " + err);
}

// A device buffer that only ever grows.
struct Buf {
  void* p = nullptr;
  std::size_t bytes = 0;
  void* Need(std::size_t n) {
    if (n > bytes) {
      if (p != nullptr) Check(cudaFree(p), "cudaFree");
      p = nullptr;
      bytes = 0;
      Check(cudaMalloc(&p, n), "cudaMalloc");
      bytes = n;
    }
    return p;
  }
  template <typename T>
  T* As(std::size_t count) { return static_cast<T*>(Need(count * sizeof(T))); }
  ~Buf() {
    if (p != nullptr) cudaFree(p);
  }
};

struct LayerBufs {
  Buf xr, h, qkv, qk, gate, attn, x_mid, h2, act, x_out, rstd1, rstd2, lse;
};

class GpuCache : public DeviceCache {
 public:
  int max_seq = 0, pages = 0, len = 0;
  bool has_prev = false;
  std::vector<Buf> k, v;   // per layer: [pages, kPage, KV, D] bf16
  Buf page_table, prev_emb, seq_len_dev, pos_dev;
};

struct MuonGroupState {
  int rows = 0, cols = 0;
  float lr = 0;
  std::vector<std::size_t> params;     // indices into the parameter table
  Buf buf1, buf2, x32, X, Y, A, B, row_ss, row_scale, all_scale, line_ss, scale, line_scale, tables;
  bool on_host = false;                // a shape neither device path takes: updated on the host
  bool tiny = false;                   // small matrices (the gate projections): one launch does the whole group's step
  std::vector<std::vector<float>> h_buf1, h_buf2;
};
struct AdamGroupState {
  ParamKind kind;
  float lr, beta1, beta2, wd;
  std::vector<std::size_t> params;
  std::vector<Buf> m, v;
};

class GpuEngine final : public DeviceEngine {
 public:
  GpuEngine(const EngineConfig& cfg, int device) : cfg_(cfg), device_(device) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    Check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    Check(cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking), "cudaStreamCreate");
    Check(cudaEventCreateWithFlags(&ev_main_, cudaEventDisableTiming), "cudaEventCreate");
    BuildParams();
    master_ = params_buf_[0].As<float>(total_);
    value_ = params_buf_[1].As<bf16>(total_);
    grad_ = params_buf_[2].As<float>(total_);
    Check(cudaMemsetAsync(master_, 0, total_ * sizeof(float), stream_), "memset");
    Check(cudaMemsetAsync(value_, 0, total_ * sizeof(bf16), stream_), "memset");
    Check(cudaMemsetAsync(grad_, 0, total_ * sizeof(float), stream_), "memset");
    status_ = status_buf_.As<int>(4);
    Check(cudaMemsetAsync(status_, 0, 4 * sizeof(int), stream_), "memset");
    layers_.resize(static_cast<std::size_t>(cfg_.num_layers));
    side_done_.resize(static_cast<std::size_t>(cfg_.num_layers), nullptr);
    for (auto& e : side_done_) Check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    Check(cudaStreamSynchronize(stream_), "sync");
  }
  ~GpuEngine() override {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (auto& e : side_done_)
      if (e != nullptr) cudaEventDestroy(e);
    cudaEventDestroy(ev_main_);
    cudaStreamDestroy(side_);
    cudaStreamDestroy(stream_);
  }

  const EngineConfig& config() const override { return cfg_; }
  const std::vector<CpuParam>& params() const override { return params_; }
  const std::vector<float>& losses() const override { return losses_; }
  const std::vector<float>& logits() const override { return logits_; }
  std::int64_t valid_targets() const override { return valid_; }
  float grad_norm() const override { return grad_norm_; }
  std::int64_t LaunchCount() const override { return launches_; }

  bool ReadActivation(const std::string& name, int layer, std::vector<float>* out) override {
    Use();
    const EngineConfig& c = cfg_;
    const std::size_t m = static_cast<std::size_t>(M_), C = static_cast<std::size_t>(c.hidden_dim);
    const std::size_t wide = static_cast<std::size_t>(c.query_dim() + 2 * c.kv_dim());
    const std::size_t hk = static_cast<std::size_t>(c.num_heads + c.num_kv_heads) * c.head_dim();
    if (name.rfind("value:", 0) == 0) {     // the bf16 compute copy of a parameter
      const auto it = index_.find(name.substr(6));
      if (it == index_.end()) return false;
      const CpuParam& p = params_[it->second];
      Check(cudaStreamSynchronize(stream_), "sync");
      std::vector<bf16> raw(p.count);
      ToHost(raw.data(), value_ + p.offset, p.count * sizeof(bf16), "value read");
      out->resize(p.count);
      for (std::size_t i = 0; i < p.count; ++i) (*out)[i] = __bfloat162float(raw[i]);
      return true;
    }
    Buf* b = nullptr;
    std::size_t n = m * C;
    if (name == "emb") b = &emb_;
    else if (name == "x0") b = &x0_;
    else if (name == "xn") b = &xn_;
    else if (layer >= 0 && layer < c.num_layers) {
      LayerBufs& lb = layers_[static_cast<std::size_t>(layer)];
      if (name == "xr") b = &lb.xr;
      else if (name == "h") b = &lb.h;
      else if (name == "qkv") b = &lb.qkv, n = m * wide;
      else if (name == "qk") b = &lb.qk, n = m * hk;
      else if (name == "attn") b = &lb.attn, n = m * static_cast<std::size_t>(c.query_dim());
      else if (name == "x_mid") b = &lb.x_mid;
      else if (name == "h2") b = &lb.h2;
      else if (name == "act") b = &lb.act, n = m * static_cast<std::size_t>(c.mlp_dim());
      else if (name == "x_out") b = &lb.x_out;
    }
    if (b == nullptr || b->p == nullptr || b->bytes < n * sizeof(bf16)) return false;
    Check(cudaStreamSynchronize(stream_), "sync");
    std::vector<bf16> raw(n);
    ToHost(raw.data(), b->p, n * sizeof(bf16), "activation read");
    out->resize(n);
    for (std::size_t i = 0; i < n; ++i) (*out)[i] = __bfloat162float(raw[i]);
    return true;
  }

  int Status() override {
    Use();
    Check(cudaStreamSynchronize(stream_), "sync");
    Check(cudaStreamSynchronize(side_), "sync");
    int code = 0;
    ToHost(&code, status_, sizeof(int), "status read");
    return code;
  }

  // ------------------------------------------------------------------------------------------------ parameters
  void ReadParam(std::size_t index, bool grad, std::int64_t offset, std::int64_t count, float* dst) override {
    Use();
    const CpuParam& p = params_.at(index);
    Check(cudaStreamSynchronize(stream_), "sync");
    Check(cudaStreamSynchronize(side_), "sync");
    ToHost(dst, (grad ? grad_ : master_) + p.offset + offset, static_cast<std::size_t>(count) * sizeof(float), "param read");
  }
  void WriteParam(std::size_t index, bool grad, std::int64_t offset, std::int64_t count, const float* src) override {
    Use();
    const CpuParam& p = params_.at(index);
    Check(cudaStreamSynchronize(stream_), "sync");
    float* dst = (grad ? grad_ : master_) + p.offset + offset;
    ToDevice(dst, src, static_cast<std::size_t>(count) * sizeof(float), "param write");
    if (!grad) {
      nc::cast_f32_bf16(dst, value_ + p.offset + offset, count, stream_);
      ++launches_;
      Check(cudaStreamSynchronize(stream_), "sync");
    }
  }
  void ZeroGrad() override {
    Use();
    Check(cudaMemsetAsync(grad_, 0, total_ * sizeof(float), stream_), "zero grad");
  }

  // ------------------------------------------------------------------------------------------------ training
  float ForwardLoss(const int* tokens, const int* targets, int batch, int seq, bool keep_logits) override {
    Use();
    Stage(tokens, targets, batch, seq);
    Trunk(batch, seq, /*save=*/true, nullptr);
    Head(/*want_grad=*/false, 1.0f, nullptr, 0.0, keep_logits);
    return FinishLoss();
  }
  void Backward(float scale, const float* row_weights, double divisor) override {
    Use();
    if (!have_saved_) throw std::runtime_error("Backward without a preceding ForwardLoss");
    Head(/*want_grad=*/true, scale, row_weights, divisor, false);
    BackwardBody();
  }
  float ForwardBackward(const int* tokens, const int* targets, int batch, int seq, float scale) override {
    Use();
    Stage(tokens, targets, batch, seq);
    Trunk(batch, seq, true, nullptr);
    Head(true, scale, nullptr, 0.0, false);
    BackwardBody();
    return FinishLoss();
  }

  // ------------------------------------------------------------------------------------------------ optimizer
  void OptimInit(const OptimConfig& c) override {
    Use();
    ocfg_ = c;
    adam_.clear();
    muon_.clear();
    const float scale = std::sqrt(768.0f / static_cast<float>(cfg_.hidden_dim)), f = c.init_lr_frac;
    adam_.push_back({ParamKind::kLmHead, c.unembedding_lr * scale * f, 0.8f, 0.96f, 0.01f, {}, {}, {}});
    adam_.push_back({ParamKind::kWte, c.embedding_lr * scale * f, 0.8f, 0.995f, 0.001f, {}, {}, {}});
    adam_.push_back({ParamKind::kValueEmbed, c.embedding_lr * scale * 0.5f * f, 0.8f, 0.995f, 0.01f, {}, {}, {}});
    adam_.push_back({ParamKind::kResid, c.scalar_lr * 0.01f * f, 0.8f, 0.95f, 0.05f, {}, {}, {}});
    adam_.push_back({ParamKind::kX0, c.scalar_lr * f, 0.96f, 0.95f, 0.0f, {}, {}, {}});
    adam_.push_back({ParamKind::kSmear, 0.2f * f, 0.8f, 0.95f, 0.0f, {}, {}, {}});
    for (std::size_t i = 0; i < params_.size(); ++i) {
      const CpuParam& p = params_[i];
      if (p.kind != ParamKind::kMatrix) {
        for (auto& g : adam_)
          if (g.kind == p.kind) g.params.push_back(i);
        continue;
      }
      MuonGroupState* grp = nullptr;
      for (auto& g : muon_)
        if (g.rows == p.rows && g.cols == p.cols) grp = &g;
      if (grp == nullptr) {
        muon_.emplace_back();
        grp = &muon_.back();
        grp->rows = p.rows, grp->cols = p.cols;
        grp->lr = c.matrix_lr * f * std::sqrt(std::max(1.0f, static_cast<float>(p.rows) / static_cast<float>(p.cols)));
        grp->on_host = std::min(p.rows, p.cols) < 64 || p.rows % 8 != 0 || p.cols % 8 != 0;
        if (grp->on_host && static_cast<long long>(p.rows) * p.cols <= 1024 && std::min(p.rows, p.cols) <= 32) {
          grp->on_host = false;
          grp->tiny = true;
        }
      }
      grp->params.push_back(i);
    }
    for (auto& g : adam_) {
      g.m.resize(g.params.size());
      g.v.resize(g.params.size());
      for (std::size_t k = 0; k < g.params.size(); ++k) {
        const std::size_t n = params_[g.params[k]].count;
        Check(cudaMemsetAsync(g.m[k].As<float>(n), 0, n * sizeof(float), stream_), "memset");
        Check(cudaMemsetAsync(g.v[k].As<float>(n), 0, n * sizeof(float), stream_), "memset");
      }
    }
    for (auto& g : muon_) {
      const std::size_t P = g.params.size(), n = static_cast<std::size_t>(g.rows) * g.cols;
      const std::size_t lines = static_cast<std::size_t>(g.rows >= g.cols ? g.rows : g.cols);
      if (g.on_host) {
        g.h_buf1.assign(P, std::vector<float>(n, 0.0f));
        g.h_buf2.assign(P, std::vector<float>(lines, 0.0f));
        continue;
      }
      const std::size_t k = static_cast<std::size_t>(std::min(g.rows, g.cols));
      Check(cudaMemsetAsync(g.buf1.As<float>(P * n), 0, P * n * sizeof(float), stream_), "memset");
      Check(cudaMemsetAsync(g.buf2.As<float>(P * lines), 0, P * lines * sizeof(float), stream_), "memset");
      if (!g.tiny) {
        g.x32.As<float>(P * n), g.X.As<bf16>(P * n), g.Y.As<bf16>(P * n), g.A.As<bf16>(P * k * k), g.B.As<bf16>(P * k * k);
        g.row_ss.As<float>(P * g.rows), g.row_scale.As<float>(P * g.rows), g.all_scale.As<float>(P);
        g.line_ss.As<float>(P * lines), g.scale.As<float>(P), g.line_scale.As<float>(P * lines);
      }
      // address tables: gradients, buf1 slices, buf2 slices, masters, values
      std::vector<long long> t(5 * P);
      for (std::size_t j = 0; j < P; ++j) {
        const CpuParam& p = params_[g.params[j]];
        t[j] = reinterpret_cast<long long>(grad_ + p.offset);
        t[P + j] = reinterpret_cast<long long>(g.buf1.As<float>(P * n) + j * n);
        t[2 * P + j] = reinterpret_cast<long long>(g.buf2.As<float>(P * lines) + j * lines);
        t[3 * P + j] = reinterpret_cast<long long>(master_ + p.offset);
        t[4 * P + j] = reinterpret_cast<long long>(value_ + p.offset);
      }
      Check(cudaMemcpyAsync(g.tables.As<long long>(5 * P), t.data(), t.size() * sizeof(long long),
                            cudaMemcpyHostToDevice, stream_), "tables");
      Check(cudaStreamSynchronize(stream_), "sync");
    }
    norm_.As<double>(1);
    norm_clip_.As<float>(2);
    Check(cudaStreamSynchronize(stream_), "sync");
    optim_ready_ = true;
  }

  void OptimStep(int step) override {
    Use();
    if (!optim_ready_) throw std::runtime_error("OptimStep before OptimInit");
    Join();   // weight gradients come from the side stream
    double* ss = norm_.As<double>(1);
    float* nc2 = norm_clip_.As<float>(2);
    Check(cudaMemsetAsync(ss, 0, sizeof(double), stream_), "memset");
    nc::sumsq_f32(grad_, static_cast<long long>(total_), ss, stream_);
    nc::finish_norm(ss, ocfg_.clip, nc2, stream_);
    launches_ += 2;
    const float* clip = nc2 + 1;
    const float lrm = ocfg_.LrMultiplier(step);
    for (auto& g : adam_)
      for (std::size_t k = 0; k < g.params.size(); ++k) {
        const CpuParam& p = params_[g.params[k]];
        nc::adamw_update(master_ + p.offset, value_ + p.offset, grad_ + p.offset, g.m[k].As<float>(p.count),
                         g.v[k].As<float>(p.count), static_cast<long long>(p.count), g.lr * lrm, g.beta1, g.beta2,
                         ocfg_.adam_eps, g.wd, step, clip, stream_);
        ++launches_;
      }
    const float momentum = ocfg_.MuonMomentum(step), wd = ocfg_.WeightDecay(step);
    float host_clip = 1.0f;
    bool have_host_clip = false;
    for (auto& g : muon_) {
      if (g.on_host) {
        if (!have_host_clip) {
          float both[2];
          Check(cudaStreamSynchronize(stream_), "sync");
          ToHost(both, nc2, sizeof(both), "clip read");
          host_clip = both[1];
          have_host_clip = true;
        }
        MuonOnHost(&g, g.lr * lrm, momentum, wd, host_clip);
      } else if (g.tiny) {
        const int P = static_cast<int>(g.params.size());
        const long long* t = g.tables.As<long long>(1);
        const char* err = nc::muon_tiny(t, t + P, t + 2 * P, t + 3 * P, t + 4 * P, P, g.rows, g.cols, momentum,
                                        ocfg_.muon_beta2, g.lr * lrm, wd, ocfg_.muon_ns_steps, clip, kPolar, stream_);
        if (err != nullptr) throw std::runtime_error(err);
        ++launches_;
      } else {
        MuonOnDevice(&g, g.lr * lrm, momentum, wd, clip);
      }
    }
    float both[2];
    Check(cudaStreamSynchronize(stream_), "sync");
    ToHost(both, nc2, sizeof(both), "norm read");
    grad_norm_ = both[0];
  }

  // ------------------------------------------------------------------------------------------------ inference
  std::unique_ptr<DeviceCache> NewCache(int max_seq) override {
    Use();
    auto c = std::make_unique<GpuCache>();
    c->max_seq = max_seq;
    c->pages = (max_seq + kPage - 1) / kPage;
    const std::size_t per = static_cast<std::size_t>(c->pages) * kPage * cfg_.kv_dim();
    c->k.resize(static_cast<std::size_t>(cfg_.num_layers));
    c->v.resize(static_cast<std::size_t>(cfg_.num_layers));
    for (int i = 0; i < cfg_.num_layers; ++i) {
      Check(cudaMemsetAsync(c->k[i].As<bf16>(per), 0, per * sizeof(bf16), stream_), "memset");
      Check(cudaMemsetAsync(c->v[i].As<bf16>(per), 0, per * sizeof(bf16), stream_), "memset");
    }
    std::vector<int> table(static_cast<std::size_t>(c->pages));
    for (int i = 0; i < c->pages; ++i) table[i] = i;
    Check(cudaMemcpyAsync(c->page_table.As<int>(table.size()), table.data(), table.size() * sizeof(int),
                          cudaMemcpyHostToDevice, stream_), "page table");
    c->prev_emb.As<bf16>(static_cast<std::size_t>(cfg_.hidden_dim));
    c->seq_len_dev.As<int>(1);
    Check(cudaStreamSynchronize(stream_), "sync");
    return c;
  }
  void Prefill(DeviceCache* cache, const int* tokens, int count, std::vector<float>* last_logits) override {
    Use();
    auto* c = static_cast<GpuCache*>(cache);
    if (c->len != 0) throw std::runtime_error("Prefill expects a fresh cache");
    if (count + c->len > c->max_seq) throw std::runtime_error("prompt does not fit the KV cache");
    std::vector<int> none(static_cast<std::size_t>(count), -1);
    Stage(tokens, none.data(), 1, count);
    Trunk(1, count, false, c);
    c->len = count;
    c->has_prev = true;
    LastLogits(count - 1, last_logits);
  }
  void Decode(DeviceCache* cache, int token, std::vector<float>* logits) override {
    Use();
    auto* c = static_cast<GpuCache*>(cache);
    if (c->len + 1 > c->max_seq) throw std::runtime_error("KV cache is full");
    const int none = -1;
    Stage(&token, &none, 1, 1);
    Trunk(1, 1, false, c);
    c->len += 1;
    LastLogits(0, logits);
  }

 private:
  void Use() { Check(cudaSetDevice(device_), "cudaSetDevice"); }
  // Every copy goes through the engine's own stream. A plain cudaMemcpy is ordered against the legacy default stream
  // only, and for pageable host memory it may return while the last staged piece is still on its way to the device:
  // a kernel on this (non-blocking) stream could then read the destination before the data has landed.
  void ToDevice(void* dst, const void* src, std::size_t bytes, const char* what) {
    Check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream_), what);
    Check(cudaStreamSynchronize(stream_), what);
  }
  void ToHost(void* dst, const void* src, std::size_t bytes, const char* what) {
    Check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream_), what);
    Check(cudaStreamSynchronize(stream_), what);
  }

  void BuildParams() {
    const EngineConfig& c = cfg_;
    const int L = c.num_layers, C = c.hidden_dim, V = c.padded_vocab_size;
    auto add = [&](std::string name, std::vector<std::int64_t> shape, int rows, int cols, ParamKind kind, int layer) {
      CpuParam p;
      p.name = std::move(name), p.shape = std::move(shape), p.rows = rows, p.cols = cols, p.kind = kind, p.layer = layer;
      p.count = 1;
      for (auto d : p.shape) p.count *= static_cast<std::size_t>(d);
      p.offset = total_;
      total_ += (p.count + kAlign - 1) / kAlign * kAlign;
      params_.push_back(std::move(p));
    };
    add("lm_head.weight", {V, C}, V, C, ParamKind::kLmHead, -1);
    add("transformer.wte.weight", {V, C}, V, C, ParamKind::kWte, -1);
    for (int i = 0; i < L; ++i)
      if (c.has_value_embedding(i))
        add("value_embeds." + std::to_string(i) + ".weight", {V, c.kv_dim()}, V, c.kv_dim(), ParamKind::kValueEmbed, i);
    add("resid_lambdas", {L}, 0, 0, ParamKind::kResid, -1);
    add("x0_lambdas", {L}, 0, 0, ParamKind::kX0, -1);
    add("smear_gate.weight", {1, kSmearCh}, 1, kSmearCh, ParamKind::kSmear, -1);
    add("smear_lambda", {1}, 0, 0, ParamKind::kSmear, -1);
    add("backout_lambda", {1}, 0, 0, ParamKind::kSmear, -1);
    for (int i = 0; i < L; ++i) {
      const std::string p = "transformer.h." + std::to_string(i) + ".";
      add(p + "attn.c_q.weight", {c.query_dim(), C}, c.query_dim(), C, ParamKind::kMatrix, i);
      add(p + "attn.c_k.weight", {c.kv_dim(), C}, c.kv_dim(), C, ParamKind::kMatrix, i);
      add(p + "attn.c_v.weight", {c.kv_dim(), C}, c.kv_dim(), C, ParamKind::kMatrix, i);
      add(p + "attn.c_proj.weight", {C, C}, C, C, ParamKind::kMatrix, i);
      if (c.has_value_embedding(i))
        add(p + "attn.ve_gate.weight", {c.num_kv_heads, kGateCh}, c.num_kv_heads, kGateCh, ParamKind::kMatrix, i);
      add(p + "mlp.c_fc.weight", {c.mlp_dim(), C}, c.mlp_dim(), C, ParamKind::kMatrix, i);
      add(p + "mlp.c_proj.weight", {C, c.mlp_dim()}, C, c.mlp_dim(), ParamKind::kMatrix, i);
    }
    for (std::size_t i = 0; i < params_.size(); ++i) index_[params_[i].name] = i;
    // the fused QKV product needs c_q | c_k | c_v back to back (true when their sizes are multiples of the alignment)
    fused_qkv_ = (static_cast<std::size_t>(c.query_dim()) * C) % kAlign == 0 && (static_cast<std::size_t>(c.kv_dim()) * C) % kAlign == 0;
  }
  const CpuParam& P(const std::string& name) const { return params_[index_.at(name)]; }
  const CpuParam& LP(int layer, const char* what) const {
    return P("transformer.h." + std::to_string(layer) + "." + what + ".weight");
  }
  bf16* V(const CpuParam& p) const { return value_ + p.offset; }
  float* G(const CpuParam& p) const { return grad_ + p.offset; }
  float* M(const CpuParam& p) const { return master_ + p.offset; }

  // ---- GEMM helpers (operand orders as in gemm_tcgen05.h) -----------------------------------------------------
  void Gemm(nc::GemmArgs g, cudaStream_t s) {
    g.status = status_;
    const bool plain = g.epi == nc::kEpiBf16 && g.alpha == 1.0f;
    const bool res = g.epi == nc::kEpiBf16Res && g.alpha == 1.0f && g.beta == 1.0f;
    const char* err;
    if (g.M <= 64 && g.N >= 128 && g.N <= 16384 && !g.a_mn_major && !g.b_mn_major && g.batch == 1 &&
        (plain || res || g.epi == nc::kEpiRelu2)) {
      err = nc::gemm_skinny(g, s);
    } else {
      err = nc::gemm_bf16(g, s);
    }
    ++launches_;
    CheckLaunch(err, "gemm");
  }
  // y[M, N] = x[M, K] w[N, K]^T (+ residual), or act = relu(.)^2
  void Linear(const bf16* x, long long ldx, const bf16* w, int M_, int N, int K, bf16* y, long long ldy,
              const bf16* residual = nullptr, long long ldr = 0, bool relu2 = false) {
    nc::GemmArgs g;
    g.A = x, g.lda = ldx, g.B = w, g.ldb = K, g.M = M_, g.N = N, g.K = K, g.C = y, g.ldc = ldy;
    if (residual != nullptr) {
      g.epi = nc::kEpiBf16Res, g.R = residual, g.ldr = ldr, g.alpha = 1.0f, g.beta = 1.0f;
    } else if (relu2) {
      g.epi = nc::kEpiRelu2, g.C2 = y;
    }
    Gemm(g, stream_);
  }
  // dx[M, K] = dy[M, N] w[N, K]  (optionally * 2 sqrt(act), the backward of relu^2 in terms of the saved activation)
  void Dgrad(const bf16* dy, long long lddy, const bf16* w, int M_, int N, int K, bf16* dx, long long lddx,
             const bf16* act = nullptr, long long ldact = 0) {
    nc::GemmArgs g;
    g.A = dy, g.lda = lddy, g.B = w, g.ldb = K, g.b_mn_major = true, g.M = M_, g.N = K, g.K = N, g.C = dx, g.ldc = lddx;
    if (act != nullptr) g.epi = nc::kEpiDRelu2, g.R = act, g.ldr = ldact, g.beta = 1.0f;
    Gemm(g, stream_);
  }
  // grad[N, K] += dy[M, N]^T x[M, K], on the side stream
  void Wgrad(const bf16* dy, long long lddy, const bf16* x, long long ldx, int M_, int N, int K, float* grad) {
    nc::GemmArgs g;
    g.A = dy, g.lda = lddy, g.a_mn_major = true, g.B = x, g.ldb = ldx, g.b_mn_major = true;
    g.M = N, g.N = K, g.K = M_, g.C = grad, g.ldc = K, g.epi = nc::kEpiF32, g.alpha = 1.0f, g.beta = 1.0f;
    Gemm(g, side_);
  }
  void SideAfterMain() {   // the side stream may read what the main stream has produced so far
    Check(cudaEventRecord(ev_main_, stream_), "event");
    Check(cudaStreamWaitEvent(side_, ev_main_, 0), "wait");
  }
  void Join() {            // the main stream waits for everything on the side stream
    cudaEvent_t e = side_done_.empty() ? ev_main_ : side_done_[0];
    Check(cudaEventRecord(e, side_), "event");
    Check(cudaStreamWaitEvent(stream_, e, 0), "wait");
  }

  // ---- inputs ---------------------------------------------------------------------------------------------------
  void Stage(const int* tokens, const int* targets, int batch, int seq) {
    const std::size_t m = static_cast<std::size_t>(batch) * seq;
    B_ = batch, T_ = seq, M_ = static_cast<int>(m);
    Check(cudaMemcpyAsync(tok_.As<int>(m), tokens, m * sizeof(int), cudaMemcpyHostToDevice, stream_), "tokens");
    Check(cudaMemcpyAsync(tgt_.As<int>(m), targets, m * sizeof(int), cudaMemcpyHostToDevice, stream_), "targets");
    h_targets_.assign(targets, targets + m);
    valid_ = 0;
    for (int t : h_targets_) valid_ += t != -1 ? 1 : 0;
    have_saved_ = false;
  }
  void Rope(int upto) {
    if (upto <= rope_len_) return;
    const int n = std::max(upto, std::max(2 * rope_len_, cfg_.seq_len)), half = cfg_.head_dim() / 2;
    std::vector<float> c(static_cast<std::size_t>(n) * half), s(c.size());
    for (int d = 0; d < half; ++d) {
      const float inv = 1.0f / std::pow(cfg_.rope_base, (2.0f * static_cast<float>(d)) / static_cast<float>(cfg_.head_dim()));
      for (int t = 0; t < n; ++t) {
        const float ang = static_cast<float>(t) * inv;
        c[static_cast<std::size_t>(t) * half + d] = std::cos(ang);
        s[static_cast<std::size_t>(t) * half + d] = std::sin(ang);
      }
    }
    Check(cudaStreamSynchronize(stream_), "sync");
    ToDevice(cos_.As<float>(c.size()), c.data(), c.size() * sizeof(float), "rope");
    ToDevice(sin_.As<float>(s.size()), s.data(), s.size() * sizeof(float), "rope");
    rope_len_ = n;
  }

  // ---- forward --------------------------------------------------------------------------------------------------
  // Training / scoring: `cache` null, all of [B, T] attends inside itself. Inference: B == 1, the T new tokens sit
  // at positions cache->len .. cache->len + T - 1 (T > 1 only on a fresh cache).
  void Trunk(int B, int T, bool save, GpuCache* cache) {
    const EngineConfig& c = cfg_;
    const int C = c.hidden_dim, H = c.num_heads, KV = c.num_kv_heads, D = c.head_dim(), Mr = B * T;
    const int qd = c.query_dim(), kd = c.kv_dim(), wide = qd + 2 * kd, hk = (H + KV) * D;
    const std::size_t mc = static_cast<std::size_t>(Mr) * C;
    const int* tok = tok_.As<int>(Mr);
    const int t0 = cache != nullptr ? cache->len : 0;
    Rope(cache != nullptr ? cache->max_seq : T);
    const float* cosT = cos_.As<float>(1);
    const float* sinT = sin_.As<float>(1);
    const int* positions = nullptr;
    if (cache != nullptr) {
      std::vector<int> pos(static_cast<std::size_t>(T));
      for (int t = 0; t < T; ++t) pos[t] = t0 + t;
      Check(cudaMemcpyAsync(cache->pos_dev.As<int>(pos.size()), pos.data(), pos.size() * sizeof(int),
                            cudaMemcpyHostToDevice, stream_), "positions");
      positions = cache->pos_dev.As<int>(pos.size());
      const int new_len = t0 + T;
      Check(cudaMemcpyAsync(cache->seq_len_dev.As<int>(1), &new_len, sizeof(int), cudaMemcpyHostToDevice, stream_), "len");
    }
    bf16* emb_raw = emb_raw_.As<bf16>(mc);
    bf16* emb = emb_.As<bf16>(mc);
    bf16* x0 = x0_.As<bf16>(mc);
    float* rstd_e = rstd_e_.As<float>(Mr);
    float* sig = sig_.As<float>(Mr);
    nc::embedding_fwd(tok, V(P("transformer.wte.weight")), emb_raw, Mr, C, stream_, c.padded_vocab_size, status_);
    nc::rmsnorm_fwd(emb_raw, C, emb, rstd_e, Mr, C, kRmsEps, stream_);
    const bf16* prev = cache != nullptr && cache->has_prev ? cache->prev_emb.As<bf16>(C) : nullptr;
    nc::smear_fwd(emb, V(P("smear_gate.weight")), M(P("smear_lambda")), prev, x0, sig, Mr, T, C, stream_);
    launches_ += 3;
    if (cache != nullptr)
      Check(cudaMemcpyAsync(cache->prev_emb.As<bf16>(C), emb + static_cast<std::size_t>(Mr - 1) * C, C * sizeof(bf16),
                            cudaMemcpyDeviceToDevice, stream_), "prev emb");
    const bf16* x = x0;
    const float* resid = M(P("resid_lambdas"));
    const float* x0lam = M(P("x0_lambdas"));
    for (int i = 0; i < c.num_layers; ++i) {
      LayerBufs& lb = layers_[save ? i : 0];
      bf16* xr = lb.xr.As<bf16>(mc);
      bf16* h = lb.h.As<bf16>(mc);
      float* rstd1 = lb.rstd1.As<float>(Mr);
      nc::blend_norm_fwd(x, x0, resid + i, x0lam + i, xr, h, rstd1, Mr, C, kRmsEps, stream_);
      ++launches_;
      bf16* qkv = lb.qkv.As<bf16>(static_cast<std::size_t>(Mr) * wide);
      if (fused_qkv_) {
        Linear(h, C, V(LP(i, "attn.c_q")), Mr, wide, C, qkv, wide);
      } else {
        Linear(h, C, V(LP(i, "attn.c_q")), Mr, qd, C, qkv, wide);
        Linear(h, C, V(LP(i, "attn.c_k")), Mr, kd, C, qkv + qd, wide);
        Linear(h, C, V(LP(i, "attn.c_v")), Mr, kd, C, qkv + qd + kd, wide);
      }
      bf16* v = qkv + qd + kd;
      if (c.has_value_embedding(i)) {
        bf16* gate = lb.gate.As<bf16>(static_cast<std::size_t>(Mr) * KV);
        // the gate kernel reads the embedding rows straight from the table
        nc::value_gate_fwd(h, C, V(P("value_embeds." + std::to_string(i) + ".weight")), V(LP(i, "attn.ve_gate")), v, wide,
                           gate, Mr, KV, D, stream_, tok, c.padded_vocab_size, status_);
        ++launches_;
      }
      bf16* attn = lb.attn.As<bf16>(static_cast<std::size_t>(Mr) * qd);
      const int wl = c.window_left(i);
      const float scale = 1.0f / std::sqrt(static_cast<float>(D));
      if (cache != nullptr && T == 1) {
        bf16* q1 = lb.qk.As<bf16>(static_cast<std::size_t>(hk));
        if (D == 128) {
          CheckLaunch(nc::decode_prep_append(qkv, wide, v, wide, cosT, sinT, positions, cache->page_table.As<int>(1),
                                             cache->pages, kPage, q1, cache->k[i].As<bf16>(1), cache->v[i].As<bf16>(1), 1,
                                             H, KV, D, kRmsEps, kQkScale, stream_, cache->pages, status_),
                      "decode_prep_append");
          ++launches_;
        } else {
          nc::qk_prep_fwd(qkv, wide, q1, hk, cosT, sinT, positions, 1, 1, H + KV, D, kRmsEps, kQkScale, stream_);
          nc::kv_append(cache->k[i].As<bf16>(1), cache->v[i].As<bf16>(1), cache->page_table.As<int>(1), cache->pages,
                        positions, q1 + qd, hk, v, wide, 1, 1, kPage, kd, stream_, cache->pages, status_);
          launches_ += 2;
        }
        nc::DecodeArgs a;
        a.B = 1, a.H = H, a.KV = KV, a.D = D, a.q = q1, a.q_stride_b = hk;
        a.k_pool = cache->k[i].As<bf16>(1), a.v_pool = cache->v[i].As<bf16>(1);
        a.page_table = cache->page_table.As<int>(1), a.max_pages = cache->pages, a.page_size = kPage;
        a.seq_lens = cache->seq_len_dev.As<int>(1), a.window_left = wl, a.scale = scale, a.out = attn;
        const int keys = wl >= 0 ? std::min(cache->max_seq, wl + 1) : cache->max_seq;
        a.splits = nc::decode_splits(1, KV, keys);
        if (a.splits > 1) {
          a.part_acc = part_acc_.As<float>(static_cast<std::size_t>(H) * a.splits * D);
          a.part_ml = part_ml_.As<float>(static_cast<std::size_t>(H) * a.splits * 2);
        }
        CheckLaunch(nc::paged_decode_attention(a, stream_), "paged_decode_attention");
        launches_ += a.splits > 1 ? 2 : 1;
      } else {
        bf16* qk = lb.qk.As<bf16>(static_cast<std::size_t>(Mr) * hk);
        nc::qk_prep_fwd(qkv, wide, qk, hk, cosT, sinT, positions, Mr, T, H + KV, D, kRmsEps, kQkScale, stream_);
        ++launches_;
        if (cache != nullptr) {
          nc::kv_append(cache->k[i].As<bf16>(1), cache->v[i].As<bf16>(1), cache->page_table.As<int>(1), cache->pages,
                        positions, qk + qd, hk, v, wide, 1, T, kPage, kd, stream_, cache->pages, status_);
          ++launches_;
        }
        nc::AttnArgs a;
        a.B = B, a.H = H, a.KVH = KV, a.Tq = T, a.Tk = T, a.D = D, a.q_offset = 0, a.window_left = wl, a.scale = scale;
        a.Q = qk, a.q_stride_t = hk, a.q_stride_h = D, a.q_stride_b = static_cast<long long>(T) * hk;
        a.K = qk + qd, a.k_stride_t = hk, a.k_stride_h = D, a.k_stride_b = static_cast<long long>(T) * hk;
        a.V = v, a.v_stride_t = wide, a.v_stride_h = D, a.v_stride_b = static_cast<long long>(T) * wide;
        a.O = attn, a.o_stride_t = qd, a.o_stride_h = D, a.o_stride_b = static_cast<long long>(T) * qd;
        a.lse = lb.lse.As<float>(static_cast<std::size_t>(B) * H * T);
        a.status = status_;
        CheckLaunch(nc::attention_fwd2(a, stream_), "attention_fwd2");
        ++launches_;
      }
      bf16* x_mid = lb.x_mid.As<bf16>(mc);
      Linear(attn, qd, V(LP(i, "attn.c_proj")), Mr, C, qd, x_mid, C, xr, C);
      bf16* h2 = lb.h2.As<bf16>(mc);
      float* rstd2 = lb.rstd2.As<float>(Mr);
      nc::rmsnorm_fwd(x_mid, C, h2, rstd2, Mr, C, kRmsEps, stream_);
      ++launches_;
      bf16* act = lb.act.As<bf16>(static_cast<std::size_t>(Mr) * c.mlp_dim());
      Linear(h2, C, V(LP(i, "mlp.c_fc")), Mr, c.mlp_dim(), C, act, c.mlp_dim(), nullptr, 0, true);
      // without saving, layer outputs alternate between two buffers (layer i reads what layer i-1 wrote)
      bf16* x_out = (save ? lb.x_out : (i % 2 ? x_alt_ : lb.x_out)).As<bf16>(mc);
      Linear(act, c.mlp_dim(), V(LP(i, "mlp.c_proj")), Mr, C, c.mlp_dim(), x_out, C, x_mid, C);
      if (i == c.backout_layer()) {
        Check(cudaMemcpyAsync(x_backout_.As<bf16>(mc), x_out, mc * sizeof(bf16), cudaMemcpyDeviceToDevice, stream_), "backout copy");
      }
      x = x_out;
    }
    x_last_ = x;
    bf16* x_pre = x_pre_.As<bf16>(mc);
    nc::backout_fwd(x, x_backout_.As<bf16>(mc), M(P("backout_lambda")), x_pre, static_cast<long long>(mc), stream_);
    nc::rmsnorm_fwd(x_pre, C, xn_.As<bf16>(mc), rstd_f_.As<float>(Mr), Mr, C, kRmsEps, stream_);
    launches_ += 2;
    have_saved_ = save;
  }

  // LM head in row chunks: GEMM -> soft cap + cross entropy (in place, with the backward when asked) -> dgrad / wgrad.
  void Head(bool want_grad, float scale, const float* row_weights, double divisor, bool keep_logits) {
    const EngineConfig& c = cfg_;
    const int C = c.hidden_dim, PV = c.padded_vocab_size, Mr = M_;
    const int chunk = std::min(head_chunk_rows_, Mr);
    const CpuParam& lm = P("lm_head.weight");
    bf16* logits = head_logits_.As<bf16>(static_cast<std::size_t>(chunk) * PV);
    float* losses = head_losses_.As<float>(Mr);
    const bf16* xn = xn_.As<bf16>(1);
    float* dscale = dscale_.As<float>(1);
    const float* rs = nullptr;
    if (want_grad) {
      const double denom = divisor > 0.0 ? divisor : static_cast<double>(std::max<std::int64_t>(valid_, 1));
      const float ds = static_cast<float>(static_cast<double>(scale) / denom);
      Check(cudaMemcpyAsync(dscale, &ds, sizeof(float), cudaMemcpyHostToDevice, stream_), "dlogit scale");
      if (row_weights != nullptr) {
        Check(cudaMemcpyAsync(row_scale_.As<float>(Mr), row_weights, static_cast<std::size_t>(Mr) * sizeof(float),
                              cudaMemcpyHostToDevice, stream_), "row weights");
        rs = row_scale_.As<float>(Mr);
      }
      dxn_.As<bf16>(static_cast<std::size_t>(Mr) * C);
    }
    if (keep_logits) logits_.assign(static_cast<std::size_t>(Mr) * PV, 0.0f);
    std::vector<bf16> host_chunk;
    for (int a = 0; a < Mr; a += chunk) {
      const int rows = std::min(chunk, Mr - a);
      if (want_grad) Join();   // the previous chunk's weight-gradient product still reads the logits buffer
      Linear(xn + static_cast<std::size_t>(a) * C, C, V(lm), rows, PV, C, logits, PV);
      if (keep_logits) {
        host_chunk.resize(static_cast<std::size_t>(rows) * PV);
        Check(cudaStreamSynchronize(stream_), "sync");
        ToHost(host_chunk.data(), logits, host_chunk.size() * sizeof(bf16), "logits");
        float* dst = logits_.data() + static_cast<std::size_t>(a) * PV;
        for (std::size_t j = 0; j < host_chunk.size(); ++j) dst[j] = __bfloat162float(host_chunk[j]);
      }
      nc::classifier_fwd_bwd(logits, PV, tgt_.As<int>(1) + a, losses + a, rs != nullptr ? rs + a : nullptr,
                             want_grad ? dscale : nullptr, rows, c.vocab_size, PV, kSoftcap, -1, want_grad, stream_,
                             status_);
      ++launches_;
      if (want_grad) {
        Dgrad(logits, PV, V(lm), rows, PV, C, dxn_.As<bf16>(1) + static_cast<std::size_t>(a) * C, C);
        SideAfterMain();
        Wgrad(logits, PV, xn + static_cast<std::size_t>(a) * C, C, rows, PV, C, G(lm));
      }
    }
    losses_.resize(static_cast<std::size_t>(Mr));
    Check(cudaMemcpyAsync(losses_.data(), losses, losses_.size() * sizeof(float), cudaMemcpyDeviceToHost, stream_), "losses");
  }
  float FinishLoss() {
    Check(cudaStreamSynchronize(stream_), "sync");
    double s = 0.0;
    for (std::size_t i = 0; i < losses_.size(); ++i)
      if (h_targets_[i] != -1) s += losses_[i];
    return static_cast<float>(s / static_cast<double>(std::max<std::int64_t>(valid_, 1)));
  }
  void LastLogits(int row, std::vector<float>* out) {
    const EngineConfig& c = cfg_;
    const int C = c.hidden_dim, PV = c.padded_vocab_size;
    bf16* lg = head_logits_.As<bf16>(static_cast<std::size_t>(PV));
    Linear(xn_.As<bf16>(1) + static_cast<std::size_t>(row) * C, C, V(P("lm_head.weight")), 1, PV, C, lg, PV);
    float* capped = capped_.As<float>(static_cast<std::size_t>(c.vocab_size));
    nc::softcap_logits(lg, PV, capped, 1, c.vocab_size, kSoftcap, stream_);
    ++launches_;
    out->resize(static_cast<std::size_t>(c.vocab_size));
    Check(cudaMemcpyAsync(out->data(), capped, out->size() * sizeof(float), cudaMemcpyDeviceToHost, stream_), "logits");
    Check(cudaStreamSynchronize(stream_), "sync");
  }

  // ---- backward (after Head(want_grad) has produced d(xn) and the LM-head gradient) ------------------------------
  void BackwardBody() {
    const EngineConfig& c = cfg_;
    const int B = B_, T = T_, Mr = M_, C = c.hidden_dim, H = c.num_heads, KV = c.num_kv_heads, D = c.head_dim();
    const int qd = c.query_dim(), kd = c.kv_dim(), wide = qd + 2 * kd, hk = (H + KV) * D, F = c.mlp_dim();
    const std::size_t mc = static_cast<std::size_t>(Mr) * C;
    const int* tok = tok_.As<int>(Mr);
    const float* cosT = cos_.As<float>(1);
    const float* sinT = sin_.As<float>(1);
    // sizes of the shared scratch are fixed before anything is enqueued: growing a buffer later would move it
    s_a_.As<bf16>(mc);
    s_b_.As<bf16>(static_cast<std::size_t>(Mr) * std::max(qd, C));
    bf16* dx_pre = dx_pre_.As<bf16>(mc);      // read by the top layer's side-stream product: a buffer of its own
    nc::rmsnorm_bwd(x_pre_.As<bf16>(mc), dxn_.As<bf16>(mc), rstd_f_.As<float>(Mr), nullptr, dx_pre, Mr, C, stream_);
    bf16* dxb = dxb_.As<bf16>(mc);
    nc::backout_bwd(dx_pre, x_backout_.As<bf16>(mc), M(P("backout_lambda")), dxb, G(P("backout_lambda")),
                    static_cast<long long>(mc), stream_);
    launches_ += 2;
    const bf16* x0 = x0_.As<bf16>(mc);
    bf16* dx0 = dx0_.As<bf16>(mc);
    bool have_dx0 = false;
    const bf16* dx = dx_pre;                    // gradient flowing into the current layer's output
    const float* resid = M(P("resid_lambdas"));
    const float* x0lam = M(P("x0_lambdas"));
    for (int i = c.num_layers - 1; i >= 0; --i) {
      LayerBufs& lb = layers_[i];
      const int par = i & 1;
      // scratch of this parity was last read by the side stream two layers ago
      if (i + 2 < c.num_layers) Check(cudaStreamWaitEvent(stream_, side_done_[i + 2], 0), "wait");
      if (i == c.backout_layer()) {
        bf16* sum = s_sum_[par].As<bf16>(mc);
        nc::add_bf16(dx, dxb, sum, static_cast<long long>(mc), stream_);
        ++launches_;
        dx = sum;
      }
      const bf16* act = lb.act.As<bf16>(1);
      const bf16* h2 = lb.h2.As<bf16>(1);
      const bf16* x_mid = lb.x_mid.As<bf16>(1);
      // MLP
      bf16* dpre = s_dpre_[par].As<bf16>(static_cast<std::size_t>(Mr) * F);
      SideAfterMain();
      Wgrad(dx, C, act, F, Mr, C, F, G(LP(i, "mlp.c_proj")));
      Dgrad(dx, C, V(LP(i, "mlp.c_proj")), Mr, C, F, dpre, F, act, F);
      SideAfterMain();
      Wgrad(dpre, F, h2, C, Mr, F, C, G(LP(i, "mlp.c_fc")));
      bf16* dh2 = s_b_.As<bf16>(mc);
      Dgrad(dpre, F, V(LP(i, "mlp.c_fc")), Mr, F, C, dh2, C);
      bf16* dx_mid = s_dxmid_[par].As<bf16>(mc);
      nc::rmsnorm_bwd(x_mid, dh2, lb.rstd2.As<float>(1), dx, dx_mid, Mr, C, stream_);
      ++launches_;
      // attention output projection
      const bf16* attn = lb.attn.As<bf16>(1);
      SideAfterMain();
      Wgrad(dx_mid, C, attn, qd, Mr, C, qd, G(LP(i, "attn.c_proj")));
      bf16* dattn = s_b_.As<bf16>(static_cast<std::size_t>(Mr) * std::max(qd, C));
      Dgrad(dx_mid, C, V(LP(i, "attn.c_proj")), Mr, C, qd, dattn, qd);
      bf16* dqkv = s_dqkv_[par].As<bf16>(static_cast<std::size_t>(Mr) * wide);
      bf16* dqk = s_dqk_.As<bf16>(static_cast<std::size_t>(Mr) * hk);
      const bf16* qkv = lb.qkv.As<bf16>(1);
      const bf16* qk = lb.qk.As<bf16>(1);
      {
        nc::AttnArgs a;
        a.B = B, a.H = H, a.KVH = KV, a.Tq = T, a.Tk = T, a.D = D, a.q_offset = 0, a.window_left = c.window_left(i);
        a.scale = 1.0f / std::sqrt(static_cast<float>(D));
        a.Q = qk, a.q_stride_t = hk, a.q_stride_h = D, a.q_stride_b = static_cast<long long>(T) * hk;
        a.K = qk + qd, a.k_stride_t = hk, a.k_stride_h = D, a.k_stride_b = static_cast<long long>(T) * hk;
        a.V = qkv + qd + kd, a.v_stride_t = wide, a.v_stride_h = D, a.v_stride_b = static_cast<long long>(T) * wide;
        a.O = const_cast<bf16*>(attn), a.o_stride_t = qd, a.o_stride_h = D, a.o_stride_b = static_cast<long long>(T) * qd;
        a.lse = lb.lse.As<float>(1);
        a.dO = dattn, a.do_stride_t = qd, a.do_stride_h = D, a.do_stride_b = static_cast<long long>(T) * qd;
        a.delta = delta_.As<float>(static_cast<std::size_t>(B) * H * T);
        const long long t128 = (T + 127) / 128 * 128;
        const std::size_t ds_elems = static_cast<std::size_t>(B) * H * t128 * t128;
        if (ds_elems * sizeof(bf16) <= (6ull << 30)) {
          a.dS = ds_.As<bf16>(ds_elems);
          a.ds_tk = t128, a.ds_tq = t128;
        }
        a.dQ = dqk, a.dq_stride_t = hk, a.dq_stride_h = D, a.dq_stride_b = static_cast<long long>(T) * hk;
        a.dK = dqk + qd, a.dk_stride_t = hk, a.dk_stride_h = D, a.dk_stride_b = static_cast<long long>(T) * hk;
        a.dV = dqkv + qd + kd, a.dv_stride_t = wide, a.dv_stride_h = D, a.dv_stride_b = static_cast<long long>(T) * wide;
        a.status = status_;
        CheckLaunch(nc::attention_bwd(a, stream_), "attention_bwd");
        launches_ += 3;
      }
      nc::qk_prep_bwd(qkv, wide, dqk, hk, dqkv, wide, cosT, sinT, Mr, T, H + KV, D, kRmsEps, kQkScale, stream_);
      ++launches_;
      const bf16* h = lb.h.As<bf16>(1);
      float* dh12 = nullptr;
      if (c.has_value_embedding(i)) {
        const CpuParam& table = P("value_embeds." + std::to_string(i) + ".weight");
        bf16* ve = s_ve_.As<bf16>(static_cast<std::size_t>(Mr) * kd);
        bf16* dve = s_dve_.As<bf16>(static_cast<std::size_t>(Mr) * kd);
        dh12 = dh12_.As<float>(static_cast<std::size_t>(Mr) * kGateCh);
        nc::embedding_fwd(tok, V(table), ve, Mr, kd, stream_, c.padded_vocab_size, status_);
        nc::value_gate_bwd(h, C, ve, V(LP(i, "attn.ve_gate")), lb.gate.As<bf16>(1), dqkv + qd + kd, wide, dve, dh12,
                           G(LP(i, "attn.ve_gate")), Mr, KV, D, stream_);
        nc::embedding_bwd(tok, dve, kd, G(table), Mr, kd, stream_, c.padded_vocab_size, status_);
        launches_ += 3;
      }
      bf16* dh = s_a_.As<bf16>(mc);
      SideAfterMain();
      if (fused_qkv_) {
        Wgrad(dqkv, wide, h, C, Mr, wide, C, G(LP(i, "attn.c_q")));
        Dgrad(dqkv, wide, V(LP(i, "attn.c_q")), Mr, wide, C, dh, C);
      } else {
        Wgrad(dqkv, wide, h, C, Mr, qd, C, G(LP(i, "attn.c_q")));
        Wgrad(dqkv + qd, wide, h, C, Mr, kd, C, G(LP(i, "attn.c_k")));
        Wgrad(dqkv + qd + kd, wide, h, C, Mr, kd, C, G(LP(i, "attn.c_v")));
        nc::GemmArgs g;   // dh = dq Wq + dk Wk + dv Wv through the residual epilogue
        Dgrad(dqkv, wide, V(LP(i, "attn.c_q")), Mr, qd, C, dh, C);
        for (int part = 0; part < 2; ++part) {
          const bf16* dy = dqkv + qd + part * kd;
          const bf16* w = V(LP(i, part == 0 ? "attn.c_k" : "attn.c_v"));
          g = nc::GemmArgs();
          g.A = dy, g.lda = wide, g.B = w, g.ldb = C, g.b_mn_major = true, g.M = Mr, g.N = C, g.K = kd, g.C = dh, g.ldc = C;
          g.epi = nc::kEpiBf16Res, g.R = dh, g.ldr = C, g.alpha = 1.0f, g.beta = 1.0f;
          Gemm(g, stream_);
        }
      }
      Check(cudaEventRecord(side_done_[i], side_), "event");
      const bf16* x_in = i == 0 ? x0 : layers_[i - 1].x_out.As<bf16>(1);
      bf16* dx_next = s_dx_[par].As<bf16>(mc);
      // this buffer's previous content (written by layer i + 2) was read by layer i + 1's side-stream products
      if (i + 1 < c.num_layers) Check(cudaStreamWaitEvent(stream_, side_done_[i + 1], 0), "wait");
      // norm backward + blend backward + the gate's columns + both scalar gradients: one launch, dxr never stored
      CheckLaunch(nc::norm_blend_bwd(lb.xr.As<bf16>(1), dh, lb.rstd1.As<float>(1), dx_mid, dh12, dh12 != nullptr ? kGateCh : 0,
                                     x_in, x0, resid + i, x0lam + i, dx_next, dx0, have_dx0, G(P("resid_lambdas")) + i,
                                     G(P("x0_lambdas")) + i, Mr, C, stream_),
                  "norm_blend_bwd");
      ++launches_;
      have_dx0 = true;
      dx = dx_next;
    }
    // embedding side
    bf16* dsum = s_b_.As<bf16>(mc);
    nc::add_bf16(dx0, dx, dsum, static_cast<long long>(mc), stream_);
    bf16* de = s_a_.As<bf16>(mc);
    nc::smear_bwd(emb_.As<bf16>(mc), V(P("smear_gate.weight")), M(P("smear_lambda")), sig_.As<float>(Mr), dsum, de,
                  G(P("smear_gate.weight")), G(P("smear_lambda")), Mr, T, C, stream_);
    bf16* de_raw = s_b_.As<bf16>(mc);
    nc::rmsnorm_bwd(emb_raw_.As<bf16>(mc), de, rstd_e_.As<float>(Mr), nullptr, de_raw, Mr, C, stream_);
    nc::embedding_bwd(tok, de_raw, C, G(P("transformer.wte.weight")), Mr, C, stream_, c.padded_vocab_size, status_);
    launches_ += 4;
    Join();
    have_saved_ = false;
  }

  // ---- Muon -----------------------------------------------------------------------------------------------------
  void BatchedGemm(const bf16* A, bool a_mn, const bf16* B, bool b_mn, int M_, int N, int K, int lda, int ldb, bf16* C,
                   int P, long long sA, long long sB, long long sC, const bf16* R, float alpha, float beta) {
    nc::GemmArgs g;
    g.A = A, g.B = B, g.lda = lda, g.ldb = ldb, g.a_mn_major = a_mn, g.b_mn_major = b_mn, g.M = M_, g.N = N, g.K = K;
    g.batch = P, g.strideA = sA, g.strideB = sB, g.strideC = sC, g.C = C, g.ldc = N;
    if (R != nullptr) g.epi = nc::kEpiBf16Res, g.R = R, g.ldr = N, g.strideR = sC, g.alpha = alpha, g.beta = beta;
    Gemm(g, stream_);
  }
  void MuonOnDevice(MuonGroupState* g, float lr, float momentum, float wd, const float* clip) {
    const int P = static_cast<int>(g->params.size()), rows = g->rows, cols = g->cols;
    const long long n = static_cast<long long>(rows) * cols;
    const bool reduce_cols = rows >= cols, tall = rows > cols;
    const int lines = reduce_cols ? rows : cols, line_len = reduce_cols ? cols : rows, k = tall ? cols : rows;
    const long long* t = g->tables.As<long long>(1);
    float* x32 = g->x32.As<float>(1);
    bf16* X = g->X.As<bf16>(1);
    bf16* Y = g->Y.As<bf16>(1);
    bf16* A = g->A.As<bf16>(1);
    bf16* Bm = g->B.As<bf16>(1);
    nc::muon_nesterov_batched(t, t + P, x32, g->row_ss.As<float>(1), P, rows, cols, momentum, clip, stream_);
    nc::muon_prescale(g->row_ss.As<float>(1), g->row_scale.As<float>(1), g->all_scale.As<float>(1), P, rows, stream_);
    nc::muon_scale_rows_batched(x32, g->row_scale.As<float>(1), g->all_scale.As<float>(1), X, P, rows, cols, stream_);
    launches_ += 3;
    const long long kk = static_cast<long long>(k) * k;
    for (int it = 0; it < std::min(std::max(ocfg_.muon_ns_steps, 0), 5); ++it) {
      const float ca = static_cast<float>(kPolar[it][0]), cb = static_cast<float>(kPolar[it][1]),
                  cc = static_cast<float>(kPolar[it][2]);
      if (tall) {
        BatchedGemm(X, true, X, true, cols, cols, rows, cols, cols, A, P, n, n, kk, nullptr, 1.0f, 0.0f);    // X^T X
        BatchedGemm(A, false, A, false, k, k, k, k, k, Bm, P, kk, kk, kk, A, cc, cb);                         // b A + c A A
        BatchedGemm(X, false, Bm, false, rows, cols, cols, cols, cols, Y, P, n, kk, n, X, 1.0f, ca);          // a X + X B
      } else {
        BatchedGemm(X, false, X, false, rows, rows, cols, cols, cols, A, P, n, n, kk, nullptr, 1.0f, 0.0f);  // X X^T
        BatchedGemm(A, false, A, false, k, k, k, k, k, Bm, P, kk, kk, kk, A, cc, cb);
        BatchedGemm(Bm, false, X, true, rows, cols, rows, rows, cols, Y, P, kk, n, n, X, 1.0f, ca);           // a X + B X
      }
      std::swap(X, Y);
    }
    nc::muon_line_sumsq(X, g->line_ss.As<float>(1), P, rows, cols, reduce_cols, stream_);
    nc::muon_poststats(g->line_ss.As<float>(1), t + 2 * P, g->scale.As<float>(1), g->line_scale.As<float>(1), P, lines,
                       line_len, std::sqrt(static_cast<float>(std::min(rows, cols))), ocfg_.muon_beta2, stream_);
    nc::muon_apply_batched(t + 3 * P, t + 4 * P, X, g->scale.As<float>(1), g->line_scale.As<float>(1), reduce_cols, P,
                           rows, cols, lr, wd, stream_);
    launches_ += 3;
  }
  void MuonOnHost(MuonGroupState* g, float lr, float momentum, float wd, float clip) {
    const std::size_t n = static_cast<std::size_t>(g->rows) * g->cols;
    std::vector<float> w(n), gr(n);
    std::vector<bf16> wb(n);
    Check(cudaStreamSynchronize(stream_), "sync");
    for (std::size_t j = 0; j < g->params.size(); ++j) {
      const CpuParam& p = params_[g->params[j]];
      ToHost(w.data(), M(p), n * sizeof(float), "muon host");
      ToHost(gr.data(), G(p), n * sizeof(float), "muon host");
      MuonUpdateHost(w.data(), gr.data(), g->h_buf1[j].data(), g->h_buf2[j].data(), g->rows, g->cols, lr, momentum, wd,
                     ocfg_.muon_beta2, ocfg_.muon_ns_steps, clip);
      for (std::size_t e = 0; e < n; ++e) wb[e] = __float2bfloat16(w[e]);
      ToDevice(M(p), w.data(), n * sizeof(float), "muon host");
      ToDevice(V(p), wb.data(), n * sizeof(bf16), "muon host");
    }
  }

  EngineConfig cfg_;
  int device_ = 0;
  cudaStream_t stream_ = nullptr, side_ = nullptr;
  cudaEvent_t ev_main_ = nullptr;
  std::vector<cudaEvent_t> side_done_;
  std::vector<CpuParam> params_;
  std::map<std::string, std::size_t> index_;
  std::size_t total_ = 0;
  bool fused_qkv_ = false;
  Buf params_buf_[3], status_buf_;
  float* master_ = nullptr;
  bf16* value_ = nullptr;
  float* grad_ = nullptr;
  int* status_ = nullptr;
  std::int64_t launches_ = 0;
  // step state
  int B_ = 0, T_ = 0, M_ = 0, rope_len_ = 0, head_chunk_rows_ = 11264;
  bool have_saved_ = false;
  std::int64_t valid_ = 0;
  std::vector<int> h_targets_;
  std::vector<float> losses_, logits_;
  const bf16* x_last_ = nullptr;
  Buf tok_, tgt_, cos_, sin_, emb_raw_, emb_, x0_, rstd_e_, sig_, x_alt_, x_backout_, x_pre_, xn_, rstd_f_;
  Buf head_logits_, head_losses_, dscale_, row_scale_, dxn_, capped_, part_acc_, part_ml_;
  Buf s_a_, s_b_, dx_pre_, dxb_, dx0_, s_dqk_, s_ve_, s_dve_, dh12_, delta_, ds_;
  Buf s_sum_[2], s_dpre_[2], s_dxmid_[2], s_dqkv_[2], s_dx_[2];
  std::vector<LayerBufs> layers_;
  // optimizer
  OptimConfig ocfg_;
  bool optim_ready_ = false;
  std::vector<AdamGroupState> adam_;
  std::vector<MuonGroupState> muon_;
  Buf norm_, norm_clip_;
  float grad_norm_ = 0.0f;
};

}  // namespace
}  // namespace ncb

extern "C" {

__attribute__((visibility("default"))) int ncb_gpu_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

__attribute__((visibility("default"))) int ncb_gpu_device_at(int ordinal, ncb::DeviceDescription* out) {
  cudaDeviceProp prop;
  if (out == nullptr || ordinal < 0 || ordinal >= ncb_gpu_device_count() ||
      cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess)
    return 0;
  out->index = ordinal, out->compute_major = prop.major, out->compute_minor = prop.minor;
  out->total_memory_bytes = static_cast<std::int64_t>(prop.totalGlobalMem);
  std::snprintf(out->name, sizeof(out->name), "%s", prop.name);
  return 1;
}

__attribute__((visibility("default"))) ncb::DeviceEngine* ncb_gpu_engine_create(const ncb::EngineConfig* cfg, int device,
                                                                                 char* error, int error_capacity) {
  try {
    if (cfg == nullptr) throw std::runtime_error("config is null");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) throw std::runtime_error("no such CUDA device");
    if (prop.major != 10) throw std::runtime_error(std::string("the kernels are built for sm_100a; device is ") + prop.name);
    if (cfg->head_dim() != 128 && cfg->head_dim() != 64) throw std::runtime_error("head_dim must be 64 or 128 on the GPU");
    return new ncb::GpuEngine(*cfg, device);
  } catch (const std::exception& e) {
    if (error != nullptr && error_capacity > 0) std::snprintf(error, static_cast<std::size_t>(error_capacity), "%s", e.what());
    return nullptr;
  }
}

}  // extern "C"
