// The seam between the host runtime (libnanochat_core.so: C ABI, native CLI, drivers) and a device engine.
//
// In the reference the backend is a link-time choice: the same workflow code links either the CPU kernels or the
// CUDA kernels, and every `nanochat_model_*` / `nanochat_generate*` call then runs on that backend
// (bindings/nanochat_capi.cc:355-400, src/model_factory.cc). Here the choice is made at run time: the core library
// has no CUDA dependency (it must load on a machine without a GPU) and opens `libnanochat_gpu.so`, which holds the
// sm_100a kernels and the C++ engine that drives them, when a CUDA device is selected
// (`nanochat_select_device("cuda:0")`, or NANOCHAT_DEVICE=cuda:0 in the environment).
//
// `DeviceEngine` is what the drivers above the seam need from a backend: the training step pieces, parameter access
// by name, an optimizer and per-sequence inference. Token ids and results cross the seam in host memory.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "engine.h"

namespace ncb {

class DeviceCache {
 public:
  virtual ~DeviceCache() = default;
};

struct DeviceDescription {
  int index = 0, compute_major = 0, compute_minor = 0;
  std::int64_t total_memory_bytes = 0;
  char name[128] = {0};
};

class DeviceEngine {
 public:
  virtual ~DeviceEngine() = default;
  virtual const EngineConfig& config() const = 0;
  virtual const std::vector<CpuParam>& params() const = 0;

  // Mean cross entropy over the valid targets (host ids in, a host float out: this call synchronises). Keeps what
  // Backward needs. With `keep_logits` the raw logits [B*T, padded_vocab] are also brought to the host.
  virtual float ForwardLoss(const int* tokens, const int* targets, int batch, int seq, bool keep_logits) = 0;
  virtual void Backward(float scale, const float* row_weights, double divisor) = 0;
  // ForwardLoss + Backward(scale) with the LM head's forward and backward fused per row chunk (no second pass over
  // the head); what `nanochat_train_step` and the training driver use.
  virtual float ForwardBackward(const int* tokens, const int* targets, int batch, int seq, float scale) = 0;
  virtual void ZeroGrad() = 0;
  virtual const std::vector<float>& losses() const = 0;   // per row, of the last ForwardLoss
  virtual const std::vector<float>& logits() const = 0;   // of the last ForwardLoss(keep_logits)
  virtual std::int64_t valid_targets() const = 0;

  // fp32 master weights (or gradients) of parameter `index`, `count` elements from `offset`; a write also refreshes
  // the bf16 compute copy.
  virtual void ReadParam(std::size_t index, bool grad, std::int64_t offset, std::int64_t count, float* dst) = 0;
  virtual void WriteParam(std::size_t index, bool grad, std::int64_t offset, std::int64_t count, const float* src) = 0;

  virtual void OptimInit(const OptimConfig& cfg) = 0;
  virtual void OptimStep(int step) = 0;   // 1-based
  virtual float grad_norm() const = 0;

  virtual std::unique_ptr<DeviceCache> NewCache(int max_seq) = 0;
  virtual void Prefill(DeviceCache* cache, const int* tokens, int count, std::vector<float>* last_logits) = 0;
  virtual void Decode(DeviceCache* cache, int token, std::vector<float>* logits) = 0;

  // An activation the last training-shaped forward kept ("emb", "x0", "xn", or per layer "xr", "h", "qkv", "qk",
  // "attn", "x_mid", "h2", "act", "x_out"), widened to fp32; for tests that compare engines stage by stage.
  // Returns false for an unknown name.
  virtual bool ReadActivation(const std::string& name, int layer, std::vector<float>* out) = 0;

  // First bounded-wait failure any kernel recorded on this device (0 = none); synchronises.
  virtual int Status() = 0;
  virtual std::int64_t LaunchCount() const = 0;
};

// Entry points of libnanochat_gpu.so (looked up with dlsym).
extern "C" {
typedef int (*ncb_gpu_device_count_fn)();
typedef int (*ncb_gpu_device_at_fn)(int ordinal, ncb::DeviceDescription* out);
typedef ncb::DeviceEngine* (*ncb_gpu_engine_create_fn)(const ncb::EngineConfig* cfg, int device, char* error,
                                                       int error_capacity);
}

// Adapts a DeviceEngine to the names the generic drivers (`engine_drivers.h`) call on a model.
struct DeviceModelView {
  DeviceEngine* e;
  const EngineConfig& config() const { return e->config(); }
  std::unique_ptr<DeviceCache> NewCache(int max_seq) { return e->NewCache(max_seq); }
  void Prefill(DeviceCache* c, const int* t, int n, std::vector<float>* out) { e->Prefill(c, t, n, out); }
  void Decode(DeviceCache* c, int tok, std::vector<float>* out) { e->Decode(c, tok, out); }
  float ForwardLoss(const int* t, const int* g, int b, int s, bool keep = false) { return e->ForwardLoss(t, g, b, s, keep); }
  void Backward(float scale, const float* w = nullptr, double d = 0.0) { e->Backward(scale, w, d); }
  void ZeroGrad() { e->ZeroGrad(); }
  const std::vector<float>& losses() const { return e->losses(); }
  const std::vector<float>& logits() const { return e->logits(); }
  std::int64_t valid_targets() const { return e->valid_targets(); }
};
struct DeviceOptimView {
  DeviceEngine* e;
  void Step(int step) { e->OptimStep(step); }
};

}  // namespace ncb
