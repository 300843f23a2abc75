// Definitions of the opaque handles of the C ABI (shared by the capi*.cc files).
#pragma once
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include "core.h"
#include "device_engine.h"
#include "nanochat/capi.h"

struct nanochat_tokenizer {
  std::unique_ptr<ncb::Tokenizer> tok;
};
struct nanochat_loader {
  std::unique_ptr<ncb::DataLoader> loader;
  nanochat_tokenizer* tok = nullptr;  // not owned
  int batch = 0, seq = 0;
};
struct nanochat_checkpoint {
  ncb::Checkpoint ck;
  std::vector<nanochat_record> records, optimizer;
  std::vector<std::vector<nanochat_record>> attr_store;
  std::string config_json;
  std::vector<const char*> note_ptrs;
};

void ncb_set_error(const std::string& msg);

// The GPU engine library (libnanochat_gpu.so beside this library), opened on first use; null when it is not there
// or cannot be loaded. `ncb_selected_cuda_device` is the CUDA ordinal models are created on, or -1 for the CPU.
struct ncb_gpu_library {
  ncb::ncb_gpu_device_count_fn device_count = nullptr;
  ncb::ncb_gpu_device_at_fn device_at = nullptr;
  ncb::ncb_gpu_engine_create_fn create = nullptr;
};
const ncb_gpu_library* ncb_gpu();
bool ncb_select_device(const std::string& name, std::string* error);
int ncb_selected_cuda_device();
// Process-wide override of the sliding window of `S` layers (0: ceil(seq/4/128)*128), applied to every model the
// C ABI creates afterwards; `nanochat_config` keeps the reference's layout and has no field for it.
int& ncb_short_window_override();

inline ncb::ModelConfig ncb_to_model_config(const nanochat_config& c) {
  ncb::ModelConfig m;
  m.num_layers = c.num_layers, m.num_heads = c.num_heads, m.num_kv_heads = c.num_kv_heads;
  m.hidden_dim = c.hidden_dim, m.seq_len = c.seq_len, m.vocab_size = c.vocab_size;
  m.padded_vocab_size = c.padded_vocab_size;
  m.rope_base = c.rope_base;
  m.window_pattern = c.window_pattern != nullptr ? c.window_pattern : "";
  m.value_embedding = c.value_embedding != 0;
  return m;
}
