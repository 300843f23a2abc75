// Single-client multi-replica runtime of the native CPU engine, and the training driver on top of it.
//
// A `MeshRuntime` owns one model replica (and optimizer) per mesh position, one worker thread per replica. A step
// splits one global batch over the replicas, each replica runs its micro-batches with the backward scaled by
// 1 / (grad_accum * world), the gradients are summed with the ring all-reduce over in-process mailboxes, and every
// replica takes the same optimizer step, so the replicas stay bit-identical. This is the reference's in-process
// "mesh" data parallelism (src/mesh_runtime.cc:112-220, src/mesh_collective.cc, include/nanochat/mesh.h: a rank-1
// "data" axis) and its driver (src/mesh_train.cc). The GPU path of this framework runs one process per GPU instead
// and does not go through this class.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "collective.h"
#include "engine.h"

namespace ncb {

// A rank-1 mesh: the device index at each position of the single "data" axis.
struct MeshSpec {
  std::vector<int> devices;
  int size() const { return static_cast<int>(devices.size()); }
};

struct MeshMetrics {
  std::vector<float> loss;  // per replica, mean over its micro-batches
  float grad_norm = 0.0f;   // after the reduce: identical on every replica
  float step_seconds = 0.0f;
};

class MeshRuntime {
 public:
  // `batch`: global batch in sequences per step (divisible by world * grad_accum); `seq` 0 selects cfg.seq_len.
  MeshRuntime(const MeshSpec& mesh, const EngineConfig& cfg, const OptimConfig& optim, int batch, int grad_accum,
              int seq, std::uint64_t seed, std::string* error);
  ~MeshRuntime();
  bool ok() const { return ok_; }
  int world() const { return static_cast<int>(replicas_.size()); }
  int batch() const { return batch_; }
  int seq() const { return seq_; }
  int step() const { return step_; }
  // One step over [batch, seq] row-major ids. Returns the global mean loss; on a lost replica sets `error`.
  float TrainStep(const int* tokens, const int* targets, std::string* error);
  const MeshMetrics& metrics() const { return metrics_; }
  CpuModel* replica(int r) { return r >= 0 && r < world() ? replicas_[r].model.get() : nullptr; }
  std::uint64_t ParamDigest(int replica) const;  // FNV-1a 64 over the fp32 bytes of every parameter in order
  bool Save(const std::string& path, std::string* error) const;          // replica 0, with optimizer state and step
  bool Load(const std::string& path, std::string* error);               // every replica; restores state and step
  bool LoadWeights(const std::string& path, std::string* error);        // parameters only
  // Test hook: the next step's first message from replica `from` to its ring neighbour is dropped, so the
  // neighbour's receive times out (`timeout_ms` bounds every receive of the gradient reduce).
  void InjectDrop(int from);
  void set_timeout_ms(int ms) { timeout_ms_ = ms; }

 private:
  struct Replica {
    std::unique_ptr<CpuModel> model;
    std::unique_ptr<CpuOptimizer> optim;
    std::unique_ptr<Transport> link;
  };
  bool ok_ = false;
  int batch_, accum_, seq_, step_ = 0, timeout_ms_ = 60000;
  std::unique_ptr<MemoryHub> hub_;
  std::vector<Replica> replicas_;
  MeshMetrics metrics_;
};

struct MeshTrainConfig {
  EngineConfig model;
  MeshSpec mesh;
  OptimConfig optim;
  std::string warm_start_path;
  double flops_per_token = 0.0, peak_flops = 0.0;
  std::vector<std::string> parquet;
  std::string tokenizer_path, packed_rows_path;
  std::uint64_t data_seed = 0;
  int batch = 8, grad_accum = 1, seq = 0;
  std::uint64_t seed = 42;
  int num_iterations = 10, log_every = 0, save_every = 0;
  bool resume = false;
  std::string out_dir, checkpoint_path;
};

struct MeshTrainSummary {
  int steps = 0;
  bool interrupted = false;
  double mean_loss = 0.0, steady_mfu = 0.0;
  std::string checkpoint;
};

// The driver: owns the loader, the step loop, `metrics.jsonl`, `summary.json`, the checkpoint interval and the
// resume; stops cleanly (with a checkpoint) on SIGINT. Returns the last loss, 0 on error.
float RunMeshTrain(const MeshTrainConfig& config, MeshTrainSummary* out, std::string* error);

// One rank of a multi-process data-parallel CPU job (the reference's `nanochat_cli train --rank R --world-size W`,
// src/train.cc:628-724: backward scaled by 1 / (grad_accum * world), gradients summed over the ranks, every rank
// takes the same optimizer step; rank 0 writes the checkpoint and the metrics). `config.batch` is the per-rank
// micro-batch here. Ranks meet through `RendezvousAndConnect` on 127.0.0.1:`port` and reduce with the TCP ring.
struct DistConfig {
  int rank = 0, world = 1, port = 29500, timeout_ms = 600000;
};
float RunDistributedTrain(const MeshTrainConfig& config, const DistConfig& dist, MeshTrainSummary* out,
                          std::string* error);

// 6 * matmul parameters + 12 * layers * heads * head_dim * mean visible keys (the usual estimate).
double EstimateFlopsPerToken(const EngineConfig& cfg);

}  // namespace ncb
