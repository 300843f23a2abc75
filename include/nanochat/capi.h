/* Flat C ABI of the host runtime and the CPU engine (libnanochat_core.so).
 *
 * Names, struct layouts and conventions follow the reference's include/nanochat/capi.h so that a client
 * written against it links unchanged: status code + thread-local error string, opaque handles, caller-owned
 * output buffers. Functions that exist only here are prefixed `ncb_`. */
#ifndef NANOCHAT_CAPI_H_
#define NANOCHAT_CAPI_H_
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef enum { NANOCHAT_STATUS_OK = 0, NANOCHAT_STATUS_ERROR = 1 } nanochat_status;

typedef struct nanochat_model nanochat_model;
typedef struct nanochat_optim nanochat_optim;
typedef struct nanochat_loader nanochat_loader;
typedef struct nanochat_tokenizer nanochat_tokenizer;
typedef struct nanochat_checkpoint nanochat_checkpoint;

typedef struct {
  int num_layers, num_heads, num_kv_heads, hidden_dim, seq_len, vocab_size, padded_vocab_size;
  float rope_base;
  const char* window_pattern;
  int value_embedding;
} nanochat_config;

typedef struct {
  int64_t total, transformer_matrices, lm_head, embeddings, scalars;
  double flops_per_token;
} nanochat_params;

typedef struct {
  int device_index, compute_major, compute_minor;
  int64_t total_memory_bytes;
  const char* device_name;
} nanochat_device;

typedef struct {
  const char* name;
  void* value;
  void* grad;
  int64_t count;
  int rows, cols;
} nanochat_param;

typedef struct {
  int position;
  const int* ids;
  int count;
} nanochat_focus;

typedef struct {
  const float* nll;
  const int* argmax;
  const float* focus_logits;
} nanochat_score_result;

typedef struct {
  int num_samples, max_tokens;
  float temperature;
  int top_k;
  uint64_t seed;
  int stop_id, bos_id;
  const int* stop_ids;
} nanochat_generate_params;

typedef struct {
  int count;
  const int* tokens;
  const uint8_t* mask;
  const int* lengths;
  const int* offsets;
} nanochat_sequences;

typedef struct {
  int num_prompts, prompt_len;
  const int* row_stops;
  nanochat_generate_params params;
} nanochat_generate_multi_params;

typedef struct {
  float unembedding_lr, embedding_lr, matrix_lr, scalar_lr, weight_decay;
  int muon_ns_steps;
  float muon_beta2, adam_eps, clip;
  int num_iterations, warmup_steps;
  float warmdown_ratio, final_lr_frac, weight_decay_base;
  float muon_momentum_warmup_steps, muon_momentum_start, muon_momentum_peak, muon_momentum_final;
} nanochat_optim_config;

size_t nanochat_optim_config_size(void);
nanochat_status nanochat_init(void);
const char* nanochat_last_error(void);
const char* nanochat_version(void);
const char* nanochat_backend(void);
int nanochat_compute_type_size(void);
void nanochat_device_info(nanochat_device* out);
int nanochat_device_count(void);
/* Backend selection at run time (the reference fixes it at link time): "cpu" (default), "cuda" or "cuda:N". The
 * environment variable NANOCHAT_DEVICE gives the initial choice. After a CUDA device is selected, `nanochat_backend`
 * answers "cuda", `nanochat_device_count/_at` enumerate the CUDA devices, and every model created afterwards (and
 * its optimizer, scoring, generation and evaluation calls) runs on that device through the sm_100a kernels of
 * libnanochat_gpu.so, which must sit beside this library. `nanochat_param_info` then returns null data pointers:
 * use nanochat_param_read / nanochat_param_write. The in-process mesh runtime stays on the CPU engine. */
nanochat_status nanochat_select_device(const char* name);
/* First bounded-wait failure a kernel recorded on the model's device (0 = none; always 0 on the CPU), and the number
 * of kernel launches the model's engine has issued. */
/* One micro-batch: forward + backward with the gradients accumulated times `scale` (no zeroing, no optimizer step);
 * on a CUDA device the LM head runs once, fused forward and backward. Returns the micro-batch loss. */
float ncb_forward_backward(nanochat_model* model, const int* tokens, const int* targets, int batch, int seq, float scale);
int ncb_model_device_status(nanochat_model* model);
int64_t ncb_model_launch_count(nanochat_model* model);
/* An activation kept by the model's last forward on a CUDA device ("emb", "x0", "xn"; per layer "xr", "h", "qkv", "qk",
 * "attn", "x_mid", "h2", "act", "x_out"), widened to fp32: for comparing engines stage by stage. Returns the element
 * count (the copy is truncated to `capacity`), -1 for an unknown name or a model on the CPU. */
int64_t ncb_model_read_activation(nanochat_model* model, const char* name, int layer, float* dst, int64_t capacity);
int nanochat_device_at(int ordinal, nanochat_device* out);

nanochat_status nanochat_params_get(const nanochat_config* config, nanochat_params* out);
nanochat_status nanochat_optim_config_preset(const char* name, nanochat_optim_config* out);

/* ---- CPU engine ---------------------------------------------------------------------------------- */
nanochat_model* nanochat_model_create(const nanochat_config* config, uint64_t seed);
void nanochat_model_free(nanochat_model* model);
float nanochat_forward_loss(nanochat_model* model, const int* tokens, const int* targets, int batch, int seq);
void nanochat_backward(nanochat_model* model);
void nanochat_backward_weighted(nanochat_model* model, const float* row_weights, float scale);
void nanochat_backward_accumulate(nanochat_model* model, float scale);
float nanochat_train_step(nanochat_model* model, nanochat_optim* optimizer, const int* tokens, const int* targets,
                          int batch, int seq);
float nanochat_rl_step(nanochat_model* model, nanochat_optim* optimizer, const int* tokens, const int* targets,
                       const float* advantages, int batch, int seq, int num_passes, int examples_per_rank, int step);
void nanochat_zero_grad(nanochat_model* model);
int nanochat_param_count(nanochat_model* model);
int nanochat_param_info(nanochat_model* model, int index, nanochat_param* out);
int64_t nanochat_param_read(nanochat_model* model, int index, int grad, int64_t offset, int64_t count, void* data);
int64_t nanochat_param_write(nanochat_model* model, int index, int grad, int64_t offset, int64_t count,
                             const void* data);
void nanochat_save(nanochat_model* model, const char* path);
void nanochat_load(nanochat_model* model, const char* path);
nanochat_optim* nanochat_optim_create(nanochat_model* model, const nanochat_optim_config* config);
void nanochat_optim_step(nanochat_optim* optimizer, int step);
float nanochat_optim_grad_norm(nanochat_optim* optimizer);
void nanochat_optim_free(nanochat_optim* optimizer);
void nanochat_score_batch(nanochat_model* model, const int* tokens, int batch, int seq, const int* lengths,
                          const nanochat_focus* focus, nanochat_score_result* out);
void nanochat_generate(nanochat_model* model, const int* prompt, int length, const nanochat_generate_params* params,
                       nanochat_sequences* out);
void nanochat_generate_multi(nanochat_model* model, const int* prompts, const nanochat_generate_multi_params* params,
                             nanochat_sequences* out);
float nanochat_eval_bpb(nanochat_model* model, nanochat_loader* loader, int steps);

/* ---- checkpoints ---------------------------------------------------------------------------------- */
typedef struct nanochat_record {
  const char* name;
  int32_t dtype;
  int32_t ndim;
  const int64_t* dims;
  const void* data;
  int64_t bytes;
  int64_t attribute_count;
  const struct nanochat_record* attributes;
} nanochat_record;

typedef enum { NANOCHAT_STAGE_BASE = 0, NANOCHAT_STAGE_SFT = 1, NANOCHAT_STAGE_RL = 2 } nanochat_stage;
typedef enum { NANOCHAT_PRECISION_FP32 = 0, NANOCHAT_PRECISION_BF16 = 1, NANOCHAT_PRECISION_FP8 = 2 } nanochat_precision;

typedef struct {
  int32_t schema;
  int32_t stage;
  int64_t step;
  int64_t world_size;
  int32_t precision;
  const char* config_json;
  const char* tokenizer_id;
  const char* git_revision;
  const char* created_utc;
  const char* const* notes;
  int32_t note_count;
} nanochat_checkpoint_metadata;

nanochat_status nanochat_checkpoint_dtype(int32_t index, const char** name, int32_t* code, int32_t* size);
nanochat_status nanochat_checkpoint_write(const char* path, const nanochat_record* records, int64_t record_count,
                                          const nanochat_record* optimizer, int64_t optimizer_count);
nanochat_status nanochat_checkpoint_read(const char* path, nanochat_checkpoint** owner,
                                         const nanochat_record** records, int64_t* record_count,
                                         const nanochat_record** optimizer, int64_t* optimizer_count);
void nanochat_checkpoint_free(nanochat_checkpoint* owner);
nanochat_status nanochat_checkpoint_metadata_read(const char* path, nanochat_checkpoint** owner,
                                                  nanochat_checkpoint_metadata* out);
int32_t nanochat_checkpoint_metadata_stage(const nanochat_checkpoint_metadata* meta);
int64_t nanochat_checkpoint_metadata_step(const nanochat_checkpoint_metadata* meta);
int64_t nanochat_checkpoint_metadata_world_size(const nanochat_checkpoint_metadata* meta);
const char* nanochat_checkpoint_metadata_config_json(const nanochat_checkpoint_metadata* meta);
/* Record files (fixtures: magic[8], u32 version, u32 count, records). dtype codes: 0 f32, 1 i32, 2 f64, 3 i64, 4 u8.
 * `ncb_record_file_read` keeps the records alive until `ncb_record_file_free(owner)`; `magic` receives 8 characters
 * and a terminating zero. */
typedef struct ncb_record_file ncb_record_file;
nanochat_status ncb_record_file_read(const char* path, ncb_record_file** owner, char magic[9],
                                     const nanochat_record** records, int64_t* record_count);
void ncb_record_file_free(ncb_record_file* owner);
nanochat_status ncb_record_file_write(const char* path, const char* magic, const nanochat_record* records,
                                      int64_t record_count);
/* Same as nanochat_checkpoint_write, with the metadata block of the file given explicitly (JSON config as
 * produced by nanochat_checkpoint_metadata_config_json). */
nanochat_status ncb_checkpoint_write_meta(const char* path, const nanochat_record* records, int64_t record_count,
                                          const nanochat_record* optimizer, int64_t optimizer_count,
                                          const nanochat_config* config, int32_t stage, int64_t step,
                                          int64_t world_size, int32_t precision, const char* tokenizer_id,
                                          const char* notes);

/* ---- data ------------------------------------------------------------------------------------------ */
nanochat_loader* nanochat_loader_create(const char** parquet, int count, const char* text_column,
                                        nanochat_tokenizer* tokenizer, int batch, int seq, uint64_t seed,
                                        int tokenizer_threads, size_t document_buffer);
int nanochat_loader_next(nanochat_loader* loader, int* tokens, int* targets);
const uint8_t* nanochat_loader_token_bytes(nanochat_loader* loader, int* vocab);
void nanochat_loader_free(nanochat_loader* loader);
/* Loaders over other sources: token documents given directly (offsets has count + 1 entries), a text file with
 * one document per line, or a synthetic Zipf(s) stream. rank/world select every world-th document. */
nanochat_loader* ncb_loader_from_documents(const int* tokens, const int64_t* offsets, int64_t count, int batch,
                                           int seq, size_t document_buffer, int rank, int world);
nanochat_loader* ncb_loader_from_text(const char* path, nanochat_tokenizer* tokenizer, int batch, int seq,
                                      size_t document_buffer, int rank, int world);
nanochat_loader* ncb_loader_zipf(int vocab, int doc_len, double s, uint64_t seed, int batch, int seq,
                                 size_t document_buffer);
nanochat_status ncb_loader_save_cursor(nanochat_loader* loader, const char* path);
nanochat_status ncb_loader_load_cursor(nanochat_loader* loader, const char* path);
uint64_t ncb_loader_epoch(nanochat_loader* loader);

nanochat_tokenizer* nanochat_tokenizer_load(const char* path);
int nanochat_encode(nanochat_tokenizer* tokenizer, const char* text, int* out, int capacity);
int nanochat_decode(nanochat_tokenizer* tokenizer, const int* ids, int count, char* out, int capacity);
void nanochat_tokenizer_free(nanochat_tokenizer* tokenizer);
int ncb_tokenizer_vocab_size(nanochat_tokenizer* tokenizer);
int ncb_tokenizer_special_id(nanochat_tokenizer* tokenizer, const char* name);
int ncb_encode_n(nanochat_tokenizer* tokenizer, const char* text, int64_t length, int prepend, int append, int* out,
                 int capacity);
nanochat_status ncb_tokenizer_save(nanochat_tokenizer* tokenizer, const char* path);
/* Trains a tokenizer on a text file (one document per line) or one parquet column. */
nanochat_tokenizer* ncb_tokenizer_train(const char* text_path, const char* parquet_path, const char* text_column,
                                        int vocab_size, int64_t doc_cap, int64_t max_chars);
/* Splits text with the fixed pattern; writes piece end offsets (bytes). Returns the number of pieces. */
int ncb_split_pattern(const char* text, int64_t length, int64_t* ends, int capacity);
/* Reads one string column of a parquet file; returns the row count and fills offsets/bytes when given. */
int64_t ncb_parquet_read(const char* path, const char* column, char* bytes, int64_t byte_capacity, int64_t* offsets,
                         int64_t offset_capacity, int64_t* total_bytes);
/* Sampling with the per-row streams of the native generation loop: row `row_ids[r]` draws from
 * Rng(MixSeed(seed, row_ids[r])), one draw per sampled position; `draw_index` is the position's index. `logits`:
 * [rows, vocab] fp32 (soft-capped). Greedy when temperature <= 0. */
void ncb_sample_rows(const float* logits, int rows, int vocab, float temperature, int top_k, uint64_t seed,
                     const int64_t* row_ids, int64_t draw_index, int* out);
int ncb_sample_token(const float* logits, int vocab, float temperature, int top_k, uint64_t seed, uint64_t row,
                     uint64_t step);


/* ---- in-process mesh runtime (CPU engine): one model replica per mesh position, gradients summed with a ring
 * all-reduce inside the process, one optimizer step per replica; names and layouts follow the reference. */
typedef struct nanochat_mesh nanochat_mesh;
typedef struct nanochat_runtime nanochat_runtime;
nanochat_mesh* nanochat_mesh_create(const int* indices, int count); /* count < 1 becomes 1; null = 0, 1, ... */
void nanochat_mesh_free(nanochat_mesh* mesh);
int nanochat_mesh_size(nanochat_mesh* mesh);
/* `batch`: global batch in sequences (a multiple of mesh size * grad_accum); `seq` 0 selects config.seq_len. */
nanochat_runtime* nanochat_runtime_create(const nanochat_mesh* mesh, const nanochat_config* config,
                                          const nanochat_optim_config* optim, int batch, int grad_accum, int seq,
                                          uint64_t seed);
void nanochat_runtime_free(nanochat_runtime* runtime);
int nanochat_runtime_world_size(nanochat_runtime* runtime);
/* One step over batch * seq row-major ids; returns the global mean loss, 0 on error. */
float nanochat_runtime_train_step(nanochat_runtime* runtime, const int* tokens, const int* targets);
typedef struct {
  int device_count;
  const float* loss; /* device_count per-replica losses; valid until the next step */
  float grad_norm;
  float step_seconds;
} nanochat_metrics;
nanochat_status nanochat_runtime_metrics(nanochat_runtime* runtime, nanochat_metrics* out);
int nanochat_runtime_param_count(nanochat_runtime* runtime, int replica);
int nanochat_runtime_param_info(nanochat_runtime* runtime, int replica, int index, nanochat_param* out);
int64_t nanochat_runtime_param_read(nanochat_runtime* runtime, int replica, int index, int grad, int64_t offset,
                                    int64_t count, void* data);
/* FNV-1a 64 over the fp32 bytes of every parameter of the replica. */
nanochat_status nanochat_runtime_param_digest(nanochat_runtime* runtime, int replica, uint64_t* out);
void nanochat_runtime_save(nanochat_runtime* runtime, const char* path);         /* replica 0, optimizer + step */
void nanochat_runtime_load(nanochat_runtime* runtime, const char* path);         /* every replica */
void nanochat_runtime_load_weights(nanochat_runtime* runtime, const char* path); /* parameters only */
int nanochat_runtime_step(nanochat_runtime* runtime);
/* Failure-detection test hook: the next step's first ring message from replica `from` is dropped and every
 * receive of the reduce is bounded by `timeout_ms`; the step then fails with an error instead of hanging. */
void ncb_runtime_inject_drop(nanochat_runtime* runtime, int from, int timeout_ms);

typedef struct {
  const char* const* parquet;
  int parquet_count;
  const char* tokenizer_path;
  const char* packed_rows_path; /* an NCSFT001 shard; empty selects parquet */
  uint64_t data_seed;
} nanochat_mesh_data_config;
typedef struct {
  int batch, grad_accum, seq;
  uint64_t seed;
  int num_iterations, log_every, save_every, resume;
} nanochat_mesh_run_config;
typedef struct {
  const char* out_dir;
  const char* checkpoint_path; /* empty selects out_dir/checkpoint.ckpt */
} nanochat_mesh_output_config;
typedef struct {
  nanochat_config model;
  const nanochat_mesh* mesh;
  const char* preset; /* "default" or "track3"; ignored when `optimizer` is given */
  const nanochat_optim_config* optimizer;
  const char* warm_start_path;
  double flops_per_token; /* 0: the model estimate */
  double peak_flops;      /* 0: MFU is reported as 0 */
  nanochat_mesh_data_config data;
  nanochat_mesh_run_config run;
  nanochat_mesh_output_config output;
} nanochat_mesh_train_config;
typedef struct {
  int steps;
  int interrupted;
  double mean_loss;
  double steady_mfu;
  char checkpoint[4096];
} nanochat_mesh_train_summary;
/* Runs one job: metrics.jsonl, summary.json and the checkpoint under out_dir; SIGINT stops it with a checkpoint.
 * Returns the last loss, 0 on error. */
float nanochat_mesh_train_run(const nanochat_mesh_train_config* config, nanochat_mesh_train_summary* out);

/* Sliding window (tokens to the left) of `S` layers for every model created afterwards; 0 = ceil(seq/4/128)*128. */
void ncb_set_short_window(int tokens);

/* ---- performance model: analytic roofline of one training step as `nanochat.roofline.v3` JSON (or a text table).
 * `device`: b200 | h100 | t4 | cpu; measured_* > 0 override the B200 peaks. Returns the text length, negative on error. */
int64_t ncb_roofline(const nanochat_config* config, const char* device, const char* precision, int batch, int grad_accum,
                     int world_size, int64_t total_tokens, double link_gbps, double latency_us, double overlap,
                     int muon_ns_steps, double measured_bf16_tflops, double measured_hbm_gbs, int as_table, char* out,
                     int64_t capacity);
double ncb_muon_flops_per_step(const nanochat_config* config, int ns_steps);

/* ---- planning layer (host only): model specification + device declaration -> operator plan; training-run plan.
 * `ncb_plan_json`: `spec_path` is a closed JSON model specification (unknown keys are errors), `caps_path` a device
 * declaration (`caps/<device>.json`); the result is `nanochat.plan.v1` JSON with one row per operation family
 * (`kernel` when the device declares the family's capability, else `composition`). A device that lacks a capability
 * the model requires is an error that names it. `graph`: train | prefill | decode | generate | eval.
 * `ncb_train_plan_json`: horizon, batch size, learning-rate and weight-decay scaling for a depth (hidden = depth *
 * aspect_ratio rounded to head_dim); `total_batch_size` -1 asks for the predicted optimum. Both return the text
 * length (the text is truncated to `capacity - 1`), negative on error. */
int64_t ncb_plan_json(const char* spec_path, const char* caps_path, const char* precision, const char* graph, char* out,
                      int64_t capacity);
nanochat_status ncb_spec_config(const char* spec_path, nanochat_config* out, char* pattern, int pattern_capacity);
int64_t ncb_train_plan_json(int depth, int aspect_ratio, int head_dim, int seq_len, int vocab_size,
                            int device_batch_size, const char* window_pattern, int64_t total_batch_size,
                            int64_t num_iterations, double target_flops, int target_param_data_ratio, char* out,
                            int64_t capacity);
double ncb_prefill_flops(const nanochat_config* config, int prompt_tokens);
double ncb_decode_flops_per_token(const nanochat_config* config, int context_tokens);

/* One rank of a multi-process CPU data-parallel job (TCP ring over 127.0.0.1, rendezvous on `port`): the same
 * config as the mesh driver, `run.batch` is the per-rank micro-batch, `mesh` is ignored. Rank 0 writes the artifacts. */
float ncb_dist_train_run(const nanochat_mesh_train_config* config, int rank, int world, int port, int timeout_ms,
                         nanochat_mesh_train_summary* out);

/* ---- host collectives (TCP over 127.0.0.1 between CPU ranks; an in-process ring for tests) */
typedef struct ncb_tcp ncb_tcp;
ncb_tcp* ncb_tcp_create(int rank, int world);
int ncb_tcp_port(ncb_tcp* transport);
nanochat_status ncb_tcp_connect(ncb_tcp* transport, const int* ports, int count, int timeout_ms);
nanochat_status ncb_tcp_all_reduce_sum(ncb_tcp* transport, float* data, int64_t count, int timeout_ms);
void ncb_tcp_free(ncb_tcp* transport);
nanochat_status ncb_memory_ring_all_reduce(float* data, int world, int64_t count, int drop_from, int timeout_ms);

#ifdef __cplusplus
}
#endif
#endif /* NANOCHAT_CAPI_H_ */
