// CPU engine: parameters, forward, backward, inference. See engine.h.
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <chrono>
#if defined(__GLIBC__)
#include <malloc.h>
#endif
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>

namespace ncb {

namespace {

constexpr float kRmsEps = 1.1920929e-07f;  // fp32 epsilon
constexpr float kSoftcap = 15.0f;
constexpr float kQkScale = 1.2f;
constexpr int kGateCh = 12;
constexpr int kSmearCh = 24;
constexpr std::size_t kAlign = 64;

// The three products below carry the model's FLOPs. Inner loops are written so that the compiler vectorizes them
// (float lanes, folded into a double every 256 elements, which keeps the 1e-5 agreement with the fp64-accumulating
// oracle), are cloned for AVX2+FMA / AVX-512 with run-time dispatch, and rows are spread over OpenMP threads.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__) && !defined(__SANITIZE_THREAD__) && \
    !defined(__SANITIZE_ADDRESS__)  // ifunc resolvers run before a sanitizer runtime is up
#define NCB_SIMD_CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))
#else
#define NCB_SIMD_CLONES
#endif

// Wall-clock totals per named section of the CPU engine, printed at exit when NANOCHAT_CPU_PROFILE=1 (the CPU
// engine's counterpart of the per-operator profile of the GPU path).
class SectionTimer {
 public:
  explicit SectionTimer(const char* name) : name_(Enabled() ? name : nullptr) {
    if (name_ != nullptr) start_ = std::chrono::steady_clock::now();
  }
  ~SectionTimer() {
    if (name_ == nullptr) return;
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start_).count();
    Table& t = table();
    std::lock_guard<std::mutex> lock(t.mu);
    auto& e = t.rows[name_];
    e.first += ms;
    e.second += 1;
  }
  static bool Enabled() {
    static const bool on = [] {
      const char* e = std::getenv("NANOCHAT_CPU_PROFILE");
      return e != nullptr && e[0] == '1';
    }();
    return on;
  }

 private:
  struct Table {
    std::mutex mu;
    std::map<std::string, std::pair<double, long>> rows;
    ~Table() {
      if (rows.empty()) return;
      std::fprintf(stderr, "[cpu engine] section                 total ms    calls\n");
      for (const auto& r : rows)
        std::fprintf(stderr, "[cpu engine] %-22s %10.1f %8ld\n", r.first.c_str(), r.second.first, r.second.second);
    }
  };
  static Table& table() {
    static Table t;
    return t;
  }
  const char* name_;
  std::chrono::steady_clock::time_point start_;
};

NCB_SIMD_CLONES double Dot(const float* a, const float* b, int n) {
  double total = 0.0;
  for (int i0 = 0; i0 < n; i0 += 256) {
    const int i1 = std::min(n, i0 + 256);
    float part = 0.0f;
#pragma omp simd reduction(+ : part)
    for (int i = i0; i < i1; ++i) part += a[i] * b[i];
    total += part;
  }
  return total;
}
NCB_SIMD_CLONES void Axpy(float g, const float* x, float* y, int n) {
#pragma omp simd
  for (int i = 0; i < n; ++i) y[i] += g * x[i];
}

// C[M,N] (+)= A[M,K] B[K,N], all row-major: the one product every linear layer and the Newton-Schulz iteration
// reduce to. The micro-kernel keeps a 6 x 32 block of C in twelve 16-float accumulators and walks K with one
// broadcast of A per row and two loads of B per step (12 multiply-adds per 2 loads, no horizontal sums). K is cut
// into chunks of 256 whose float sums are added to C one after the other, which bounds the rounding error the way
// the per-256 folding of Dot does. Panels of 32 columns of B stay in cache while the row blocks of A stream past.
typedef float Vf16 __attribute__((vector_size(64), aligned(4), may_alias));   // 16 floats, unaligned access allowed

template <int MR>
NCB_SIMD_CLONES void Micro32(const float* A, std::size_t lda, const float* B, std::size_t ldb, float* C,
                             std::size_t ldc, int K, bool accumulate) {
  Vf16 total[MR][2];
  for (int r = 0; r < MR; ++r)
    for (int h = 0; h < 2; ++h)
      total[r][h] = accumulate ? *reinterpret_cast<const Vf16*>(C + r * ldc + 16 * h) : Vf16{};
  for (int k0 = 0; k0 < K; k0 += 256) {
    const int k1 = std::min(K, k0 + 256);
    Vf16 acc[MR][2];
    for (int r = 0; r < MR; ++r) acc[r][0] = Vf16{}, acc[r][1] = Vf16{};
    for (int k = k0; k < k1; ++k) {
      const Vf16 b0 = *reinterpret_cast<const Vf16*>(B + k * ldb), b1 = *reinterpret_cast<const Vf16*>(B + k * ldb + 16);
      for (int r = 0; r < MR; ++r) {
        const float a = A[r * lda + k];     // scalar * vector: the compiler broadcasts
        acc[r][0] += a * b0;
        acc[r][1] += a * b1;
      }
    }
    for (int r = 0; r < MR; ++r) total[r][0] += acc[r][0], total[r][1] += acc[r][1];
  }
  for (int r = 0; r < MR; ++r)
    for (int h = 0; h < 2; ++h) *reinterpret_cast<Vf16*>(C + r * ldc + 16 * h) = total[r][h];
}

// Columns past the last panel of 32 (and any shape too small for a panel): plain loops, same chunking of K.
void GemmEdge(const float* A, std::size_t lda, const float* B, std::size_t ldb, float* C, std::size_t ldc, int m0,
              int m1, int n0, int n1, int K, bool accumulate) {
  for (int m = m0; m < m1; ++m)
    for (int n = n0; n < n1; ++n) {
      float total = accumulate ? C[m * ldc + n] : 0.0f;
      for (int k0 = 0; k0 < K; k0 += 256) {
        float part = 0.0f;
        for (int k = k0; k < std::min(K, k0 + 256); ++k) part += A[m * lda + k] * B[k * ldb + n];
        total += part;
      }
      C[m * ldc + n] = total;
    }
}

void GemmNN(const float* A, std::size_t lda, const float* B, std::size_t ldb, float* C, std::size_t ldc, int M, int N,
            int K, bool accumulate) {
  const int panels = N / 32, blocks = (M + 5) / 6;
  const long long work = static_cast<long long>(M) * N * K;
#pragma omp parallel for collapse(2) schedule(static) if (work > 200000)
  for (int p = 0; p < panels; ++p)
    for (int b = 0; b < blocks; ++b) {
      const int m = b * 6, n = p * 32, rows = std::min(6, M - m);
      const float* a = A + m * lda;
      const float* bp = B + n;
      float* c = C + m * ldc + n;
      switch (rows) {
        case 6: Micro32<6>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
        case 5: Micro32<5>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
        case 4: Micro32<4>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
        case 3: Micro32<3>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
        case 2: Micro32<2>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
        default: Micro32<1>(a, lda, bp, ldb, c, ldc, K, accumulate); break;
      }
    }
  if (panels * 32 < N) GemmEdge(A, lda, B, ldb, C, ldc, 0, M, panels * 32, N, K, accumulate);
}

void TransposeInto(const float* src, int rows, int cols, std::vector<float>* dst) {   // dst[cols, rows]
  dst->resize(static_cast<std::size_t>(rows) * cols);
  float* d = dst->data();
#pragma omp parallel for schedule(static) if (static_cast<long long>(rows) * cols > 65536)
  for (int c0 = 0; c0 < cols; c0 += 32)
    for (int r = 0; r < rows; ++r)
      for (int c = c0; c < std::min(cols, c0 + 32); ++c)
        d[static_cast<std::size_t>(c) * rows + r] = src[static_cast<std::size_t>(r) * cols + c];
}

// y[M,N] = x[M,K] w[N,K]^T (+ residual)
void Linear(const float* x, const float* w, float* y, int M, int N, int K, const float* residual = nullptr) {
  if (M == 1) {   // one token (decoding): dot products straight over the rows of w, nothing to transpose
#pragma omp parallel for schedule(static) if (static_cast<long long>(N) * K > 200000)
    for (int n = 0; n < N; ++n)
      y[n] = static_cast<float>(Dot(x, w + static_cast<std::size_t>(n) * K, K)) + (residual ? residual[n] : 0.0f);
    return;
  }
  std::vector<float> wt;
  TransposeInto(w, N, K, &wt);   // [K, N]
  GemmNN(x, K, wt.data(), N, y, N, M, N, K, false);
  if (residual != nullptr) Axpy(1.0f, residual, y, M * N);
}
// dx[M,K] (+)= dy[M,N] w[N,K]
void LinearDgrad(const float* dy, const float* w, float* dx, int M, int N, int K, bool accumulate) {
  GemmNN(dy, N, w, K, dx, K, M, K, N, accumulate);
}
// gw[N,K] += dy[M,N]^T x[M,K]
void LinearWgrad(const float* dy, const float* x, float* gw, int M, int N, int K) {
  std::vector<float> dyt;
  TransposeInto(dy, M, N, &dyt);   // [N, M]
  GemmNN(dyt.data(), M, x, K, gw, K, N, K, M, true);
}

// y = x * rstd per row; rstd = 1/sqrt(mean(x^2) + eps)
void RmsNorm(const float* x, float* y, float* rstd, int M, int C) {
  for (int m = 0; m < M; ++m) {
    const float* xr = x + static_cast<std::size_t>(m) * C;
    double ss = 0.0;
    for (int c = 0; c < C; ++c) ss += static_cast<double>(xr[c]) * xr[c];
    const float r = 1.0f / std::sqrt(static_cast<float>(ss) * (1.0f / C) + kRmsEps);
    if (rstd) rstd[m] = r;
    float* yr = y + static_cast<std::size_t>(m) * C;
    for (int c = 0; c < C; ++c) yr[c] = xr[c] * r;
  }
}
// dx = rstd*dy - rstd^3 * dot(x,dy)/C * x (+ residual)
void RmsNormBwd(const float* x, const float* dy, const float* rstd, float* dx, int M, int C,
                const float* residual = nullptr) {
  for (int m = 0; m < M; ++m) {
    const float* xr = x + static_cast<std::size_t>(m) * C;
    const float* gr = dy + static_cast<std::size_t>(m) * C;
    double dot = 0.0;
    for (int c = 0; c < C; ++c) dot += static_cast<double>(xr[c]) * gr[c];
    const float r = rstd[m];
    const float coeff = r * r * r * static_cast<float>(dot) * (1.0f / C);
    float* out = dx + static_cast<std::size_t>(m) * C;
    for (int c = 0; c < C; ++c) {
      const float v = r * gr[c] - coeff * xr[c];
      out[c] = residual ? v + residual[static_cast<std::size_t>(m) * C + c] : v;
    }
  }
}

void BuildRope(int seq, int head_dim, float base, int offset, std::vector<float>* cosv, std::vector<float>* sinv) {
  const int half = head_dim / 2;
  cosv->resize(static_cast<std::size_t>(seq) * half);
  sinv->resize(static_cast<std::size_t>(seq) * half);
  for (int d = 0; d < half; ++d) {
    const float inv_freq = 1.0f / std::pow(base, (2.0f * d) / static_cast<float>(head_dim));
    for (int t = 0; t < seq; ++t) {
      const float ang = static_cast<float>(t + offset) * inv_freq;
      (*cosv)[static_cast<std::size_t>(t) * half + d] = std::cos(ang);
      (*sinv)[static_cast<std::size_t>(t) * half + d] = std::sin(ang);
    }
  }
}

// per-head RMSNorm -> rotate (half split) -> scale; x, y: [M, heads*D] rows, position of row m is pos[m]
void QkPrep(const float* x, float* y, int M, int heads, int D, const float* cosv, const float* sinv, const int* pos) {
  const int half = D / 2;
  for (int m = 0; m < M; ++m) {
    const float* c = cosv + static_cast<std::size_t>(pos[m]) * half;
    const float* s = sinv + static_cast<std::size_t>(pos[m]) * half;
    for (int h = 0; h < heads; ++h) {
      const float* xr = x + (static_cast<std::size_t>(m) * heads + h) * D;
      float* yr = y + (static_cast<std::size_t>(m) * heads + h) * D;
      double ss = 0.0;
      for (int d = 0; d < D; ++d) ss += static_cast<double>(xr[d]) * xr[d];
      const float r = 1.0f / std::sqrt(static_cast<float>(ss) * (1.0f / D) + kRmsEps);
      for (int d = 0; d < half; ++d) {
        const float x1 = xr[d] * r, x2 = xr[d + half] * r;
        yr[d] = (x1 * c[d] + x2 * s[d]) * kQkScale;
        yr[d + half] = (-x1 * s[d] + x2 * c[d]) * kQkScale;
      }
    }
  }
}
void QkPrepBwd(const float* pre, const float* grad, float* out, int M, int heads, int D, const float* cosv,
               const float* sinv, const int* pos) {
  const int half = D / 2;
  std::vector<float> g(static_cast<std::size_t>(D));
  for (int m = 0; m < M; ++m) {
    const float* c = cosv + static_cast<std::size_t>(pos[m]) * half;
    const float* s = sinv + static_cast<std::size_t>(pos[m]) * half;
    for (int h = 0; h < heads; ++h) {
      const std::size_t base = (static_cast<std::size_t>(m) * heads + h) * D;
      const float* xr = pre + base;
      const float* gr = grad + base;
      double ss = 0.0, dot = 0.0;
      for (int d = 0; d < half; ++d) {
        g[d] = kQkScale * (gr[d] * c[d] - gr[d + half] * s[d]);
        g[d + half] = kQkScale * (gr[d] * s[d] + gr[d + half] * c[d]);
      }
      for (int d = 0; d < D; ++d) {
        ss += static_cast<double>(xr[d]) * xr[d];
        dot += static_cast<double>(xr[d]) * g[d];
      }
      const float r = 1.0f / std::sqrt(static_cast<float>(ss) * (1.0f / D) + kRmsEps);
      const float coeff = r * r * r * static_cast<float>(dot) * (1.0f / D);
      for (int d = 0; d < D; ++d) out[base + d] = r * g[d] - coeff * xr[d];
    }
  }
}

}  // namespace

int EngineConfig::window_left(int layer) const {
  if (layer >= num_layers - 1 || window_pattern.empty()) return -1;
  return window_pattern[static_cast<std::size_t>(layer) % window_pattern.size()] == 'S' ? short_window() : -1;
}

// ---------------------------------------------------------------------------------------------- model
struct LayerSaved {
  std::vector<float> x, xr, rstd1, q_pre, k_pre, q, k, v, ve, gate, attn, lse, x_mid, rstd2, pre;
};
struct CpuModel::Saved {
  int B = 0, T = 0;
  std::vector<int> tokens, targets, pos;
  std::vector<float> emb_raw, emb, rstd_e, sig, x0, x_last, x_backout, x_pre, rstd_f, xn, cosv, sinv;
  std::vector<LayerSaved> layers;
};

CpuModel::CpuModel(const EngineConfig& cfg) : cfg_(cfg) {
  // Every step allocates (and frees) its activations: tens of MB in blocks of a few MB. glibc serves such blocks
  // with mmap and gives them back on free, so every step would fault all of those pages in again (a third of the
  // step at the small CPU configurations). Keeping them on the heap makes the second step reuse the first one's pages.
  static const bool heap_tuned = [] {
#if defined(__GLIBC__)
    mallopt(M_MMAP_THRESHOLD, 1 << 30);
    mallopt(M_TRIM_THRESHOLD, 1 << 30);
#endif
    return true;
  }();
  (void)heap_tuned;
  const int L = cfg.num_layers, C = cfg.hidden_dim, V = cfg.padded_vocab_size;
  auto add = [&](std::string name, std::vector<std::int64_t> shape, int rows, int cols, ParamKind kind, int layer) {
    CpuParam p;
    p.name = std::move(name), p.shape = std::move(shape), p.rows = rows, p.cols = cols, p.kind = kind, p.layer = layer;
    p.count = 1;
    for (auto d : p.shape) p.count *= static_cast<std::size_t>(d);
    params_.push_back(std::move(p));
  };
  add("lm_head.weight", {V, C}, V, C, ParamKind::kLmHead, -1);
  add("transformer.wte.weight", {V, C}, V, C, ParamKind::kWte, -1);
  for (int i = 0; i < L; ++i)
    if (cfg.has_value_embedding(i))
      add("value_embeds." + std::to_string(i) + ".weight", {V, cfg.kv_dim()}, V, cfg.kv_dim(), ParamKind::kValueEmbed, i);
  add("resid_lambdas", {L}, 0, 0, ParamKind::kResid, -1);
  add("x0_lambdas", {L}, 0, 0, ParamKind::kX0, -1);
  add("smear_gate.weight", {1, kSmearCh}, 1, kSmearCh, ParamKind::kSmear, -1);
  add("smear_lambda", {1}, 0, 0, ParamKind::kSmear, -1);
  add("backout_lambda", {1}, 0, 0, ParamKind::kSmear, -1);
  for (int i = 0; i < L; ++i) {
    const std::string p = "transformer.h." + std::to_string(i) + ".";
    add(p + "attn.c_q.weight", {cfg.query_dim(), C}, cfg.query_dim(), C, ParamKind::kMatrix, i);
    add(p + "attn.c_k.weight", {cfg.kv_dim(), C}, cfg.kv_dim(), C, ParamKind::kMatrix, i);
    add(p + "attn.c_v.weight", {cfg.kv_dim(), C}, cfg.kv_dim(), C, ParamKind::kMatrix, i);
    add(p + "attn.c_proj.weight", {C, C}, C, C, ParamKind::kMatrix, i);
    if (cfg.has_value_embedding(i))
      add(p + "attn.ve_gate.weight", {cfg.num_kv_heads, kGateCh}, cfg.num_kv_heads, kGateCh, ParamKind::kMatrix, i);
    add(p + "mlp.c_fc.weight", {cfg.mlp_dim(), C}, cfg.mlp_dim(), C, ParamKind::kMatrix, i);
    add(p + "mlp.c_proj.weight", {C, cfg.mlp_dim()}, C, cfg.mlp_dim(), ParamKind::kMatrix, i);
  }
  std::size_t off = 0;
  for (auto& p : params_) {
    p.offset = off;
    off += (p.count + kAlign - 1) / kAlign * kAlign;
  }
  value_.assign(off, 0.0f);
  grad_.assign(off, 0.0f);
}

CpuModel::~CpuModel() = default;

const CpuParam* CpuModel::Find(const std::string& name) const {
  for (const auto& p : params_)
    if (p.name == name) return &p;
  return nullptr;
}

void CpuModel::ZeroGrad() { std::fill(grad_.begin(), grad_.end(), 0.0f); }

void CpuModel::InitWeights(std::uint64_t seed) {
  // Distributions of the reference (src/model.cc:427-497); the random stream is this library's xoshiro256**.
  const int L = cfg_.num_layers;
  const float s = std::sqrt(3.0f) / std::sqrt(static_cast<float>(cfg_.hidden_dim));
  const float denom = static_cast<float>(std::max(L - 1, 1));
  std::fill(value_.begin(), value_.end(), 0.0f);
  std::uint64_t stream = 0;
  for (const auto& p : params_) {
    Rng rng(MixSeed(seed, stream++));
    float* v = value(p);
    auto uniform = [&](float lo, float hi) {
      for (std::size_t i = 0; i < p.count; ++i) v[i] = lo + (hi - lo) * rng.NextFloat();
    };
    auto normal = [&](float std_) {
      for (std::size_t i = 0; i < p.count; ++i) v[i] = std_ * static_cast<float>(rng.NextNormal());
    };
    auto ends = [&](const char* suffix) {
      const std::size_t n = std::strlen(suffix);
      return p.name.size() >= n && p.name.compare(p.name.size() - n, n, suffix) == 0;
    };
    if (p.kind == ParamKind::kWte) normal(0.8f);
    else if (p.kind == ParamKind::kLmHead) normal(0.001f);
    else if (p.kind == ParamKind::kValueEmbed) uniform(-s, s);
    else if (p.name == "resid_lambdas") for (int i = 0; i < L; ++i) v[i] = 1.15f - 0.10f * i / denom;
    else if (p.name == "x0_lambdas") for (int i = 0; i < L; ++i) v[i] = 0.20f - 0.15f * i / denom;
    else if (p.name == "smear_gate.weight" || ends("ve_gate.weight")) uniform(0.0f, 0.02f);
    else if (p.name == "smear_lambda") v[0] = 0.0f;
    else if (p.name == "backout_lambda") v[0] = 0.2f;
    else if (ends("c_q.weight") || ends("c_k.weight") || ends("c_v.weight")) uniform(-s, s);
    else if (ends("c_fc.weight")) uniform(-0.4f * s, 0.4f * s);
    // c_proj matrices stay zero
  }
}

// ---------------------------------------------------------------------------------------------- forward
namespace {

// causal / windowed GQA attention over full sequences: q [B,T,H,D], k,v [B,T,KV,D] (token-major rows).
// Scores and the weighted sums run through the vectorised Dot / Axpy (float lanes; the softmax sums fold into
// doubles), one task per (batch, head).
void Attention(const float* q, const float* k, const float* v, float* o, float* lse, int B, int T, int H, int KV,
               int D, int window_left) {
  const int group = H / KV;
  const float scale = 1.0f / std::sqrt(static_cast<float>(D));
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < H; ++h) {
      std::vector<float> sc(static_cast<std::size_t>(T));
      const int kvh = h / group;
      for (int t = 0; t < T; ++t) {
        const float* qr = q + ((static_cast<std::size_t>(b) * T + t) * H + h) * D;
        const int first = window_left < 0 ? 0 : std::max(0, t - window_left);
        float mx = -std::numeric_limits<float>::infinity();
        for (int j = first; j <= t; ++j) {
          const float* kr = k + ((static_cast<std::size_t>(b) * T + j) * KV + kvh) * D;
          sc[j] = static_cast<float>(Dot(qr, kr, D)) * scale;
          mx = std::max(mx, sc[j]);
        }
        double sum = 0.0;
        for (int j = first; j <= t; ++j) {
          sc[j] = std::exp(sc[j] - mx);
          sum += sc[j];
        }
        lse[(static_cast<std::size_t>(b) * H + h) * T + t] = mx + static_cast<float>(std::log(sum));
        const float inv = static_cast<float>(1.0 / sum);
        float* orow = o + ((static_cast<std::size_t>(b) * T + t) * H + h) * D;
        std::fill(orow, orow + D, 0.0f);
        for (int j = first; j <= t; ++j)
          Axpy(sc[j] * inv, v + ((static_cast<std::size_t>(b) * T + j) * KV + kvh) * D, orow, D);
      }
    }
}

void AttentionBwd(const float* q, const float* k, const float* v, const float* o, const float* lse, const float* dout,
                  float* dq, float* dk, float* dv, int B, int T, int H, int KV, int D, int window_left) {
  const int group = H / KV;
  const float scale = 1.0f / std::sqrt(static_cast<float>(D));
  std::fill(dq, dq + static_cast<std::size_t>(B) * T * H * D, 0.0f);
  std::fill(dk, dk + static_cast<std::size_t>(B) * T * KV * D, 0.0f);
  std::fill(dv, dv + static_cast<std::size_t>(B) * T * KV * D, 0.0f);
  // one task per (batch, kv head): the query heads of a group add into the same dK / dV rows
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int kvh = 0; kvh < KV; ++kvh)
      for (int h = kvh * group; h < (kvh + 1) * group; ++h) {
        for (int t = 0; t < T; ++t) {
          const std::size_t qi = ((static_cast<std::size_t>(b) * T + t) * H + h) * D;
          const float* qr = q + qi;
          const float* dor = dout + qi;
          const float delta = static_cast<float>(Dot(dor, o + qi, D));
          const float l = lse[(static_cast<std::size_t>(b) * H + h) * T + t];
          const int first = window_left < 0 ? 0 : std::max(0, t - window_left);
          float* dqr = dq + qi;
          for (int j = first; j <= t; ++j) {
            const std::size_t ki = ((static_cast<std::size_t>(b) * T + j) * KV + kvh) * D;
            const float s = static_cast<float>(Dot(qr, k + ki, D));
            const float dp = static_cast<float>(Dot(dor, v + ki, D));
            const float p = std::exp(s * scale - l);
            const float ds = p * (dp - delta) * scale;
            Axpy(ds, k + ki, dqr, D);
            Axpy(ds, qr, dk + ki, D);
            Axpy(p, dor, dv + ki, D);
          }
        }
      }
}

inline float Sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }

}  // namespace

void CpuModel::Trunk(const int* tokens, int B, int T, Saved* sv, std::vector<float>* xn_out) {
  const EngineConfig& c = cfg_;
  const int M = B * T, C = c.hidden_dim, H = c.num_heads, KV = c.num_kv_heads, D = c.head_dim();
  const int QD = c.query_dim(), KD = c.kv_dim(), F = c.mlp_dim();
  auto P = [&](const std::string& n) { return value(*Find(n)); };
  sv->B = B, sv->T = T;
  sv->tokens.assign(tokens, tokens + M);
  sv->pos.resize(M);
  for (int m = 0; m < M; ++m) sv->pos[m] = m % T;
  BuildRope(T, D, c.rope_base, 0, &sv->cosv, &sv->sinv);
  // embedding -> norm -> smear
  SectionTimer t_trunk("fwd trunk (everything below)");
  const float* wte = P("transformer.wte.weight");
  sv->emb_raw.resize(static_cast<std::size_t>(M) * C);
  for (int m = 0; m < M; ++m)
    std::memcpy(&sv->emb_raw[static_cast<std::size_t>(m) * C], wte + static_cast<std::size_t>(tokens[m]) * C,
                sizeof(float) * C);
  sv->emb.resize(sv->emb_raw.size());
  sv->rstd_e.resize(M);
  RmsNorm(sv->emb_raw.data(), sv->emb.data(), sv->rstd_e.data(), M, C);
  const float* gw = P("smear_gate.weight");
  const float lam_s = P("smear_lambda")[0];
  sv->sig.assign(M, 0.0f);
  sv->x0 = sv->emb;
  for (int m = 0; m < M; ++m) {
    if (m % T == 0) continue;
    const float* e = &sv->emb[static_cast<std::size_t>(m) * C];
    const float* prev = e - C;
    double pre = 0.0;
    for (int j = 0; j < kSmearCh; ++j) pre += static_cast<double>(e[j]) * gw[j];
    const float sg = Sigmoid(static_cast<float>(pre));
    sv->sig[m] = sg;
    float* x = &sv->x0[static_cast<std::size_t>(m) * C];
    for (int j = 0; j < C; ++j) x[j] = e[j] + lam_s * sg * prev[j];
  }
  std::vector<float> x = sv->x0, h(static_cast<std::size_t>(M) * C);
  sv->layers.assign(c.num_layers, LayerSaved());
  const float* lam_r = P("resid_lambdas");
  const float* lam_0 = P("x0_lambdas");
  for (int i = 0; i < c.num_layers; ++i) {
    LayerSaved& s = sv->layers[i];
    const std::string pf = "transformer.h." + std::to_string(i) + ".";
    s.x = x;
    s.xr.resize(x.size());
    {
      SectionTimer t("fwd blend+norm");
      for (std::size_t j = 0; j < x.size(); ++j) s.xr[j] = lam_r[i] * x[j] + lam_0[i] * sv->x0[j];
      s.rstd1.resize(M);
      RmsNorm(s.xr.data(), h.data(), s.rstd1.data(), M, C);
    }
    s.q_pre.resize(static_cast<std::size_t>(M) * QD);
    s.k_pre.resize(static_cast<std::size_t>(M) * KD);
    s.v.resize(static_cast<std::size_t>(M) * KD);
    {
      SectionTimer t("fwd linear");
      Linear(h.data(), P(pf + "attn.c_q.weight"), s.q_pre.data(), M, QD, C);
      Linear(h.data(), P(pf + "attn.c_k.weight"), s.k_pre.data(), M, KD, C);
      Linear(h.data(), P(pf + "attn.c_v.weight"), s.v.data(), M, KD, C);
    }
    s.q.resize(s.q_pre.size());
    s.k.resize(s.k_pre.size());
    {
    SectionTimer t_gate("fwd gate+qkprep");
    if (c.has_value_embedding(i)) {
      const float* table = P("value_embeds." + std::to_string(i) + ".weight");
      const float* gate_w = P(pf + "attn.ve_gate.weight");
      s.ve.resize(static_cast<std::size_t>(M) * KD);
      s.gate.resize(static_cast<std::size_t>(M) * KV);
      for (int m = 0; m < M; ++m) {
        std::memcpy(&s.ve[static_cast<std::size_t>(m) * KD], table + static_cast<std::size_t>(tokens[m]) * KD,
                    sizeof(float) * KD);
        for (int g = 0; g < KV; ++g) {
          float pre = 0.0f;
          for (int j = 0; j < kGateCh; ++j) pre += h[static_cast<std::size_t>(m) * C + j] * gate_w[g * kGateCh + j];
          const float gt = 3.0f * Sigmoid(pre);
          s.gate[static_cast<std::size_t>(m) * KV + g] = gt;
          for (int d = 0; d < D; ++d) {
            const std::size_t idx = static_cast<std::size_t>(m) * KD + g * D + d;
            s.v[idx] += gt * s.ve[idx];
          }
        }
      }
    }
    QkPrep(s.q_pre.data(), s.q.data(), M, H, D, sv->cosv.data(), sv->sinv.data(), sv->pos.data());
    QkPrep(s.k_pre.data(), s.k.data(), M, KV, D, sv->cosv.data(), sv->sinv.data(), sv->pos.data());
    }
    s.attn.resize(static_cast<std::size_t>(M) * QD);
    s.lse.resize(static_cast<std::size_t>(B) * H * T);
    {
      SectionTimer t("fwd attention");
      Attention(s.q.data(), s.k.data(), s.v.data(), s.attn.data(), s.lse.data(), B, T, H, KV, D, c.window_left(i));
    }
    s.x_mid.resize(x.size());
    {
      SectionTimer t("fwd linear");
      Linear(s.attn.data(), P(pf + "attn.c_proj.weight"), s.x_mid.data(), M, C, QD, s.xr.data());
    }
    s.rstd2.resize(M);
    RmsNorm(s.x_mid.data(), h.data(), s.rstd2.data(), M, C);
    s.pre.resize(static_cast<std::size_t>(M) * F);
    SectionTimer t_mlp("fwd mlp (to end of layer)");
    Linear(h.data(), P(pf + "mlp.c_fc.weight"), s.pre.data(), M, F, C);
    std::vector<float> act(s.pre.size());
    {
      const float* pre = s.pre.data();
      float* ap = act.data();
      const long long n_act = static_cast<long long>(act.size());
#pragma omp parallel for simd schedule(static)
      for (long long j = 0; j < n_act; ++j) {
        const float r = std::max(pre[j], 0.0f);
        ap[j] = r * r;
      }
    }
    Linear(act.data(), P(pf + "mlp.c_proj.weight"), x.data(), M, C, F, s.x_mid.data());
    if (i == c.backout_layer()) sv->x_backout = x;
  }
  sv->x_last = x;
  const float lam_b = P("backout_lambda")[0];
  sv->x_pre.resize(x.size());
  for (std::size_t j = 0; j < x.size(); ++j) sv->x_pre[j] = x[j] - lam_b * sv->x_backout[j];
  sv->rstd_f.resize(M);
  xn_out->resize(x.size());
  RmsNorm(sv->x_pre.data(), xn_out->data(), sv->rstd_f.data(), M, C);
}

float CpuModel::ForwardLoss(const int* tokens, const int* targets, int B, int T, bool keep_logits) {
  (void)keep_logits;  // logits are kept whenever a backward or a score may follow: always, at this scale
  saved_ = std::make_unique<Saved>();
  Saved* sv = saved_.get();
  Trunk(tokens, B, T, sv, &sv->xn);
  const int M = B * T, C = cfg_.hidden_dim, V = cfg_.vocab_size, PV = cfg_.padded_vocab_size;
  sv->targets.assign(targets, targets + M);
  {
    SectionTimer t("fwd head linear");
    logits_.assign(static_cast<std::size_t>(M) * PV, 0.0f);
    Linear(sv->xn.data(), value(*Find("lm_head.weight")), logits_.data(), M, PV, C);
  }
  SectionTimer t_cls("fwd classifier");
  losses_.assign(M, 0.0f);
  double total = 0.0;
  std::int64_t valid = 0;
#pragma omp parallel for schedule(static) reduction(+ : total, valid)
  for (int m = 0; m < M; ++m) {
    const int tg = targets[m];
    if (tg == -1) continue;
    ++valid;
    const float* row = &logits_[static_cast<std::size_t>(m) * PV];
    // one tanh and one exp per logit: the capped values are kept for the second sweep
    std::vector<float> z(static_cast<std::size_t>(V));
    float mx = -std::numeric_limits<float>::infinity();
    for (int j = 0; j < V; ++j) {
      z[j] = kSoftcap * std::tanh(row[j] / kSoftcap);
      mx = std::max(mx, z[j]);
    }
    double sum = 0.0;
    for (int j = 0; j < V; ++j) sum += std::exp(z[j] - mx);
    const float tz = (tg >= 0 && tg < V) ? z[tg] : 0.0f;
    losses_[m] = static_cast<float>(std::log(sum)) + mx - tz;
    total += losses_[m];
  }
  valid_ = valid;
  return static_cast<float>(total / static_cast<double>(std::max<std::int64_t>(valid_, 1)));
}

// ---------------------------------------------------------------------------------------------- backward
void CpuModel::Backward(float scale, const float* row_weights, double divisor) {
  if (!saved_) return;
  Saved* sv = saved_.get();
  const EngineConfig& c = cfg_;
  const int B = sv->B, T = sv->T, M = B * T, C = c.hidden_dim, H = c.num_heads, KV = c.num_kv_heads;
  const int D = c.head_dim(), QD = c.query_dim(), KD = c.kv_dim(), F = c.mlp_dim();
  const int V = c.vocab_size, PV = c.padded_vocab_size;
  auto Pv = [&](const std::string& n) { return value(*Find(n)); };
  auto Pg = [&](const std::string& n) { return grad(*Find(n)); };
  const double denom = divisor > 0.0 ? divisor : static_cast<double>(std::max<std::int64_t>(valid_, 1));
  const float dscale = static_cast<float>(static_cast<double>(scale) / denom);
  // dlogits = (softmax - onehot) * (1 - tanh^2) * row_weight * dscale
  std::vector<float> dlogits(static_cast<std::size_t>(M) * PV, 0.0f);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const int tg = sv->targets[m];
    if (tg == -1) continue;
    const float* row = &logits_[static_cast<std::size_t>(m) * PV];
    float* drow = &dlogits[static_cast<std::size_t>(m) * PV];
    // one tanh and one exp per logit: tanh is kept in the output row, exp in a scratch row, for the last sweep
    std::vector<float> e(static_cast<std::size_t>(V));
    float mx = -std::numeric_limits<float>::infinity();
    for (int j = 0; j < V; ++j) {
      drow[j] = std::tanh(row[j] / kSoftcap);
      mx = std::max(mx, kSoftcap * drow[j]);
    }
    double sum = 0.0;
    for (int j = 0; j < V; ++j) {
      e[j] = std::exp(kSoftcap * drow[j] - mx);
      sum += e[j];
    }
    const float inv = static_cast<float>(1.0 / sum);
    const float rw = row_weights ? row_weights[m] : 1.0f;
    for (int j = 0; j < V; ++j) {
      const float t = drow[j];
      const float onehot = (j == tg) ? 1.0f : 0.0f;
      drow[j] = (e[j] * inv - onehot) * (1.0f - t * t) * rw * dscale;
    }
  }
  std::vector<float> dxn(static_cast<std::size_t>(M) * C);
  LinearDgrad(dlogits.data(), Pv("lm_head.weight"), dxn.data(), M, PV, C, false);
  LinearWgrad(dlogits.data(), sv->xn.data(), Pg("lm_head.weight"), M, PV, C);
  dlogits.clear();
  dlogits.shrink_to_fit();
  // tail: final norm, backout
  std::vector<float> dx(static_cast<std::size_t>(M) * C), dxb(dx.size()), dx0(dx.size(), 0.0f);
  RmsNormBwd(sv->x_pre.data(), dxn.data(), sv->rstd_f.data(), dx.data(), M, C);
  const float lam_b = Pv("backout_lambda")[0];
  double dlam_b = 0.0;
  for (std::size_t j = 0; j < dx.size(); ++j) {
    dlam_b -= static_cast<double>(dx[j]) * sv->x_backout[j];
    dxb[j] = -lam_b * dx[j];
  }
  Pg("backout_lambda")[0] += static_cast<float>(dlam_b);
  const float* lam_r = Pv("resid_lambdas");
  const float* lam_0 = Pv("x0_lambdas");
  std::vector<float> tmp(static_cast<std::size_t>(M) * std::max(F, std::max(QD, C)));
  for (int i = c.num_layers - 1; i >= 0; --i) {
    LayerSaved& s = sv->layers[i];
    const std::string pf = "transformer.h." + std::to_string(i) + ".";
    if (i == c.backout_layer())
      for (std::size_t j = 0; j < dx.size(); ++j) dx[j] += dxb[j];
    // MLP
    std::vector<float> act(s.pre.size()), dpre(s.pre.size());
    for (std::size_t j = 0; j < act.size(); ++j) {
      const float r = std::max(s.pre[j], 0.0f);
      act[j] = r * r;
    }
    LinearWgrad(dx.data(), act.data(), Pg(pf + "mlp.c_proj.weight"), M, C, F);
    LinearDgrad(dx.data(), Pv(pf + "mlp.c_proj.weight"), dpre.data(), M, C, F, false);
    for (std::size_t j = 0; j < dpre.size(); ++j) dpre[j] *= 2.0f * std::max(s.pre[j], 0.0f);
    std::vector<float> h2(static_cast<std::size_t>(M) * C), dh2(h2.size()), dx_mid(h2.size());
    for (int m = 0; m < M; ++m)
      for (int j = 0; j < C; ++j) h2[static_cast<std::size_t>(m) * C + j] = s.x_mid[static_cast<std::size_t>(m) * C + j] * s.rstd2[m];
    LinearWgrad(dpre.data(), h2.data(), Pg(pf + "mlp.c_fc.weight"), M, F, C);
    LinearDgrad(dpre.data(), Pv(pf + "mlp.c_fc.weight"), dh2.data(), M, F, C, false);
    RmsNormBwd(s.x_mid.data(), dh2.data(), s.rstd2.data(), dx_mid.data(), M, C, dx.data());
    // attention output projection
    std::vector<float> dattn(static_cast<std::size_t>(M) * QD);
    LinearWgrad(dx_mid.data(), s.attn.data(), Pg(pf + "attn.c_proj.weight"), M, C, QD);
    LinearDgrad(dx_mid.data(), Pv(pf + "attn.c_proj.weight"), dattn.data(), M, C, QD, false);
    std::vector<float> dq(static_cast<std::size_t>(M) * QD), dk(static_cast<std::size_t>(M) * KD), dv(dk.size());
    AttentionBwd(s.q.data(), s.k.data(), s.v.data(), s.attn.data(), s.lse.data(), dattn.data(), dq.data(), dk.data(),
                 dv.data(), B, T, H, KV, D, c.window_left(i));
    std::vector<float> dq_pre(dq.size()), dk_pre(dk.size());
    QkPrepBwd(s.q_pre.data(), dq.data(), dq_pre.data(), M, H, D, sv->cosv.data(), sv->sinv.data(), sv->pos.data());
    QkPrepBwd(s.k_pre.data(), dk.data(), dk_pre.data(), M, KV, D, sv->cosv.data(), sv->sinv.data(), sv->pos.data());
    std::vector<float> h(static_cast<std::size_t>(M) * C), dh(h.size());
    for (int m = 0; m < M; ++m)
      for (int j = 0; j < C; ++j) h[static_cast<std::size_t>(m) * C + j] = s.xr[static_cast<std::size_t>(m) * C + j] * s.rstd1[m];
    std::vector<float> dh12;
    if (c.has_value_embedding(i)) {
      const float* gate_w = Pv(pf + "attn.ve_gate.weight");
      float* ggw = Pg(pf + "attn.ve_gate.weight");
      float* gtable = Pg("value_embeds." + std::to_string(i) + ".weight");
      dh12.assign(static_cast<std::size_t>(M) * kGateCh, 0.0f);
      std::vector<double> dgw(static_cast<std::size_t>(KV) * kGateCh, 0.0);
      for (int m = 0; m < M; ++m)
        for (int g = 0; g < KV; ++g) {
          const float gt = s.gate[static_cast<std::size_t>(m) * KV + g];
          double dgate = 0.0;
          for (int d = 0; d < D; ++d) {
            const std::size_t idx = static_cast<std::size_t>(m) * KD + g * D + d;
            dgate += static_cast<double>(dv[idx]) * s.ve[idx];
            gtable[static_cast<std::size_t>(sv->tokens[m]) * KD + g * D + d] += gt * dv[idx];
          }
          const float dpre_g = static_cast<float>(dgate) * gt * (1.0f - gt / 3.0f);
          for (int j = 0; j < kGateCh; ++j) {
            dgw[static_cast<std::size_t>(g) * kGateCh + j] += static_cast<double>(dpre_g) * h[static_cast<std::size_t>(m) * C + j];
            dh12[static_cast<std::size_t>(m) * kGateCh + j] += dpre_g * gate_w[g * kGateCh + j];
          }
        }
      for (std::size_t j = 0; j < dgw.size(); ++j) ggw[j] += static_cast<float>(dgw[j]);
    }
    LinearWgrad(dq_pre.data(), h.data(), Pg(pf + "attn.c_q.weight"), M, QD, C);
    LinearWgrad(dk_pre.data(), h.data(), Pg(pf + "attn.c_k.weight"), M, KD, C);
    LinearWgrad(dv.data(), h.data(), Pg(pf + "attn.c_v.weight"), M, KD, C);
    LinearDgrad(dq_pre.data(), Pv(pf + "attn.c_q.weight"), dh.data(), M, QD, C, false);
    LinearDgrad(dk_pre.data(), Pv(pf + "attn.c_k.weight"), dh.data(), M, KD, C, true);
    LinearDgrad(dv.data(), Pv(pf + "attn.c_v.weight"), dh.data(), M, KD, C, true);
    if (!dh12.empty())
      for (int m = 0; m < M; ++m)
        for (int j = 0; j < kGateCh; ++j) dh[static_cast<std::size_t>(m) * C + j] += dh12[static_cast<std::size_t>(m) * kGateCh + j];
    std::vector<float> dxr(h.size());
    RmsNormBwd(s.xr.data(), dh.data(), s.rstd1.data(), dxr.data(), M, C, dx_mid.data());
    double dlr = 0.0, dl0 = 0.0;
    for (std::size_t j = 0; j < dxr.size(); ++j) {
      dlr += static_cast<double>(dxr[j]) * s.x[j];
      dl0 += static_cast<double>(dxr[j]) * sv->x0[j];
      dx[j] = lam_r[i] * dxr[j];
      dx0[j] += lam_0[i] * dxr[j];
    }
    Pg("resid_lambdas")[i] += static_cast<float>(dlr);
    Pg("x0_lambdas")[i] += static_cast<float>(dl0);
    s = LayerSaved();
  }
  // embedding side: smear, norm, scatter
  for (std::size_t j = 0; j < dx0.size(); ++j) dx0[j] += dx[j];
  const float* gw = Pv("smear_gate.weight");
  const float lam_s = Pv("smear_lambda")[0];
  std::vector<float> de = dx0;
  std::vector<double> dgw(kSmearCh, 0.0);
  double dlam = 0.0;
  for (int m = 0; m < M; ++m) {
    if (m % T == 0) continue;
    const float* e = &sv->emb[static_cast<std::size_t>(m) * C];
    const float* prev = e - C;
    const float* d = &dx0[static_cast<std::size_t>(m) * C];
    double dgate = 0.0;
    for (int j = 0; j < C; ++j) dgate += static_cast<double>(d[j]) * prev[j];
    const float sg = sv->sig[m];
    dlam += dgate * sg;
    const float dpre = static_cast<float>(dgate) * lam_s * sg * (1.0f - sg);
    for (int j = 0; j < kSmearCh; ++j) {
      dgw[j] += static_cast<double>(dpre) * e[j];
      de[static_cast<std::size_t>(m) * C + j] += dpre * gw[j];
    }
    const float gate_next = lam_s * sg;
    for (int j = 0; j < C; ++j) de[static_cast<std::size_t>(m - 1) * C + j] += gate_next * d[j];
  }
  float* ggw = Pg("smear_gate.weight");
  for (int j = 0; j < kSmearCh; ++j) ggw[j] += static_cast<float>(dgw[j]);
  Pg("smear_lambda")[0] += static_cast<float>(dlam);
  std::vector<float> de_raw(de.size());
  RmsNormBwd(sv->emb_raw.data(), de.data(), sv->rstd_e.data(), de_raw.data(), M, C);
  float* gwte = Pg("transformer.wte.weight");
  for (int m = 0; m < M; ++m)
    for (int j = 0; j < C; ++j) gwte[static_cast<std::size_t>(sv->tokens[m]) * C + j] += de_raw[static_cast<std::size_t>(m) * C + j];
  (void)tmp;
}

// ---------------------------------------------------------------------------------------------- checkpoints
bool CpuModel::Save(const std::string& path, std::string* error) const {
  Checkpoint ck;
  static_cast<ModelConfig&>(ck.metadata.config) = cfg_;
  for (const auto& p : params_) {
    TensorRecord r;
    r.name = p.name, r.dtype = DType::kFp32, r.shape = p.shape;
    r.data.resize(p.count * 4);
    std::memcpy(r.data.data(), value_.data() + p.offset, p.count * 4);
    ck.tensors.push_back(std::move(r));
  }
  return ck.Save(path, error);
}

bool CpuModel::Load(const std::string& path, std::string* error) {
  Checkpoint ck;
  if (!ck.Load(path, false, error)) return false;
  for (const auto& p : params_) {
    const TensorRecord* r = ck.Find(p.name);
    if (r == nullptr || static_cast<std::size_t>(r->NumElements()) != p.count) {
      if (error) *error = "checkpoint has no record of the right size for " + p.name;
      return false;
    }
    float* dst = value_.data() + p.offset;
    if (r->dtype == DType::kFp32) {
      std::memcpy(dst, r->data.data(), p.count * 4);
    } else if (r->dtype == DType::kBf16) {
      const std::uint16_t* src = reinterpret_cast<const std::uint16_t*>(r->data.data());
      for (std::size_t i = 0; i < p.count; ++i) dst[i] = Bf16ToFloat(src[i]);
    } else {
      if (error) *error = "unsupported dtype for " + p.name;
      return false;
    }
  }
  return true;
}

bool CpuModel::SaveWithOptimizer(const std::string& path, const CpuOptimizer& opt, std::uint64_t step,
                                 std::uint32_t world_size, std::string* error) const {
  Checkpoint ck;
  static_cast<ModelConfig&>(ck.metadata.config) = cfg_;
  ck.metadata.step = step;
  ck.metadata.world_size = world_size;
  for (const auto& p : params_) {
    TensorRecord r;
    r.name = p.name, r.dtype = DType::kFp32, r.shape = p.shape;
    r.data.resize(p.count * 4);
    std::memcpy(r.data.data(), value_.data() + p.offset, p.count * 4);
    ck.tensors.push_back(std::move(r));
  }
  opt.ExportState(&ck.optimizer_state);
  TensorRecord st;
  st.name = "optimizer/step", st.dtype = DType::kFp32, st.shape = {1};
  const float stepf = static_cast<float>(step);
  st.data.resize(4);
  std::memcpy(st.data.data(), &stepf, 4);
  ck.optimizer_state.push_back(std::move(st));
  return ck.Save(path, error);
}

bool CpuModel::LoadWithOptimizer(const std::string& path, CpuOptimizer* opt, std::uint64_t* step, std::string* error) {
  if (!Load(path, error)) return false;
  if (opt == nullptr && step == nullptr) return true;
  Checkpoint ck;
  if (!ck.Load(path, true, error)) return false;
  if (step != nullptr) *step = ck.metadata.step;
  return opt == nullptr || opt->ImportState(ck.optimizer_state, error);
}

namespace {
const char* KindRecordName(ParamKind k) {
  switch (k) {
    case ParamKind::kLmHead: return "lm_head";
    case ParamKind::kWte: return "embedding";
    case ParamKind::kValueEmbed: return "value_embedding";
    case ParamKind::kResid: return "resid";
    case ParamKind::kX0: return "x0";
    case ParamKind::kSmear: return "smear";
    default: return "matrix";
  }
}
TensorRecord FloatRecord(const std::string& name, std::vector<std::int64_t> shape, const std::vector<const std::vector<float>*>& parts) {
  TensorRecord r;
  r.name = name, r.dtype = DType::kFp32, r.shape = std::move(shape);
  std::size_t total = 0;
  for (const auto* p : parts) total += p->size();
  r.data.resize(total * 4);
  std::size_t off = 0;
  for (const auto* p : parts) {
    std::memcpy(r.data.data() + off, p->data(), p->size() * 4);
    off += p->size() * 4;
  }
  return r;
}
bool Scatter(const TensorRecord* r, std::vector<std::vector<float>>* parts, const std::string& name, std::string* error) {
  if (r == nullptr) return true;  // an absent record keeps the fresh state
  std::size_t total = 0;
  for (const auto& p : *parts) total += p.size();
  if (r->dtype != DType::kFp32 || r->data.size() != total * 4) {
    if (error) *error = "optimizer record " + name + " has the wrong size or dtype";
    return false;
  }
  std::size_t off = 0;
  for (auto& p : *parts) {
    std::memcpy(p.data(), r->data.data() + off, p.size() * 4);
    off += p.size() * 4;
  }
  return true;
}
}  // namespace

void CpuOptimizer::ExportState(std::vector<TensorRecord>* out) const {
  for (const auto& g : adam_) {
    if (g.params.empty()) continue;
    std::vector<const std::vector<float>*> m, v;
    std::int64_t total = 0;
    for (std::size_t k = 0; k < g.params.size(); ++k) {
      m.push_back(&g.m[k]);
      v.push_back(&g.v[k]);
      total += static_cast<std::int64_t>(g.m[k].size());
    }
    const std::string base = std::string("adamw.") + KindRecordName(g.kind);
    out->push_back(FloatRecord(base + ".m", {total}, m));
    out->push_back(FloatRecord(base + ".v", {total}, v));
  }
  for (const auto& g : muon_) {
    std::vector<const std::vector<float>*> b1, b2;
    for (std::size_t k = 0; k < g.params.size(); ++k) {
      b1.push_back(&g.buf1[k]);
      b2.push_back(&g.buf2[k]);
    }
    const std::string base = "muon." + std::to_string(g.rows) + "x" + std::to_string(g.cols);
    const std::int64_t n = static_cast<std::int64_t>(g.params.size());
    out->push_back(FloatRecord(base + ".buf1", {n, g.rows, g.cols}, b1));
    out->push_back(FloatRecord(base + ".buf2", {n, std::max(g.rows, g.cols)}, b2));
  }
}

bool CpuOptimizer::ImportState(const std::vector<TensorRecord>& records, std::string* error) {
  auto find = [&](const std::string& name) -> const TensorRecord* {
    for (const auto& r : records)
      if (r.name == name) return &r;
    return nullptr;
  };
  for (auto& g : adam_) {
    if (g.params.empty()) continue;
    const std::string base = std::string("adamw.") + KindRecordName(g.kind);
    if (!Scatter(find(base + ".m"), &g.m, base + ".m", error)) return false;
    if (!Scatter(find(base + ".v"), &g.v, base + ".v", error)) return false;
  }
  for (auto& g : muon_) {
    const std::string base = "muon." + std::to_string(g.rows) + "x" + std::to_string(g.cols);
    if (!Scatter(find(base + ".buf1"), &g.buf1, base + ".buf1", error)) return false;
    if (!Scatter(find(base + ".buf2"), &g.buf2, base + ".buf2", error)) return false;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------- inference
// Contiguous cache: per layer prepared keys and gated values [max_seq, kv_dim], plus the normalised embedding of the
// last token (the smear of the next token mixes it in) - the layout of the reference's KvCacheImpl
// (src/generate.cc:89-257).
class KvCache {
 public:
  KvCache(int layers, int max_seq, int kv_dim, int hidden)
      : max_seq(max_seq), k(layers, std::vector<float>(static_cast<std::size_t>(max_seq) * kv_dim)), v(k),
        prev(static_cast<std::size_t>(hidden), 0.0f) {}
  int max_seq, len = 0;
  bool has_prev = false;
  std::vector<std::vector<float>> k, v;
  std::vector<float> prev;
};

std::unique_ptr<KvCache> CpuModel::NewCache(int max_seq) const {
  return std::make_unique<KvCache>(cfg_.num_layers, max_seq, cfg_.kv_dim(), cfg_.hidden_dim);
}

void CpuModel::Step(KvCache* cache, const int* tokens, int count, std::vector<float>* out_logits) {
  const EngineConfig& c = cfg_;
  const int C = c.hidden_dim, H = c.num_heads, KV = c.num_kv_heads, D = c.head_dim();
  const int QD = c.query_dim(), KD = c.kv_dim(), F = c.mlp_dim(), group = H / KV;
  auto P = [&](const std::string& n) { return value(*Find(n)); };
  const int start = cache->len;
  if (start + count > cache->max_seq) count = cache->max_seq - start;
  if (count <= 0) return;
  const int M = count;
  std::vector<int> pos(M);
  for (int m = 0; m < M; ++m) pos[m] = start + m;
  std::vector<float> cosv, sinv;
  BuildRope(start + count, D, c.rope_base, 0, &cosv, &sinv);
  std::vector<float> emb_raw(static_cast<std::size_t>(M) * C), emb(emb_raw.size());
  const float* wte = P("transformer.wte.weight");
  for (int m = 0; m < M; ++m)
    std::memcpy(&emb_raw[static_cast<std::size_t>(m) * C], wte + static_cast<std::size_t>(tokens[m]) * C, sizeof(float) * C);
  RmsNorm(emb_raw.data(), emb.data(), nullptr, M, C);
  const float* gw = P("smear_gate.weight");
  const float lam_s = P("smear_lambda")[0];
  std::vector<float> x0 = emb;
  for (int m = 0; m < M; ++m) {
    const float* prev = m > 0 ? &emb[static_cast<std::size_t>(m - 1) * C] : (cache->has_prev ? cache->prev.data() : nullptr);
    if (prev == nullptr) continue;
    const float* e = &emb[static_cast<std::size_t>(m) * C];
    double pre = 0.0;
    for (int j = 0; j < kSmearCh; ++j) pre += static_cast<double>(e[j]) * gw[j];
    const float sg = Sigmoid(static_cast<float>(pre));
    for (int j = 0; j < C; ++j) x0[static_cast<std::size_t>(m) * C + j] = e[j] + lam_s * sg * prev[j];
  }
  std::memcpy(cache->prev.data(), &emb[static_cast<std::size_t>(M - 1) * C], sizeof(float) * C);
  cache->has_prev = true;
  std::vector<float> x = x0, xr(x.size()), h(x.size()), x_mid(x.size()), x_backout;
  std::vector<float> q_pre(static_cast<std::size_t>(M) * QD), q(q_pre.size()), k_pre(static_cast<std::size_t>(M) * KD),
      kk(k_pre.size()), vv(k_pre.size()), attn(q_pre.size()), pre(static_cast<std::size_t>(M) * F);
  const float* lam_r = P("resid_lambdas");
  const float* lam_0 = P("x0_lambdas");
  const float scale = 1.0f / std::sqrt(static_cast<float>(D));
  for (int i = 0; i < c.num_layers; ++i) {
    const std::string pf = "transformer.h." + std::to_string(i) + ".";
    for (std::size_t j = 0; j < x.size(); ++j) xr[j] = lam_r[i] * x[j] + lam_0[i] * x0[j];
    RmsNorm(xr.data(), h.data(), nullptr, M, C);
    Linear(h.data(), P(pf + "attn.c_q.weight"), q_pre.data(), M, QD, C);
    Linear(h.data(), P(pf + "attn.c_k.weight"), k_pre.data(), M, KD, C);
    Linear(h.data(), P(pf + "attn.c_v.weight"), vv.data(), M, KD, C);
    if (c.has_value_embedding(i)) {
      const float* table = P("value_embeds." + std::to_string(i) + ".weight");
      const float* gate_w = P(pf + "attn.ve_gate.weight");
      for (int m = 0; m < M; ++m)
        for (int g = 0; g < KV; ++g) {
          float p = 0.0f;
          for (int j = 0; j < kGateCh; ++j) p += h[static_cast<std::size_t>(m) * C + j] * gate_w[g * kGateCh + j];
          const float gt = 3.0f * Sigmoid(p);
          for (int d = 0; d < D; ++d)
            vv[static_cast<std::size_t>(m) * KD + g * D + d] += gt * table[static_cast<std::size_t>(tokens[m]) * KD + g * D + d];
        }
    }
    QkPrep(q_pre.data(), q.data(), M, H, D, cosv.data(), sinv.data(), pos.data());
    QkPrep(k_pre.data(), kk.data(), M, KV, D, cosv.data(), sinv.data(), pos.data());
    std::memcpy(&cache->k[i][static_cast<std::size_t>(start) * KD], kk.data(), sizeof(float) * kk.size());
    std::memcpy(&cache->v[i][static_cast<std::size_t>(start) * KD], vv.data(), sizeof(float) * vv.size());
    const int wl = c.window_left(i);
    std::vector<float> sc(static_cast<std::size_t>(start + M));
    for (int m = 0; m < M; ++m)
      for (int hh = 0; hh < H; ++hh) {
        const int kvh = hh / group, qp = pos[m];
        const int first = wl < 0 ? 0 : std::max(0, qp - wl);
        const float* qr = &q[(static_cast<std::size_t>(m) * H + hh) * D];
        float mx = -std::numeric_limits<float>::infinity();
        for (int j = first; j <= qp; ++j) {
          const float* kr = &cache->k[i][static_cast<std::size_t>(j) * KD + kvh * D];
          double a = 0.0;
          for (int d = 0; d < D; ++d) a += static_cast<double>(qr[d]) * kr[d];
          sc[j] = static_cast<float>(a) * scale;
          mx = std::max(mx, sc[j]);
        }
        double sum = 0.0;
        for (int j = first; j <= qp; ++j) sum += std::exp(static_cast<double>(sc[j] - mx));
        std::vector<double> acc(static_cast<std::size_t>(D), 0.0);
        for (int j = first; j <= qp; ++j) {
          const double p = std::exp(static_cast<double>(sc[j] - mx)) / sum;
          const float* vr = &cache->v[i][static_cast<std::size_t>(j) * KD + kvh * D];
          for (int d = 0; d < D; ++d) acc[d] += p * vr[d];
        }
        for (int d = 0; d < D; ++d) attn[(static_cast<std::size_t>(m) * H + hh) * D + d] = static_cast<float>(acc[d]);
      }
    Linear(attn.data(), P(pf + "attn.c_proj.weight"), x_mid.data(), M, C, QD, xr.data());
    RmsNorm(x_mid.data(), h.data(), nullptr, M, C);
    Linear(h.data(), P(pf + "mlp.c_fc.weight"), pre.data(), M, F, C);
    for (auto& p : pre) {
      const float r = std::max(p, 0.0f);
      p = r * r;
    }
    Linear(pre.data(), P(pf + "mlp.c_proj.weight"), x.data(), M, C, F, x_mid.data());
    if (i == c.backout_layer()) x_backout = x;
  }
  cache->len = start + M;
  if (out_logits == nullptr) return;
  // only the last row feeds the head
  const float lam_b = P("backout_lambda")[0];
  std::vector<float> last(static_cast<std::size_t>(C)), xn(static_cast<std::size_t>(C));
  for (int j = 0; j < C; ++j)
    last[j] = x[static_cast<std::size_t>(M - 1) * C + j] - lam_b * x_backout[static_cast<std::size_t>(M - 1) * C + j];
  RmsNorm(last.data(), xn.data(), nullptr, 1, C);
  std::vector<float> raw(static_cast<std::size_t>(c.padded_vocab_size));
  Linear(xn.data(), P("lm_head.weight"), raw.data(), 1, c.padded_vocab_size, C);
  out_logits->resize(static_cast<std::size_t>(c.vocab_size));
  for (int j = 0; j < c.vocab_size; ++j) (*out_logits)[j] = kSoftcap * std::tanh(raw[j] / kSoftcap);
}

void CpuModel::Prefill(KvCache* cache, const int* tokens, int count, std::vector<float>* last_logits) {
  Step(cache, tokens, count, last_logits);
}
void CpuModel::Decode(KvCache* cache, int token, std::vector<float>* logits) { Step(cache, &token, 1, logits); }

std::vector<GeneratedRow> GenerateBatch(CpuModel* model, const int* prompt, int length, const GenerateOptions& opt,
                                        int first_row) {
  return GenerateBatchOn(model, prompt, length, opt, first_row);
}

std::vector<ScoreRow> ScoreBatch(CpuModel* model, const int* tokens, int batch, int seq, const int* lengths,
                                 const FocusRequest* focus) {
  return ScoreBatchOn(model, tokens, batch, seq, lengths, focus);
}

float RlStep(CpuModel* model, CpuOptimizer* opt, const int* tokens, const int* targets, const float* advantages,
             int batch, int seq, int num_passes, int examples_per_rank, int step) {
  return RlStepOn(model, opt, tokens, targets, advantages, batch, seq, num_passes, examples_per_rank, step);
}

// ---------------------------------------------------------------------------------------------- optimizer
namespace {
// Length of the warm-down in steps: the product in double, rounded half to even as Python's `round` does (the
// reference does the same, src/optim.cc:679-685); 0.5 * 5 is 2 steps, not 3.
int WarmdownIters(float ratio, int num_iterations) {
  return static_cast<int>(std::nearbyint(static_cast<double>(ratio) * static_cast<double>(num_iterations)));
}
}  // namespace

float OptimConfig::LrMultiplier(int step) const {
  const int it = step - 1;
  const int warmdown = WarmdownIters(warmdown_ratio, num_iterations);
  if (warmup_steps > 0 && it < warmup_steps) return static_cast<float>(it + 1) / static_cast<float>(warmup_steps);
  if (warmdown <= 0 || it <= num_iterations - warmdown) return 1.0f;
  const float progress = static_cast<float>(num_iterations - it) / static_cast<float>(warmdown);
  return progress + (1.0f - progress) * final_lr_frac;
}
float OptimConfig::MuonMomentum(int step) const {
  const int it = step - 1;
  const int warmdown = WarmdownIters(warmdown_ratio, num_iterations);
  const int warmdown_start = num_iterations - warmdown;
  if (muon_momentum_warmup_steps > 0.0f && it < muon_momentum_warmup_steps) {
    const float frac = it / muon_momentum_warmup_steps;
    return (1.0f - frac) * muon_momentum_start + frac * muon_momentum_peak;
  }
  if (warmdown > 0 && it >= warmdown_start) {
    const float progress = static_cast<float>(it - warmdown_start) / static_cast<float>(warmdown);
    return muon_momentum_peak * (1.0f - progress) + muon_momentum_final * progress;
  }
  return muon_momentum_peak;
}
float OptimConfig::WeightDecay(int step) const {
  if (num_iterations <= 0) return weight_decay_base;
  const double ratio = static_cast<double>(step - 1) / num_iterations;
  return static_cast<float>(weight_decay_base * 0.5 * (1.0 + std::cos(3.14159265358979323846 * ratio)));
}

CpuOptimizer::CpuOptimizer(CpuModel* model, const OptimConfig& cfg) : model_(model), cfg_(cfg) {
  const float scale = std::sqrt(768.0f / static_cast<float>(model->config().hidden_dim));
  const float f = cfg.init_lr_frac;
  adam_ = {
      {ParamKind::kLmHead, cfg.unembedding_lr * scale * f, 0.8f, 0.96f, 0.01f, {}, {}, {}},
      {ParamKind::kWte, cfg.embedding_lr * scale * f, 0.8f, 0.995f, 0.001f, {}, {}, {}},
      {ParamKind::kValueEmbed, cfg.embedding_lr * scale * 0.5f * f, 0.8f, 0.995f, 0.01f, {}, {}, {}},
      {ParamKind::kResid, cfg.scalar_lr * 0.01f * f, 0.8f, 0.95f, 0.05f, {}, {}, {}},
      {ParamKind::kX0, cfg.scalar_lr * f, 0.96f, 0.95f, 0.0f, {}, {}, {}},
      {ParamKind::kSmear, 0.2f * f, 0.8f, 0.95f, 0.0f, {}, {}, {}},
  };
  for (const auto& p : model->params()) {
    if (p.kind != ParamKind::kMatrix) {
      for (auto& g : adam_)
        if (g.kind == p.kind) {
          g.params.push_back(&p);
          g.m.emplace_back(p.count, 0.0f);
          g.v.emplace_back(p.count, 0.0f);
        }
      continue;
    }
    MuonGroup* grp = nullptr;
    for (auto& g : muon_)
      if (g.rows == p.rows && g.cols == p.cols) grp = &g;
    if (grp == nullptr) {
      const float lr = cfg.matrix_lr * f * std::sqrt(std::max(1.0f, static_cast<float>(p.rows) / static_cast<float>(p.cols)));
      muon_.push_back({p.rows, p.cols, lr, {}, {}, {}});
      grp = &muon_.back();
    }
    grp->params.push_back(&p);
    grp->buf1.emplace_back(p.count, 0.0f);
    grp->buf2.emplace_back(static_cast<std::size_t>(p.rows >= p.cols ? p.rows : p.cols), 0.0f);
  }
}

void CpuOptimizer::Step(int step) {
  double ss = 0.0;
  for (const auto& p : model_->params()) {
    const float* g = model_->grad(p);
    const long long n = static_cast<long long>(p.count);
    double part = 0.0;
#pragma omp parallel for simd schedule(static) reduction(+ : part) if (n > 65536)
    for (long long i = 0; i < n; ++i) part += static_cast<double>(g[i]) * g[i];
    ss += part;
  }
  grad_norm_ = static_cast<float>(std::sqrt(ss));
  const float clip = (cfg_.clip > 0.0f && grad_norm_ > cfg_.clip) ? cfg_.clip / grad_norm_ : 1.0f;
  const float lrm = cfg_.LrMultiplier(step);
  for (auto& g : adam_) {
    const float lr = g.lr * lrm;
    const float bias1 = 1.0f - std::pow(g.beta1, static_cast<float>(step));
    const float bias2 = 1.0f - std::pow(g.beta2, static_cast<float>(step));
    const float step_size = lr / bias1;
    for (std::size_t k = 0; k < g.params.size(); ++k) {
      const CpuParam& p = *g.params[k];
      float* w = model_->value(p);
      const float* gr = model_->grad(p);
      float* mk = g.m[k].data();
      float* vk = g.v[k].data();
      const float b1 = g.beta1, b2 = g.beta2, decay = 1.0f - lr * g.wd, eps = cfg_.adam_eps;
      const long long n = static_cast<long long>(p.count);
#pragma omp parallel for simd schedule(static) if (n > 65536)
      for (long long i = 0; i < n; ++i) {
        const float gi = gr[i] * clip;
        float pi = w[i] * decay;
        mk[i] += (1.0f - b1) * (gi - mk[i]);
        vk[i] += (1.0f - b2) * (gi * gi - vk[i]);
        pi -= step_size * (mk[i] / (std::sqrt(vk[i] / bias2) + eps));
        w[i] = pi;
      }
    }
  }
  const float momentum = cfg_.MuonMomentum(step);
  const float wd = cfg_.WeightDecay(step);
  // one task per matrix: the products inside a task then run on that task's thread alone (nested regions are
  // serial), which scales better over a model's many small matrices than splitting every product over all threads
  std::vector<std::pair<MuonGroup*, std::size_t>> tasks;
  for (auto& g : muon_)
    for (std::size_t k = 0; k < g.params.size(); ++k) tasks.emplace_back(&g, k);
  const int n_tasks = static_cast<int>(tasks.size());
#pragma omp parallel for schedule(dynamic, 1) if (n_tasks >= 4)
  for (int t = 0; t < n_tasks; ++t)
    MuonUpdate(tasks[t].first, tasks[t].second, tasks[t].first->lr * lrm, momentum, wd, clip);
}

namespace {
constexpr double kPolar[5][3] = {
    {8.156554524902461, -22.48329292557795, 15.878769915207462},
    {4.042929935166739, -2.808917465908714, 0.5000178451051316},
    {3.8916678022926607, -2.772484153217685, 0.5060648178503393},
    {3.285753657755655, -2.3681294933425376, 0.46449024233003106},
    {2.3465413258596377, -1.7097828382687081, 0.42323551169305323},
};
// C[n,m] = A[n,k] B[k,m]
void MatMul(const std::vector<float>& A, const std::vector<float>& B, std::vector<float>* Cm, int n, int k, int m) {
  Cm->resize(static_cast<std::size_t>(n) * m);
  GemmNN(A.data(), k, B.data(), m, Cm->data(), m, n, m, k, false);
}
std::vector<float> Transpose(const std::vector<float>& A, int n, int m) {
  std::vector<float> T(A.size());
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < m; ++j) T[static_cast<std::size_t>(j) * n + i] = A[static_cast<std::size_t>(i) * m + j];
  return T;
}
double Frob(const std::vector<float>& x) {
  double s = 0.0;
  for (float v : x) s += static_cast<double>(v) * v;
  return std::sqrt(s);
}
}  // namespace

// Nesterov momentum -> row equilibration -> Polar Express (5 coefficient sets) -> norm snap -> NorMuon -> cautious
// decay (reference backends/cpu/kernels.cc:1614-1810).
void CpuOptimizer::MuonUpdate(MuonGroup* g, std::size_t index, float lr, float momentum, float wd, float grad_scale) {
  const CpuParam& p = *g->params[index];
  MuonUpdateHost(model_->value(p), model_->grad(p), g->buf1[index].data(), g->buf2[index].data(), g->rows, g->cols, lr,
                 momentum, wd, cfg_.muon_beta2, cfg_.muon_ns_steps, grad_scale);
}

void MuonUpdateHost(float* w, const float* gr, float* b1, float* b2, int rows, int cols, float lr, float momentum,
                    float wd, float beta2, int ns_steps, float grad_scale) {
  const std::size_t count = static_cast<std::size_t>(rows) * cols;
  std::vector<float> x(count);
  for (std::size_t i = 0; i < count; ++i) {
    const float gi = gr[i] * grad_scale;
    b1[i] += (1.0f - momentum) * (gi - b1[i]);
    x[i] = (1.0f - momentum) * gi + momentum * b1[i];
  }
  float frob = static_cast<float>(Frob(x));
  const float target = frob / std::sqrt(static_cast<float>(rows));
  for (int r = 0; r < rows; ++r) {
    double s = 0.0;
    for (int c = 0; c < cols; ++c) s += static_cast<double>(x[static_cast<std::size_t>(r) * cols + c]) * x[static_cast<std::size_t>(r) * cols + c];
    const float rn = std::max(static_cast<float>(std::sqrt(s)), 1e-6f);
    for (int c = 0; c < cols; ++c) x[static_cast<std::size_t>(r) * cols + c] *= target / rn;
  }
  frob = static_cast<float>(Frob(x));
  for (auto& v : x) v /= (frob * 1.01f + 1e-6f);
  const bool tall = rows > cols;
  std::vector<float> A, A2, B, Y;
  for (int it = 0; it < std::min(std::max(ns_steps, 0), 5); ++it) {
    const float ca = static_cast<float>(kPolar[it][0]), cb = static_cast<float>(kPolar[it][1]),
                cc = static_cast<float>(kPolar[it][2]);
    const std::vector<float> xt = Transpose(x, rows, cols);
    const int k = tall ? cols : rows;
    if (tall) MatMul(xt, x, &A, cols, rows, cols); else MatMul(x, xt, &A, rows, cols, rows);
    MatMul(A, A, &A2, k, k, k);
    B.resize(A.size());
    for (std::size_t i = 0; i < A.size(); ++i) B[i] = cb * A[i] + cc * A2[i];
    if (tall) MatMul(x, B, &Y, rows, cols, cols); else MatMul(B, x, &Y, rows, rows, cols);
    for (std::size_t i = 0; i < x.size(); ++i) x[i] = ca * x[i] + Y[i];
  }
  frob = static_cast<float>(Frob(x));
  const float snap = std::sqrt(static_cast<float>(std::min(rows, cols))) / std::max(frob, 1e-6f);
  for (auto& v : x) v *= snap;
  const bool reduce_cols = rows >= cols;
  const int lines = reduce_cols ? rows : cols, line_len = reduce_cols ? cols : rows;
  std::vector<float> v_mean(static_cast<std::size_t>(lines));
  double v_total = 0.0;
  for (int l = 0; l < lines; ++l) {
    double s = 0.0;
    for (int e = 0; e < line_len; ++e) {
      const float v = reduce_cols ? x[static_cast<std::size_t>(l) * cols + e] : x[static_cast<std::size_t>(e) * cols + l];
      s += static_cast<double>(v) * v;
    }
    v_mean[l] = static_cast<float>(s / line_len);
    v_total += v_mean[l];
  }
  const float v_norm = std::sqrt(static_cast<float>(v_total) * static_cast<float>(line_len));
  std::vector<float> step_size(static_cast<std::size_t>(lines));
  double sum_scaled = 0.0;
  for (int l = 0; l < lines; ++l) {
    b2[l] += (1.0f - beta2) * (v_mean[l] - b2[l]);
    step_size[l] = 1.0f / std::sqrt(std::max(b2[l], 1e-10f));
    sum_scaled += static_cast<double>(v_mean[l] * line_len) * step_size[l] * step_size[l];
  }
  const float denom = std::max(static_cast<float>(std::sqrt(sum_scaled)), 1e-10f);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const std::size_t i = static_cast<std::size_t>(r) * cols + c;
      const float xv = x[i] * step_size[reduce_cols ? r : c] * (v_norm / denom);
      const float decay = (xv * w[i] >= 0.0f) ? lr * wd * w[i] : 0.0f;
      w[i] = w[i] - lr * xv - decay;
    }
}

}  // namespace ncb
