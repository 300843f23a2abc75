// PyTorch bindings of the sm_100a kernels. Tensors in, raw pointers + current stream out.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <string>

#include <cstdlib>

#include "gemm_tcgen05.h"

namespace {

// One status word per device; kernels record the first bounded-wait failure there.
torch::Tensor& status_tensor(int device) {
  static std::map<int, torch::Tensor> words;
  auto it = words.find(device);
  if (it == words.end()) {
    auto t = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
    it = words.emplace(device, t).first;
  }
  return it->second;
}

int* status_ptr(const torch::Tensor& like) { return status_tensor(like.get_device()).data_ptr<int>(); }
}  // namespace

namespace ncbind {
// The device's status word, for the other binding files.
int* device_status(int device) { return status_tensor(device).data_ptr<int>(); }
}  // namespace ncbind

namespace {

int64_t read_status(int64_t device) {
  return status_tensor(static_cast<int>(device)).cpu().data_ptr<int>()[0];
}
void reset_status(int64_t device) { status_tensor(static_cast<int>(device)).zero_(); }

void check_bf16_cuda(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
  TORCH_CHECK(t.dim() == 2 || t.dim() == 3, name, " must be 2-D or 3-D");
  TORCH_CHECK(t.stride(-1) == 1, name, " must have a contiguous last dimension");
}

// C = epilogue(A x B^T) with per-operand storage order.
//   a_mn == false: A is [.., M, K]   (K contiguous);   a_mn == true: A is [.., K, M]  (M contiguous)
//   b_mn == false: B is [.., N, K]   (K contiguous);   b_mn == true: B is [.., K, N]  (N contiguous)
void gemm(const torch::Tensor& A, const torch::Tensor& B, torch::Tensor& C, bool a_mn, bool b_mn, int64_t epi,
          const c10::optional<torch::Tensor>& R, const c10::optional<torch::Tensor>& C2, double alpha, double beta,
          bool allow_split_k, const c10::optional<torch::Tensor>& wait_flags, int64_t wait_value, int64_t gather_src,
          const c10::optional<torch::Tensor>& gather_counter, int64_t gather_base) {
  check_bf16_cuda(A, "A");
  check_bf16_cuda(B, "B");
  TORCH_CHECK(C.is_cuda() && C.stride(-1) == 1, "C must be a CUDA tensor with a contiguous last dimension");
  TORCH_CHECK(A.dim() == B.dim() && A.dim() == C.dim(), "A, B, C must have the same rank");
  const c10::cuda::CUDAGuard guard(A.device());
  nc::GemmArgs g;
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  g.M = static_cast<int>(a_mn ? A.size(-1) : A.size(-2));
  g.K = static_cast<int>(a_mn ? A.size(-2) : A.size(-1));
  g.N = static_cast<int>(b_mn ? B.size(-1) : B.size(-2));
  const int64_t kb = b_mn ? B.size(-2) : B.size(-1);
  TORCH_CHECK(kb == g.K, "contraction sizes differ: ", g.K, " vs ", kb);
  TORCH_CHECK(C.size(-2) == g.M && C.size(-1) == g.N, "C has the wrong shape");
  g.A = A.data_ptr();
  g.B = B.data_ptr();
  g.lda = A.stride(-2);
  g.ldb = B.stride(-2);
  g.C = C.data_ptr();
  g.ldc = C.stride(-2);
  if (A.dim() == 3) {
    g.batch = static_cast<int>(A.size(0));
    TORCH_CHECK(B.size(0) == g.batch && C.size(0) == g.batch, "batch sizes differ");
    g.strideA = A.stride(0);
    g.strideB = B.stride(0);
    g.strideC = C.stride(0);
  }
  g.epi = static_cast<int>(epi);
  if (g.epi == nc::kEpiF32) {
    TORCH_CHECK(C.scalar_type() == torch::kFloat32, "fp32 epilogue needs an fp32 output");
  } else {
    TORCH_CHECK(C.scalar_type() == torch::kBFloat16, "bf16 epilogue needs a bf16 output");
  }
  if (R.has_value()) {
    check_bf16_cuda(*R, "R");
    TORCH_CHECK(R->sizes() == C.sizes(), "R must have the shape of C");
    g.R = R->data_ptr();
    g.ldr = R->stride(-2);
    if (R->dim() == 3) g.strideR = R->stride(0);
  }
  if (C2.has_value()) {
    check_bf16_cuda(*C2, "C2");
    TORCH_CHECK(C2->sizes() == C.sizes() && C2->stride(-2) == C.stride(-2), "C2 must match C");
    g.C2 = C2->data_ptr();
  }
  g.alpha = static_cast<float>(alpha);
  g.beta = static_cast<float>(beta);
  g.allow_split_k = allow_split_k;
  g.status = status_ptr(A);
  if (wait_flags.has_value()) {
    TORCH_CHECK(wait_flags->is_cuda() && wait_flags->scalar_type() == torch::kInt32 && wait_flags->is_contiguous(),
                "wait_flags must be a contiguous CUDA int32 tensor");
    g.wait_flags = wait_flags->data_ptr<int>();
    g.wait_count = static_cast<int>(wait_flags->numel());
    g.wait_value = static_cast<int>(wait_value);
  }
  if (gather_src != 0) {
    TORCH_CHECK(gather_counter.has_value() && gather_counter->scalar_type() == torch::kInt32, "gather needs a counter");
    TORCH_CHECK(B.is_contiguous() && B.dim() == 2, "gathered B operand must be a contiguous matrix");
    g.gather_src = reinterpret_cast<const void*>(static_cast<uintptr_t>(gather_src));
    g.gather_bytes = B.numel() * 2;
    g.gather_counter = gather_counter->data_ptr<int>();
    g.gather_base = static_cast<int>(gather_base);
  }
  // decode-shaped products take the cluster split-K kernel
  static const bool skinny_enabled = [] {
    const char* e = std::getenv("NANOCHAT_GEMM_SKINNY");
    return e == nullptr || e[0] != '0';
  }();
  const bool plain = g.epi == nc::kEpiBf16 && g.alpha == 1.0f;
  const bool res = g.epi == nc::kEpiBf16Res && g.alpha == 1.0f && g.beta == 1.0f;
  if (skinny_enabled && g.M <= 64 && g.N >= 128 && g.N <= 16384 && !a_mn && !b_mn && g.batch == 1 &&
      (plain || res || g.epi == nc::kEpiRelu2) && g.wait_flags == nullptr && g.gather_src == nullptr) {
    const char* err = nc::gemm_skinny(g, at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(err == nullptr, err);
    return;
  }
  const char* err = nc::gemm_bf16(g, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
}

}  // namespace

void register_rowops(pybind11::module_& m);
void register_attention(pybind11::module_& m);
void register_optim(pybind11::module_& m);
void register_comm(pybind11::module_& m);
void register_decode(pybind11::module_& m);
void register_fp8(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "tcgen05 bf16 GEMM with fused epilogue", pybind11::arg("A"), pybind11::arg("B"),
        pybind11::arg("C"), pybind11::arg("a_mn") = false, pybind11::arg("b_mn") = false, pybind11::arg("epi") = 0,
        pybind11::arg("R") = pybind11::none(), pybind11::arg("C2") = pybind11::none(), pybind11::arg("alpha") = 1.0,
        pybind11::arg("beta") = 0.0, pybind11::arg("allow_split_k") = true,
        pybind11::arg("wait_flags") = pybind11::none(), pybind11::arg("wait_value") = 0,
        pybind11::arg("gather_src") = 0, pybind11::arg("gather_counter") = pybind11::none(),
        pybind11::arg("gather_base") = 0);
  m.def("read_status", &read_status, "first bounded-wait failure recorded on the device (0 = none); synchronizes");
  m.def("reset_status", &reset_status);
  m.def("status_tensor", [](int64_t d) { return status_tensor(static_cast<int>(d)); });
#ifdef NC_HAVE_ROWOPS
  register_rowops(m);
#endif
#ifdef NC_HAVE_ATTENTION
  register_attention(m);
#endif
#ifdef NC_HAVE_OPTIM
  register_optim(m);
#endif
#ifdef NC_HAVE_COMM
  register_comm(m);
#endif
#ifdef NC_HAVE_DECODE
  register_decode(m);
#endif
#ifdef NC_HAVE_FP8
  register_fp8(m);
#endif
}
