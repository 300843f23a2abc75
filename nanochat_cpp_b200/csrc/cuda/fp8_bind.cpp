// Tensor-level wrappers of the block-scaled fp8 kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "fp8.h"

namespace {

using torch::Tensor;

// x bf16 [M, K] (row stride a multiple of 4) -> (xq uint8 [M, K], scales fp32 [K/128, M])
std::vector<Tensor> fp8_quantize_rows(const Tensor& x) {
  const c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.stride(1) == 1, "x must be bf16 [M, K]");
  TORCH_CHECK(x.size(1) % 128 == 0 && x.stride(0) % 4 == 0, "K must be a multiple of 128");
  const int M = x.size(0), K = x.size(1);
  Tensor q = torch::empty({M, K}, x.options().dtype(torch::kUInt8));
  Tensor s = torch::empty({K / 128, M}, x.options().dtype(torch::kFloat32));
  nc::quantize_rows_1x128(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0), q.data_ptr<uint8_t>(),
                          s.data_ptr<float>(), M, K, at::cuda::getCurrentCUDAStream());
  return {q, s};
}

// w bf16 [N, K] -> (wq uint8 [N, K], scales fp32 [N/128, K/128])
std::vector<Tensor> fp8_quantize_blocks(const Tensor& w) {
  const c10::cuda::CUDAGuard g(w.device());
  TORCH_CHECK(w.dim() == 2 && w.scalar_type() == torch::kBFloat16 && w.stride(1) == 1, "w must be bf16 [N, K]");
  TORCH_CHECK(w.size(0) % 128 == 0 && w.size(1) % 128 == 0 && w.stride(0) % 4 == 0, "N and K must be multiples of 128");
  const int N = w.size(0), K = w.size(1);
  Tensor q = torch::empty({N, K}, w.options().dtype(torch::kUInt8));
  Tensor s = torch::empty({N / 128, K / 128}, w.options().dtype(torch::kFloat32));
  nc::quantize_blocks_128x128(reinterpret_cast<const __nv_bfloat16*>(w.data_ptr()), w.stride(0), q.data_ptr<uint8_t>(),
                              s.data_ptr<float>(), N, K, at::cuda::getCurrentCUDAStream());
  return {q, s};
}

void fp8_gemm(const Tensor& aq, const Tensor& sa, const Tensor& bq, const Tensor& sb, Tensor& out,
              const c10::optional<Tensor>& out2, Tensor status) {
  const c10::cuda::CUDAGuard g(aq.device());
  TORCH_CHECK(aq.is_contiguous() && bq.is_contiguous() && aq.scalar_type() == torch::kUInt8 &&
                  bq.scalar_type() == torch::kUInt8 && aq.size(1) == bq.size(1),
              "fp8 operands must be contiguous uint8 [rows, K]");
  TORCH_CHECK(sa.is_contiguous() && sb.is_contiguous() && sa.size(0) == aq.size(1) / 128 && sa.size(1) == aq.size(0) &&
                  sb.size(0) == (bq.size(0) + 127) / 128 && sb.size(1) == aq.size(1) / 128,
              "scale shapes");
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.stride(1) == 1 && out.size(0) == aq.size(0) &&
                  out.size(1) == bq.size(0),
              "out must be bf16 [M, N]");
  nc::Fp8GemmArgs a;
  a.A = aq.data_ptr<uint8_t>(), a.B = bq.data_ptr<uint8_t>();
  a.scale_a = sa.data_ptr<float>(), a.scale_b = sb.data_ptr<float>();
  a.M = aq.size(0), a.N = bq.size(0), a.K = aq.size(1);
  a.C = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  a.ldc = out.stride(0);
  if (out2.has_value()) {
    TORCH_CHECK(out2->sizes() == out.sizes() && out2->stride(0) == out.stride(0), "out2 layout");
    a.C2 = reinterpret_cast<__nv_bfloat16*>(out2->data_ptr());
  }
  a.status = status.data_ptr<int>();
  const char* err = nc::gemm_fp8_blockscaled(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
}

// x bf16 [R, K] -> (xq uint8 [R, K], scale atoms uint8); tile_rows = 128 for the A operand, mx_tile_n(N) for B
std::vector<Tensor> fp8_mx_quantize(const Tensor& x, int64_t tile_rows) {
  const c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.stride(1) == 1, "x must be bf16 [R, K]");
  const int R = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 128 == 0, "K must be a multiple of 128");
  Tensor q = torch::empty({R, K}, x.options().dtype(torch::kUInt8));
  Tensor sf = torch::empty({nc::mxfp8_scale_bytes(R, K, static_cast<int>(tile_rows))}, x.options().dtype(torch::kUInt8));
  const char* err = nc::quantize_mxfp8(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0),
                                       q.data_ptr<uint8_t>(), sf.data_ptr<uint8_t>(), R, K, static_cast<int>(tile_rows),
                                       at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
  return {q, sf};
}

void fp8_mx_gemm(const Tensor& aq, const Tensor& sfa, const Tensor& bq, const Tensor& sfb, Tensor& out,
                 const c10::optional<Tensor>& out2, Tensor status, int64_t variant) {
  const c10::cuda::CUDAGuard g(aq.device());
  TORCH_CHECK(aq.is_contiguous() && bq.is_contiguous() && aq.scalar_type() == torch::kUInt8 &&
                  bq.scalar_type() == torch::kUInt8 && aq.dim() == 2 && bq.dim() == 2 && aq.size(1) == bq.size(1),
              "fp8 operands must be contiguous uint8 [rows, K]");
  const int M = aq.size(0), N = bq.size(0), K = aq.size(1);
  TORCH_CHECK(sfa.is_contiguous() && sfa.scalar_type() == torch::kUInt8 && sfa.numel() == nc::mxfp8_scale_bytes(M, K, 128),
              "scale atoms of A: expected tile_rows = 128");
  TORCH_CHECK(sfb.is_contiguous() && sfb.scalar_type() == torch::kUInt8 &&
                  sfb.numel() == nc::mxfp8_scale_bytes(N, K, nc::mxfp8_tile_n(N)),
              "scale atoms of B: expected tile_rows = fp8_mx_tile_n(N)");
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == M &&
                  out.size(1) == N,
              "out must be bf16 [M, N]");
  nc::MxGemmArgs a;
  a.A = aq.data_ptr<uint8_t>(), a.B = bq.data_ptr<uint8_t>();
  a.sfa = sfa.data_ptr<uint8_t>(), a.sfb = sfb.data_ptr<uint8_t>();
  a.M = M, a.N = N, a.K = K;
  a.C = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  a.ldc = out.stride(0);
  if (out2.has_value()) {
    TORCH_CHECK(out2->sizes() == out.sizes() && out2->stride(0) == out.stride(0) && out2->scalar_type() == torch::kBFloat16,
                "out2 layout");
    a.C2 = reinterpret_cast<__nv_bfloat16*>(out2->data_ptr());
  }
  a.status = status.data_ptr<int>();
  a.variant = static_cast<int>(variant);
  const char* err = nc::gemm_mxfp8(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
}

}  // namespace

void register_fp8(pybind11::module_& m) {
  m.def("fp8_quantize_rows", &fp8_quantize_rows);
  m.def("fp8_quantize_blocks", &fp8_quantize_blocks);
  m.def("fp8_gemm", &fp8_gemm);
  m.def("fp8_mx_quantize", &fp8_mx_quantize);
  m.def("fp8_mx_gemm", &fp8_mx_gemm, pybind11::arg("aq"), pybind11::arg("sfa"), pybind11::arg("bq"), pybind11::arg("sfb"),
        pybind11::arg("out"), pybind11::arg("out2"), pybind11::arg("status"), pybind11::arg("variant") = 0);
  m.def("fp8_mx_tile_n", [](int64_t n) { return nc::mxfp8_tile_n(static_cast<int>(n)); });
}
