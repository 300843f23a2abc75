// Tensor-level wrappers of the communication kernels. Peer buffers are passed as lists of raw device
// addresses (one per rank, as handed out by the symmetric-memory rendezvous).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"

namespace {

using torch::Tensor;
inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream(); }

nc::PeerPtrs to_peers(const std::vector<int64_t>& ptrs, int64_t multicast_ptr = 0) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= nc::kMaxRanks, "between 1 and 8 ranks are supported");
  nc::PeerPtrs p;
  for (int i = 0; i < nc::kMaxRanks; ++i) p.p[i] = nullptr;
  for (size_t i = 0; i < ptrs.size(); ++i) p.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
  p.mc = reinterpret_cast<void*>(static_cast<uintptr_t>(multicast_ptr));
  return p;
}

void comm_signal(const std::vector<int64_t>& flag_ptrs, int64_t my_rank, int64_t slot, int64_t value) {
  nc::comm_signal(to_peers(flag_ptrs), static_cast<int>(flag_ptrs.size()), my_rank, slot, value, cur());
}

void comm_wait(const Tensor& flags, int64_t world, int64_t slot, int64_t value, Tensor status, int64_t budget_ms) {
  const c10::cuda::CUDAGuard g(flags.device());
  nc::comm_wait(flags.data_ptr<int>(), world, slot, value, status.data_ptr<int>(), cur(), static_cast<int>(budget_ms));
}

// segs: int64 [nsegs, 2] (offset, count) on the device
void comm_reduce_pull(const std::vector<int64_t>& grad_ptrs, int64_t my_rank, const Tensor& segs, int64_t total,
                      double scale, const Tensor& flags, int64_t slot, int64_t value, Tensor sumsq, Tensor status,
                      int64_t ctas) {
  const c10::cuda::CUDAGuard g(flags.device());
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == torch::kInt64 && segs.is_contiguous() && segs.size(1) == 2,
              "segs must be an int64 [n, 2] CUDA tensor");
  TORCH_CHECK(segs.size(0) <= 64, "reduce_pull takes at most 64 segments per launch");
  static_assert(sizeof(nc::Segment) == 16, "Segment layout");
  nc::comm_reduce_pull(to_peers(grad_ptrs), static_cast<int>(grad_ptrs.size()), my_rank,
                       reinterpret_cast<const nc::Segment*>(segs.data_ptr<int64_t>()), segs.size(0), total, scale,
                       flags.data_ptr<int>(), slot, value, sumsq.data_ptr<double>(), status.data_ptr<int>(), ctas,
                       cur());
}

// segs: int64 [n, 5] on the device (see comm.h)
void comm_grad_push(const Tensor& grad, const std::vector<int64_t>& recv_ptrs, int64_t recv_stride, int64_t my_rank,
                    const Tensor& segs, int64_t nvec, double scale, int64_t ctas) {
  const c10::cuda::CUDAGuard g(grad.device());
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == torch::kInt64 && segs.is_contiguous() && segs.dim() == 2 &&
                  segs.size(1) == 5 && segs.size(0) <= 128, "grad_push: segs must be int64 [n <= 128, 5]");
  TORCH_CHECK(grad.scalar_type() == torch::kFloat32 && grad.is_contiguous(), "grad_push: fp32 contiguous gradient");
  nc::comm_grad_push(grad.data_ptr<float>(), to_peers(recv_ptrs), recv_stride, my_rank,
                     reinterpret_cast<const long long*>(segs.data_ptr<int64_t>()), segs.size(0), nvec, scale, ctas, cur());
}

// segs: int64 [n, 4] on the device (see comm.h)
void comm_grad_reduce_local(Tensor& grad, const Tensor& recv, int64_t recv_stride, int64_t world, int64_t my_rank,
                            const Tensor& segs, int64_t nvec, double scale, const Tensor& flags, int64_t slot,
                            int64_t value, Tensor sumsq, Tensor status, int64_t ctas) {
  const c10::cuda::CUDAGuard g(grad.device());
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == torch::kInt64 && segs.is_contiguous() && segs.dim() == 2 &&
                  segs.size(1) == 4 && segs.size(0) <= 64, "grad_reduce_local: segs must be int64 [n <= 64, 4]");
  TORCH_CHECK(recv.scalar_type() == torch::kBFloat16 && recv.numel() >= world * recv_stride, "grad_reduce_local: recv");
  nc::comm_grad_reduce_local(grad.data_ptr<float>(), reinterpret_cast<const __nv_bfloat16*>(recv.data_ptr()),
                             recv_stride, world, my_rank, reinterpret_cast<const long long*>(segs.data_ptr<int64_t>()),
                             segs.size(0), nvec, scale, flags.data_ptr<int>(), slot, value, sumsq.data_ptr<double>(),
                             status.data_ptr<int>(), ctas, cur());
}

void comm_adamw_push(Tensor& master, const std::vector<int64_t>& value_ptrs, int64_t value_offset, const Tensor& grad,
                     Tensor& m, Tensor& v, double lr, double beta1, double beta2, double eps, double weight_decay,
                     int64_t step, const c10::optional<Tensor>& grad_scale, int64_t multicast_ptr, int64_t max_ctas) {
  const c10::cuda::CUDAGuard g(master.device());
  TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw_push");
  nc::comm_adamw_push(master.data_ptr<float>(), to_peers(value_ptrs, multicast_ptr), value_offset,
                      static_cast<int>(value_ptrs.size()), grad.data_ptr<float>(), m.data_ptr<float>(),
                      v.data_ptr<float>(), master.numel(), lr, beta1, beta2, eps, weight_decay, step,
                      grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, cur(), static_cast<int>(max_ctas));
}

void comm_muon_apply_push(Tensor& master, const std::vector<int64_t>& value_ptrs, int64_t value_offset,
                          const Tensor& xb, const Tensor& scale0, const Tensor& line_scale, bool lines_are_rows,
                          double lr, double wd, int64_t multicast_ptr) {
  const c10::cuda::CUDAGuard g(master.device());
  TORCH_CHECK(master.dim() == 2 && master.is_contiguous() && xb.is_contiguous() && master.size(1) % 2 == 0,
              "muon_apply_push");
  nc::comm_muon_apply_push(master.data_ptr<float>(), to_peers(value_ptrs, multicast_ptr), value_offset,
                           static_cast<int>(value_ptrs.size()), reinterpret_cast<const __nv_bfloat16*>(xb.data_ptr()),
                           scale0.data_ptr<float>(), line_scale.data_ptr<float>(), lines_are_rows, master.size(0),
                           master.size(1), lr, wd, cur());
}

void comm_muon_apply_push_batched(const Tensor& master_ptrs, const Tensor& value_offsets,
                                  const std::vector<int64_t>& value_ptrs, const Tensor& xb, const Tensor& scale0,
                                  const Tensor& line_scale, bool lines_are_rows, double lr, double wd,
                                  int64_t multicast_ptr) {
  const c10::cuda::CUDAGuard g(xb.device());
  TORCH_CHECK(xb.dim() == 3 && xb.is_contiguous() && xb.size(2) % 8 == 0 && master_ptrs.numel() == xb.size(0) &&
                  value_offsets.numel() == xb.size(0) && master_ptrs.scalar_type() == torch::kInt64 &&
                  value_offsets.scalar_type() == torch::kInt64 && scale0.is_contiguous() && line_scale.is_contiguous(),
              "muon_apply_push_batched");
  nc::comm_muon_apply_push_batched(reinterpret_cast<const long long*>(master_ptrs.data_ptr<int64_t>()),
                                   reinterpret_cast<const long long*>(value_offsets.data_ptr<int64_t>()),
                                   to_peers(value_ptrs, multicast_ptr), static_cast<int>(value_ptrs.size()),
                                   reinterpret_cast<const __nv_bfloat16*>(xb.data_ptr()), scale0.data_ptr<float>(),
                                   line_scale.data_ptr<float>(), lines_are_rows, xb.size(0), xb.size(1), xb.size(2), lr,
                                   wd, cur());
}

}  // namespace

void register_comm(pybind11::module_& m) {
  m.def("comm_signal", &comm_signal);
  m.def("comm_wait", &comm_wait, pybind11::arg("flags"), pybind11::arg("world"), pybind11::arg("slot"),
        pybind11::arg("value"), pybind11::arg("status"), pybind11::arg("budget_ms") = 0);
  m.def("comm_reduce_pull", &comm_reduce_pull);
  m.def("comm_grad_push", &comm_grad_push);
  m.def("comm_grad_reduce_local", &comm_grad_reduce_local);
  m.def("comm_adamw_push", &comm_adamw_push, pybind11::arg("master"), pybind11::arg("value_ptrs"),
        pybind11::arg("value_offset"), pybind11::arg("grad"), pybind11::arg("m"), pybind11::arg("v"), pybind11::arg("lr"),
        pybind11::arg("beta1"), pybind11::arg("beta2"), pybind11::arg("eps"), pybind11::arg("weight_decay"),
        pybind11::arg("step"), pybind11::arg("grad_scale"), pybind11::arg("multicast_ptr") = 0,
        pybind11::arg("max_ctas") = 0);
  m.def("comm_muon_apply_push", &comm_muon_apply_push, pybind11::arg("master"), pybind11::arg("value_ptrs"),
        pybind11::arg("value_offset"), pybind11::arg("xb"), pybind11::arg("scale0"), pybind11::arg("line_scale"),
        pybind11::arg("lines_are_rows"), pybind11::arg("lr"), pybind11::arg("wd"), pybind11::arg("multicast_ptr") = 0);
  m.def("comm_muon_apply_push_batched", &comm_muon_apply_push_batched, pybind11::arg("master_ptrs"),
        pybind11::arg("value_offsets"), pybind11::arg("value_ptrs"), pybind11::arg("xb"), pybind11::arg("scale0"),
        pybind11::arg("line_scale"), pybind11::arg("lines_are_rows"), pybind11::arg("lr"), pybind11::arg("wd"),
        pybind11::arg("multicast_ptr") = 0);
}
