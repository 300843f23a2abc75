"""Block-scaled fp8 (E4M3) linear layers: quantizers, the two-level-accumulation GEMM, and their PyTorch
definitions.

Scaling granularity: one fp32 scale per activation row and 128-wide K block, one per 128 x 128 weight block
(scale = amax / 448). The reference scales per tensor through cublasLt (docs/precision.md:236-297); fine-grained
scales keep outliers local and need the promotion kernel in `csrc/cuda/fp8.cu`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

E4M3_MAX = 448.0


# ------------------------------------------------------------------------------------------------ definitions
def ref_quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] -> (q float8_e4m3fn [M, K], scales fp32 [K/128, M])."""
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    amax = xb.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xb * (1.0 / scale).unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(M, K), scale.t().contiguous()


def ref_quantize_blocks(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] -> (q float8_e4m3fn [N, K], scales fp32 [N/128, K/128])."""
    N, K = w.shape
    wb = w.float().view(N // 128, 128, K // 128, 128)
    amax = wb.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (wb * (1.0 / scale)[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(N, K), scale.contiguous()


def ref_dequantize_rows(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * scales.t().unsqueeze(-1)).view(M, K)


def ref_dequantize_blocks(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    return (q.float().view(N // 128, 128, K // 128, 128) * scales[:, None, :, None]).view(N, K)


def ref_fp8_linear(xq, sx, wq, sw) -> torch.Tensor:
    """fp32 result of the block-scaled product (what the kernel rounds to bf16)."""
    return ref_dequantize_rows(xq, sx) @ ref_dequantize_blocks(wq, sw).t()


# ------------------------------------------------------------------------------------------------ kernels
def quantize_rows(x: torch.Tensor):
    from . import cuda as K
    q, s = K._C.fp8_quantize_rows(x)
    return q, s


def quantize_blocks(w: torch.Tensor):
    from . import cuda as K
    q, s = K._C.fp8_quantize_blocks(w)
    return q, s


def fp8_gemm(xq, sx, wq, sw, out: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None):
    """bf16 [M, N] = block-scaled xq [M, K] x wq [N, K]^T; `out2`, when given, receives relu(out)^2."""
    from . import cuda as K
    if out is None:
        out = torch.empty((xq.shape[0], wq.shape[0]), dtype=torch.bfloat16, device=xq.device)
    K._C.fp8_gemm(xq, sx, wq, sw, out, out2, K._C.status_tensor(xq.device.index))
    return out


class Fp8Weight:
    """A weight kept in E4M3 with its block scales; re-quantized after every optimizer step."""

    def __init__(self, w: torch.Tensor):
        self.q, self.s = quantize_blocks(w)

    def refresh(self, w: torch.Tensor) -> None:
        self.q, self.s = quantize_blocks(w)


def linear_fwd_fp8(x: torch.Tensor, w: Fp8Weight, relu2: bool = False):
    xq, sx = quantize_rows(x)
    if relu2:
        pre = torch.empty((x.shape[0], w.q.shape[0]), dtype=torch.bfloat16, device=x.device)
        act = torch.empty_like(pre)
        fp8_gemm(xq, sx, w.q, w.s, pre, act)
        return pre, act
    return fp8_gemm(xq, sx, w.q, w.s)
