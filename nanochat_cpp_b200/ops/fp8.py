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


# ================================================================================================ MXFP8
# E4M3 values with one power-of-two scale (UE8M0 byte, value 2^(b - 127)) per row and 32 consecutive K elements.
# The tensor core applies the scales itself (tcgen05.mma kind::mxf8f6f4.block_scale, `csrc/cuda/fp8_mx.cu`), so
# the whole K extent accumulates in tensor memory and no promotion pass on the CUDA cores is needed.
MX_BLOCK = 32


def ref_mx_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [R, K] -> (q float8_e4m3fn [R, K], biased exponents uint8 [R, K/32]).

    The scale of a block is the smallest power of two >= amax / 448 (exponent byte 127 for an all-zero block).
    """
    R, K = x.shape
    xb = x.float().view(R, K // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(-1)
    bits = (amax * (1.0 / E4M3_MAX)).view(torch.int32)
    eb = (bits >> 23) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    eb = torch.where(amax > 0, eb.clamp(1, 253), torch.full_like(eb, 127))
    inv = ((254 - eb) << 23).view(torch.float32)
    q = (xb * inv.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(R, K), eb.to(torch.uint8)


def ref_mx_dequantize(q: torch.Tensor, eb: torch.Tensor) -> torch.Tensor:
    R, K = q.shape
    scale = torch.exp2(eb.float() - 127.0)
    return (q.float().view(R, K // MX_BLOCK, MX_BLOCK) * scale.unsqueeze(-1)).view(R, K)


def mx_scales_from_atoms(sf: torch.Tensor, R: int, K: int, tile_rows: int) -> torch.Tensor:
    """Undo the kernel's scale layout: atoms uint8 -> biased exponents uint8 [R, K/32] (for tests and debugging).

    One 512-byte atom holds 128 rows x 4 scales at byte (r % 32) * 16 + (r // 32) * 4 + k32; atoms are ordered
    [row tile][128-deep K block][128-row group inside the tile].
    """
    kbs = K // 128
    atoms_per_tile = (tile_rows + 127) // 128
    tiles = (R + tile_rows - 1) // tile_rows
    a = sf.view(tiles, kbs, atoms_per_tile, 32, 4, 4)            # [tile, kb, atom, r % 32, r // 32, k32]
    a = a.permute(0, 2, 4, 3, 1, 5).reshape(tiles, atoms_per_tile * 128, kbs * 4)
    return a[:, :tile_rows].reshape(tiles * tile_rows, kbs * 4)[:R].contiguous()


def mx_tile_n(n: int) -> int:
    """Width of the GEMM's B tile for an output of n columns; the scale atoms of a weight are grouped by it."""
    from . import cuda as K
    return int(K._C.fp8_mx_tile_n(n))


def mx_quantize(x: torch.Tensor, tile_rows: int = 128):
    """bf16 [R, K] -> (uint8 e4m3 [R, K], scale atoms uint8). tile_rows: 128 for activations, mx_tile_n(N) for weights."""
    from . import cuda as K
    q, sf = K._C.fp8_mx_quantize(x, tile_rows)
    return q, sf


def mx_gemm(xq, sfx, wq, sfw, out: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None,
            variant: int = 0):
    """bf16 [M, N] = xq [M, K] x wq [N, K]^T with both operands' scales applied by the MMA; `out2` receives
    relu(out)^2 (pass out2 = out to keep only the activation). variant: 0 = CTA pairs computing 256-row tiles
    when M > 128, 1 = one CTA per 128-row tile, 2 = CTA pairs."""
    from . import cuda as K
    if out is None:
        out = torch.empty((xq.shape[0], wq.shape[0]), dtype=torch.bfloat16, device=xq.device)
    K._C.fp8_mx_gemm(xq, sfx, wq, sfw, out, out2, K._C.status_tensor(xq.device.index), variant)
    return out


class MxWeight:
    """A weight [N, K] kept as MXFP8 (values + scale atoms grouped by the GEMM's B tile); refresh after every update."""

    def __init__(self, w: torch.Tensor):
        self.tile_n = mx_tile_n(w.shape[0])
        self.q, self.s = mx_quantize(w, self.tile_n)

    def refresh(self, w: torch.Tensor) -> None:
        self.q, self.s = mx_quantize(w, self.tile_n)


def linear_fwd_mx(x: torch.Tensor, w: MxWeight, relu2: bool = False):
    xq, sx = mx_quantize(x, 128)
    if relu2:
        pre = torch.empty((x.shape[0], w.q.shape[0]), dtype=torch.bfloat16, device=x.device)
        act = torch.empty_like(pre)
        mx_gemm(xq, sx, w.q, w.s, pre, act)
        return pre, act
    return mx_gemm(xq, sx, w.q, w.s)
