"""Muon on the GPU: fused elementwise stages + batched tcgen05 products.

Same arithmetic as `ops.ref.muon_update` (reference `backends/cpu/kernels.cc:1614-1810`) with the
Polar Express iterate kept in bf16 between products, as the reference's bf16 CUDA build does
(docs/model.md:402-416). Per shape group `[P, rows, cols]`:

  1. `muon_nesterov`  momentum + Nesterov blend, per-row sum of squares         (1 launch / matrix)
  2. `muon_prescale`  row equilibration + Frobenius normalisation as one row scale (1 launch, one CTA / matrix)
  3. `muon_scale_rows` applies it and writes the bf16 iterate                   (1 launch / matrix)
  4. 5 x { A = X X^T (or X^T X), B = b A + c A A, X = a X + B X (or X B) }      (3 batched GEMMs / step,
     residual-add epilogue, no separate axpby passes)
  5. `muon_line_sumsq` + `muon_poststats`: Muon+ rescale, NorMuon second moment and per-line step (2 launches)
  6. `muon_apply`  cautious decay + update of the fp32 master and bf16 copy     (1 launch / matrix)
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops.ref import POLAR_COEFFS


def polar_express_bf16(X: torch.Tensor, ns_steps: int) -> torch.Tensor:
    """X: [P, rows, cols] bf16, normalised. Returns the orthogonalised stack (bf16)."""
    from ..ops import cuda as K
    P, rows, cols = X.shape
    tall = rows > cols
    k = cols if tall else rows
    A = torch.empty(P, k, k, dtype=torch.bfloat16, device=X.device)
    B = torch.empty_like(A)
    Y = torch.empty_like(X)
    for it in range(min(max(ns_steps, 0), 5)):
        ca, cb, cc = POLAR_COEFFS[it]
        if tall:
            K.gemm(X, X, a_mn=True, b_mn=True, out=A)                       # X^T X
            K.gemm(A, A, epi=K.EPI_BF16_RES, r=A, alpha=cc, beta=cb, out=B)  # b A + c A A   (A symmetric)
            K.gemm(X, B, epi=K.EPI_BF16_RES, r=X, alpha=1.0, beta=ca, out=Y)  # a X + X B     (B symmetric)
        else:
            K.gemm(X, X, out=A)                                              # X X^T
            K.gemm(A, A, epi=K.EPI_BF16_RES, r=A, alpha=cc, beta=cb, out=B)
            K.gemm(B, X, b_mn=True, epi=K.EPI_BF16_RES, r=X, alpha=1.0, beta=ca, out=Y)  # a X + B X
        X, Y = Y, X
    return X


class MuonGroupState:
    """Scratch of one shape group, allocated once."""

    def __init__(self, P: int, rows: int, cols: int, device):
        self.x32 = torch.empty(P, rows, cols, dtype=torch.float32, device=device)
        self.X = torch.empty(P, rows, cols, dtype=torch.bfloat16, device=device)
        self.row_ss = torch.empty(P, rows, dtype=torch.float32, device=device)
        self.row_scale = torch.empty(P, rows, dtype=torch.float32, device=device)
        self.all_scale = torch.empty(P, dtype=torch.float32, device=device)
        lines = rows if rows >= cols else cols
        self.scale = torch.empty(P, dtype=torch.float32, device=device)
        self.line_scale = torch.empty(P, lines, dtype=torch.float32, device=device)
        self._tables = {}

    def table(self, key: str, tensors, values=None) -> torch.Tensor:
        """Device array of the tensors' addresses (or of the given integers), cached while they stay the same."""
        ptrs = tuple(values) if values is not None else tuple(t.data_ptr() for t in tensors)
        hit = self._tables.get(key)
        if hit is None or hit[0] != ptrs:
            hit = (ptrs, torch.tensor(ptrs, dtype=torch.int64, device=self.x32.device))
            self._tables[key] = hit
        return hit[1]


@torch.no_grad()
def muon_group_step(grads: List[torch.Tensor], masters: List[torch.Tensor], values: List[Optional[torch.Tensor]],
                    buf1: List[torch.Tensor], buf2: List[torch.Tensor], scratch: MuonGroupState, *, lr: float,
                    momentum: float, beta2: float, weight_decay: float, ns_steps: int,
                    grad_scale: Optional[torch.Tensor], apply_fn=None) -> None:
    """`apply_fn(p, master, X_p, scale_p, line_scale_p, lines_are_rows, lr, wd)` replaces the final update
    launch (the data-parallel engine uses it to push the new parameters to every rank)."""
    from ..ops import cuda as K
    C = K._C
    P = len(grads)
    rows, cols = masters[0].shape
    reduce_cols = rows >= cols
    gs = None if grad_scale is None else grad_scale.reshape(1)
    batched = cols % 8 == 0 and all(t.is_contiguous() for t in grads) and all(t.is_contiguous() for t in buf1)
    if batched:
        C.muon_nesterov_batched(scratch.table("g", grads), scratch.table("b1", buf1), scratch.x32[:P],
                                scratch.row_ss[:P], momentum, gs)
    else:
        for p in range(P):
            C.muon_nesterov(grads[p], buf1[p], scratch.x32[p], scratch.row_ss[p], momentum, gs)
    row_ss = scratch.row_ss[:P]
    row_scale, all_scale = scratch.row_scale[:P], scratch.all_scale[:P]
    C.muon_prescale(row_ss, row_scale, all_scale)
    if batched:
        C.muon_scale_rows_batched(scratch.x32[:P], row_scale, all_scale, scratch.X[:P])
    else:
        for p in range(P):
            C.muon_scale_rows(scratch.x32[p], row_scale[p], all_scale[p:p + 1], scratch.X[p])
    X = polar_express_bf16(scratch.X[:P], ns_steps)
    red = -1 if reduce_cols else -2
    line_len = cols if reduce_cols else rows
    if batched and X.is_contiguous():
        line_ss = C.muon_line_sumsq(X, reduce_cols)             # [P, lines]
    else:
        line_ss = X.float().square().sum(red)
    scale, line_scale = scratch.scale[:P], scratch.line_scale[:P]
    C.muon_poststats(line_ss.contiguous(), scratch.table("b2", buf2), scale, line_scale, line_len,
                     math.sqrt(float(min(rows, cols))), beta2)
    if apply_fn is None and batched and X.is_contiguous() and all(m.is_contiguous() for m in masters):
        vt = scratch.table("v", values) if all(v is not None for v in values) else None
        C.muon_apply_batched(scratch.table("m", masters), vt, X, scale, line_scale, reduce_cols, lr, weight_decay)
        return
    batch_fn = getattr(apply_fn, "batched", None)
    if batch_fn is not None and batched and X.is_contiguous() and all(m.is_contiguous() for m in masters):
        batch_fn(scratch, masters, X, scale, line_scale, reduce_cols, lr, weight_decay)     # one launch for the group
        return
    for p in range(P):
        if apply_fn is not None:
            apply_fn(p, masters[p], X[p], scale[p:p + 1], line_scale[p], reduce_cols, lr, weight_decay)
        else:
            C.muon_apply(masters[p], values[p], X[p], scale[p:p + 1], line_scale[p], reduce_cols, lr, weight_decay)
