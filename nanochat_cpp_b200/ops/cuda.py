"""CUDA implementations of the operators: wrappers over the compiled extension `_C`.

Importing this module loads `nanochat_cpp_b200/_C.so`; it raises if the file is missing so that a
GPU run can never continue on a silent PyTorch fallback.
"""
from __future__ import annotations

import importlib.util
import os

import torch

from . import ref

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_HERE, "_C.so")


def _load():
    if not os.path.exists(_SO):
        raise RuntimeError(f"{_SO} is not built: run `python -m nanochat_cpp_b200.build` "
                           "(the CUDA operators have no PyTorch fallback on a GPU)")
    spec = importlib.util.spec_from_file_location("nanochat_cpp_b200._C", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_C = _load()

EPI_BF16, EPI_BF16_RES, EPI_RELU2, EPI_DRELU2, EPI_F32 = 0, 1, 2, 3, 4


def check_status(device=None) -> None:
    """Raise if any kernel recorded a bounded-wait failure. Synchronizes the device."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    code = _C.read_status(dev)
    if code != 0:
        _C.reset_status(dev)
        raise RuntimeError(f"a kernel gave up waiting (status code {code}); see csrc/cuda/ptx.cuh")


# ---------------------------------------------------------------------------
# GEMMs
# ---------------------------------------------------------------------------
def gemm(a, b, *, a_mn=False, b_mn=False, epi=EPI_BF16, out=None, r=None, out2=None, alpha=1.0, beta=0.0,
         split_k=True):
    """out = epilogue(A x B^T). See csrc/cuda/bindings.cpp for operand orders."""
    m = a.shape[-1] if a_mn else a.shape[-2]
    n = b.shape[-1] if b_mn else b.shape[-2]
    if out is None:
        shape = (*a.shape[:-2], m, n)
        out = torch.empty(shape, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    _C.gemm(a, b, out, a_mn, b_mn, epi, r, out2, alpha, beta, split_k)
    return out


def linear_fwd(x, w, *, out=None, residual=None):
    if residual is not None:
        return gemm(x, w, epi=EPI_BF16_RES, r=residual, out=out, alpha=1.0, beta=1.0)
    return gemm(x, w, out=out)


def linear_relu2_fwd(x, w):
    pre = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    act = torch.empty_like(pre)
    gemm(x, w, epi=EPI_RELU2, out=pre, out2=act)
    return pre, act


def linear_dgrad(dy, w, *, residual=None):
    # dx[M,K] = dy[M,N] @ w[N,K]: B operand is w read MN-major (its K index is contiguous)
    if residual is not None:
        return gemm(dy, w, b_mn=True, epi=EPI_BF16_RES, r=residual, alpha=1.0, beta=1.0)
    return gemm(dy, w, b_mn=True)


def linear_dgrad_relu2(dy, w, pre):
    return gemm(dy, w, b_mn=True, epi=EPI_DRELU2, r=pre)


def linear_wgrad(dy, x, grad, *, accumulate=True):
    # grad[N,K] (+)= dy[M,N]^T @ x[M,K]: both operands are read MN-major
    gemm(dy, x, a_mn=True, b_mn=True, epi=EPI_F32, out=grad, beta=1.0 if accumulate else 0.0)
    return grad


def __getattr__(name):
    # Operators without a kernel yet are an error on a GPU, not a fallback.
    raise AttributeError(f"ops.cuda has no operator {name!r}")
