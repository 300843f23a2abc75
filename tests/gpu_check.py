"""Helpers for the GPU numerics tests: per-element tolerances, canaries around outputs, finite differences.

`close_elementwise` bounds every element separately (|err| <= atol + rtol * |want|): a wrong low-magnitude region, a
dropped factor on a small tensor or a stale tile passes a max-normalised bound but not this one. `guarded` allocates
an output inside a poisoned buffer and checks that the kernel wrote nothing outside its span. `fd_regression` compares
an analytic gradient with central differences of the kernel itself, element by element, on inputs that sit on a
binary grid so that x +/- delta is exactly representable in bf16.
"""
import math

import torch

BF16_EPS = 2.0 ** -8          # spacing of bf16 relative to the value (one unit in the last place)


def close_elementwise(got, want, *, rtol=2 * BF16_EPS, atol=0.0, name="", frac=0.0):
    """Every element within atol + rtol*|want| (`frac` > 0 allows that fraction of outliers: a few elements of a
    long bf16 accumulation can land one rounding step away from the fp32 result)."""
    got, want = got.float(), want.float()
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    bad = err > bound
    n_bad = int(bad.sum())
    if n_bad > frac * err.numel():
        i = int(torch.argmax(err - bound))
        raise AssertionError(f"{name}: {n_bad} of {err.numel()} elements out of tolerance; worst at flat index {i}: "
                             f"got {got.reshape(-1)[i].item():.6g} want {want.reshape(-1)[i].item():.6g} "
                             f"bound {bound.reshape(-1)[i].item():.3g}")


def dot_atol(a_absmax: float, b_absmax: float, k: int, out_dtype=torch.bfloat16) -> float:
    """Absolute slack for one element of a K-term product whose result may be ~0 by cancellation: the output is a
    rounding of a sum whose partial sums reach sqrt(K) * |a||b|, so an fp32 accumulation in a different order moves
    it by about sqrt(K) * 2^-24 of that, and a bf16 intermediate (split-K partials, residual) by 2^-9 of the value
    it rounds."""
    scale = a_absmax * b_absmax * math.sqrt(float(k))
    return scale * (2.0 ** -9 if out_dtype == torch.bfloat16 else 2.0 ** -18)


class guarded:
    """`with guarded(shape, dtype) as g:` gives `g.out` (zeros, a view in the middle of a larger poisoned buffer);
    leaving the block checks that the guard regions before and after it still hold the poison."""

    def __init__(self, shape, dtype, pad=4096, device="cuda"):
        n = 1
        for s in shape:
            n *= s
        self.pad, self.n = pad, n
        self.buf = torch.empty(n + 2 * pad, dtype=dtype, device=device)
        self.poison = 12345.0 if dtype in (torch.float32, torch.bfloat16, torch.float16) else 77
        self.buf.fill_(self.poison)
        self.out = self.buf[pad:pad + n].view(*shape)
        self.out.zero_()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if exc[0] is None:
            lo, hi = self.buf[:self.pad], self.buf[self.pad + self.n:]
            want = torch.full_like(lo, self.poison)
            assert torch.equal(lo, want) and torch.equal(hi, want), "kernel wrote outside its output"
        return False


def on_grid(shape, step=2.0 ** -4, span=1.5, gen=None, device="cuda"):
    """bf16 values that are multiples of `step` in [-span, span]: adding +/- step is exact in bf16."""
    n = int(round(span / step))
    k = torch.randint(-n, n + 1, shape, generator=gen, device=device)
    return (k.float() * step).to(torch.bfloat16)


def fd_regression(loss_fn, x, grad, *, delta=2.0 ** -4, probes=96, gen=None, min_corr=0.97, slope_tol=0.06, name="",
                  block=1, aligned=False):
    """Central differences of `loss_fn()` (a Python float, recomputed by the kernel under test) with respect to
    `probes` random perturbations of the bf16 tensor `x` (modified in place and restored), regressed against the
    analytic gradient `grad`: the slope must be 1 within `slope_tol` and the correlation at least `min_corr`. A
    missing factor shows in the slope, a gradient that lands on the wrong elements in the correlation.

    With `block` > 1 a probe moves `block` consecutive elements by +/- delta with random signs and is compared with
    the same signed sum of the analytic gradient: the signal of a directional derivative grows with the block while
    the rounding noise of the bf16 outputs it is measured through does not. With `aligned` the signs of a probe are
    those of the analytic gradient on the block (times one random sign for the whole probe): the direction with the
    largest derivative, which lets `delta` stay small enough for the function to be linear across the probe. Any
    direction is a valid probe: a wrong gradient still predicts a derivative the kernel does not show."""
    flat = x.view(-1)
    g = grad.reshape(-1).float()
    starts = torch.randint(0, flat.numel() // block, (probes,), generator=gen, device=flat.device) * block
    fd, an = [], []
    for i in starts.tolist():
        old = flat[i:i + block].clone()
        sign = (torch.randint(0, 2, (block,), generator=gen, device=flat.device) * 2 - 1).to(old.dtype)
        if aligned:
            gs = torch.where(g[i:i + block] >= 0, 1.0, -1.0).to(old.dtype)
            sign = gs * sign[0]
        flat[i:i + block] = old + sign * delta
        fp = loss_fn()
        flat[i:i + block] = old - sign * delta
        fm = loss_fn()
        flat[i:i + block] = old
        fd.append((fp - fm) / (2 * delta))
        an.append(float((g[i:i + block] * sign.float()).sum()))
    fd_t, an_t = torch.tensor(fd, dtype=torch.float64), torch.tensor(an, dtype=torch.float64)
    denom = float((an_t * an_t).sum())
    assert denom > 0, f"{name}: analytic gradient is zero at every probe"
    slope = float((fd_t * an_t).sum()) / denom
    corr = float((fd_t * an_t).sum() / (fd_t.norm() * an_t.norm() + 1e-30))
    assert abs(slope - 1.0) <= slope_tol and corr >= min_corr, f"{name}: slope {slope:.4f} correlation {corr:.4f}"
    return slope, corr
