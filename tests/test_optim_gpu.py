"""GPU Muon (batched kernels + bf16 Newton-Schulz on tcgen05) against the fp32 PyTorch definition."""
import pytest
import torch

from nanochat_cpp_b200.ops import ref
from nanochat_cpp_b200.optim.muon_cuda import MuonGroupState, muon_group_step

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P,rows,cols", [(3, 256, 256), (2, 512, 128), (2, 128, 512)])
def test_muon_group_step_matches_definition(P, rows, cols):
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    lines = rows if rows >= cols else cols
    grads = [torch.randn(rows, cols, device="cuda", generator=g) * 1e-2 for _ in range(P)]
    masters = [torch.randn(rows, cols, device="cuda", generator=g) * 0.05 for _ in range(P)]
    values = [m.to(torch.bfloat16) for m in masters]
    buf1 = [torch.randn(rows, cols, device="cuda", generator=g) * 1e-3 for _ in range(P)]
    buf2 = [torch.rand(lines, device="cuda", generator=g) * 1e-3 + 1e-4 for _ in range(P)]
    rm, rb1, rb2 = torch.stack(masters).clone(), torch.stack(buf1).clone(), torch.stack(buf2).clone()
    before = torch.stack(masters).clone()
    kw = dict(lr=0.02, momentum=0.9, beta2=0.9, weight_decay=0.1, ns_steps=5)
    scale = torch.tensor(0.5, device="cuda")
    ref.muon_update(torch.stack(grads), rm, None, rb1, rb2, grad_scale=scale, **kw)
    muon_group_step(grads, masters, values, buf1, buf2, MuonGroupState(P, rows, cols, "cuda"), grad_scale=scale, **kw)
    got, want = torch.stack(masters) - before, rm - before
    rel = float((got - want).norm() / want.norm())
    assert rel < 3e-2, rel                                   # the iterate lives in bf16 between products
    assert torch.allclose(torch.stack(buf1), rb1, atol=1e-6)
    assert float((torch.stack(buf2) - rb2).norm() / rb2.norm()) < 2e-2
    for m, v in zip(masters, values):
        assert torch.equal(v, m.to(torch.bfloat16))


@pytest.mark.parametrize("P,rows,cols", [(10, 10, 12), (1, 1, 24), (3, 12, 10), (2, 32, 32)])
def test_one_launch_muon_step_of_small_matrices(P, rows, cols):
    """The gate projections: one launch for the whole group's step, fp32, against the definition."""
    from nanochat_cpp_b200.ops import cuda as K
    g = torch.Generator(device="cuda").manual_seed(rows * 100 + cols)
    lines = rows if rows >= cols else cols
    grads = [torch.randn(rows, cols, device="cuda", generator=g) * 1e-2 for _ in range(P)]
    masters = [torch.randn(rows, cols, device="cuda", generator=g) * 0.05 for _ in range(P)]
    values = [torch.zeros(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    buf1 = [torch.randn(rows, cols, device="cuda", generator=g) * 1e-3 for _ in range(P)]
    buf2 = [torch.rand(lines, device="cuda", generator=g) * 1e-3 + 1e-4 for _ in range(P)]
    rm, rb1, rb2 = torch.stack(masters).clone(), torch.stack(buf1).clone(), torch.stack(buf2).clone()
    before = torch.stack(masters).clone()
    scale = torch.tensor(0.5, device="cuda")
    ref.muon_update(torch.stack(grads), rm, None, rb1, rb2, grad_scale=scale, lr=0.02, momentum=0.9, beta2=0.9,
                    weight_decay=0.1, ns_steps=5)
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")
    n0 = K.launch_count()
    K._C.muon_tiny(tab(grads), tab(buf1), tab(buf2), tab(masters), tab(values), rows, cols, 0.9, 0.9, 0.02, 0.1, 5,
                   scale.reshape(1), [list(c) for c in ref.POLAR_COEFFS])
    assert K.launch_count() - n0 == 1
    got, want = torch.stack(masters) - before, rm - before
    assert float((got - want).norm() / want.norm()) < 1e-3
    assert torch.allclose(torch.stack(buf1), rb1, atol=1e-7)
    assert torch.allclose(torch.stack(buf2), rb2, rtol=1e-3, atol=1e-9)
    for p in range(P):
        assert torch.equal(values[p], masters[p].to(torch.bfloat16))
    with pytest.raises(RuntimeError, match="at most 1024"):
        K._C.muon_tiny(tab(grads), tab(buf1), tab(buf2), tab(masters), None, 64, 64, 0.9, 0.9, 0.02, 0.1, 5, None,
                       [list(c) for c in ref.POLAR_COEFFS])
