"""The layout of the bf16 reduce-scatter (parallel.fused.plan_reduce_scatter), checked on the CPU by emulating all
ranks: every rank "pushes" the elements other ranks own into the owners' receive slots, every owner sums its own
fp32 values with the received bf16 values in rank order. Every element of every parameter must be owned exactly
once, and the owner's result must equal the direct sum with the peers' contributions rounded to bf16."""
import pytest
import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.models.params import ParamStore
from nanochat_cpp_b200.parallel.dp import assign_owners
from nanochat_cpp_b200.parallel.fused import plan_reduce_scatter


@pytest.mark.parametrize("world", [2, 3, 8])
def test_plan_covers_every_element_once_and_reduces_right(world):
    cfg = Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=64, seq_len=32, vocab_size=250,
                 padded_vocab_size=256, window_pattern="SSSL")
    store = ParamStore(cfg, "cpu", torch.bfloat16)
    owners = assign_owners(store, world)
    L = cfg.num_layers
    placed, cap = plan_reduce_scatter(store.specs, owners, world, L)
    g = torch.Generator().manual_seed(world)
    grads = [torch.randn(store.total, generator=g) * 1e-2 for _ in range(world)]
    # coverage: the owned runs of all ranks tile the parameters exactly
    seen = torch.zeros(store.total, dtype=torch.int32)
    for r in range(world):
        last_pos = -1
        for b in range(L + 2):
            for off, cnt, pos in placed[r][b]:
                seen[off:off + cnt] += 1
                assert pos % 8 == 0 and pos > last_pos and pos + cnt <= cap
                last_pos = pos
    is_param = torch.zeros(store.total, dtype=torch.bool)
    for s in store.specs:
        is_param[s.offset:s.offset + s.count] = True
    assert torch.equal(seen[is_param], torch.ones(int(is_param.sum()), dtype=torch.int32))
    assert int(seen[~is_param].sum()) == 0
    # emulate: push (bf16) into recv[owner][src], then the owner's ordered sum
    recv = [[torch.zeros(cap, dtype=torch.bfloat16) for _ in range(world)] for _ in range(world)]
    for src in range(world):
        for owner in range(world):
            if owner == src:
                continue
            for b in range(L + 2):
                for off, cnt, pos in placed[owner][b]:
                    recv[owner][src][pos:pos + cnt] = grads[src][off:off + cnt].to(torch.bfloat16)
    for owner in range(world):
        for b in range(L + 2):
            for off, cnt, pos in placed[owner][b]:
                acc = torch.zeros(cnt)
                want = torch.zeros(cnt)
                for r in range(world):
                    if r == owner:
                        acc += grads[r][off:off + cnt]
                        want += grads[r][off:off + cnt]
                    else:
                        acc += recv[owner][r][pos:pos + cnt].float()
                        want += grads[r][off:off + cnt].to(torch.bfloat16).float()
                assert torch.equal(acc, want)
                exact = sum(grads[r][off:off + cnt] for r in range(world))
                assert (acc - exact).abs().max() <= 2 ** -8 * sum(gr[off:off + cnt].abs() for gr in grads).max() + 1e-12
