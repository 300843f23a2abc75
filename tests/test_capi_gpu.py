"""The C ABI on a CUDA device: the C++ GPU engine (libnanochat_gpu.so, no Python or PyTorch in its loop) against the
Python package's GPU model on the same weights, the same tokens and the same kernels."""
import numpy as np
import pytest
import torch

from nanochat_cpp_b200 import cpu_engine as E
from nanochat_cpp_b200.config import Config

pytestmark = pytest.mark.gpu


def _cfg():
    return Config(num_layers=4, num_heads=4, num_kv_heads=2, hidden_dim=512, seq_len=256, vocab_size=1000,
                  padded_vocab_size=1024, window_pattern="SSSL")


@pytest.fixture
def cuda_backend():
    E.select_device("cuda:0")
    try:
        yield
    finally:
        E.select_device("cpu")


def _python_model(cfg, seed=5):
    from nanochat_cpp_b200.models import GPT
    m = GPT(cfg, "cuda", torch.bfloat16, seed=seed)
    g = torch.Generator().manual_seed(seed)
    for s in m.params.specs:       # zero-initialised projections would leave most of the graph without gradients
        if s.name.endswith("c_proj.weight"):
            m.params.m(s.name).copy_((torch.randn(s.shape, generator=g) * 0.02).cuda())
    m.params.m("smear_lambda").fill_(0.3)
    m.params.m("lm_head.weight").copy_((torch.randn(cfg.padded_vocab_size, cfg.hidden_dim, generator=g) * 0.05).cuda())
    # both engines start from bf16-representable masters, so their bf16 copies agree bit for bit
    m.params.master.copy_(m.params.master.to(torch.bfloat16).float())
    m.params.sync_compute()
    return m


def _copy_weights(py_model, native):
    for s in py_model.params.specs:
        native.write(s.name, py_model.params.m(s.name).detach().float().cpu().numpy())


def test_backend_and_devices_follow_the_selection(cuda_backend):
    assert E.backend() == "cuda" and E.device_count() >= 1
    E.select_device("cpu")
    assert E.backend() == "cpu" and E.device_count() == 1
    with pytest.raises(RuntimeError):
        E.select_device("cuda:99")


def test_three_training_steps_match_the_python_gpu_path(cuda_backend):
    from nanochat_cpp_b200.ops import cuda as K
    from nanochat_cpp_b200.train import TrainConfig, Trainer
    cfg = _cfg()
    py = _python_model(cfg)
    tr = Trainer(cfg, TrainConfig(batch=4, grad_accum=1, num_iterations=100, seed=5), device="cuda", model=py)
    native = E.NativeModel(cfg, seed=1)
    assert set(native.names()) == {s.name for s in py.params.specs}
    _copy_weights(py, native)
    opt = E.NativeOptimizer(native, num_iterations=100)
    before = {s.name: py.params.m(s.name).detach().float().cpu().numpy().reshape(-1).copy() for s in py.params.specs}
    g = torch.Generator().manual_seed(9)
    for step in range(3):
        tok = torch.randint(0, 64, (4, cfg.seq_len + 1), generator=g)
        tokens, targets = tok[:, :-1].contiguous(), tok[:, 1:].clone()
        targets[0, :5] = -1
        want = float(tr.train_step([(tokens.cuda(), targets.cuda())]))
        got = native.train_step(tokens.numpy(), targets.numpy(), opt)
        assert abs(got - want) < 1e-3 * max(1.0, abs(want)), (step, got, want)
    assert native.device_status() == 0 and native.launch_count() > 100
    K.check_status()
    # The updates after three optimizer steps. Both optimizers are sign-like at the start (Muon orthogonalises the
    # gradient, AdamW divides it by its own magnitude), so the order-dependent rounding of the fp32 gradient sums
    # (split-K and embedding atomics) moves individual elements visibly: what must agree is the direction and the
    # size of every parameter's update.
    for s in py.params.specs:
        a = native.read(s.name) - before[s.name]
        b = py.params.m(s.name).detach().float().cpu().numpy().reshape(-1) - before[s.name]
        na, nb = float(np.linalg.norm(a)), float(np.linalg.norm(b))
        if nb < 1e-7:
            assert na < 1e-6, s.name
            continue
        cos = float(a @ b) / (na * nb)
        assert cos > 0.9 and abs(na / nb - 1.0) < 0.03, (s.name, cos, na, nb)


def test_separate_forward_and_backward_give_the_fused_step_gradients(cuda_backend):
    cfg = _cfg()
    py = _python_model(cfg, seed=6)
    native = E.NativeModel(cfg, seed=1)
    _copy_weights(py, native)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, 64, (2, cfg.seq_len + 1), generator=g)
    tokens, targets = tok[:, :-1].contiguous().numpy(), tok[:, 1:].contiguous().numpy()
    native.zero_grad()
    loss_a = native.forward_loss(tokens, targets)
    native.backward()
    grads_a = {n: native.read(n, grad=True) for n in ("lm_head.weight", "transformer.h.1.attn.c_q.weight",
                                                      "transformer.h.3.mlp.c_proj.weight", "resid_lambdas",
                                                      "value_embeds.1.weight", "transformer.wte.weight")}
    py.zero_grad()
    loss_b = float(py.forward_backward(torch.from_numpy(tokens).cuda(), torch.from_numpy(targets).cuda()))
    assert abs(loss_a - loss_b) < 1e-3
    for n, ga in grads_a.items():
        gb = py.params.g(n).detach().float().cpu().numpy().reshape(-1)
        rel = float(np.linalg.norm(ga - gb) / (np.linalg.norm(gb) + 1e-12))
        assert rel < 2e-2, (n, rel)


def test_generation_and_scoring_run_on_the_device(cuda_backend):
    from nanochat_cpp_b200.inference import GenerateParams, InferenceEngine, generate_multi
    cfg = _cfg()
    py = _python_model(cfg, seed=7)
    native = E.NativeModel(cfg, seed=1)
    _copy_weights(py, native)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab_size, (1, 40), generator=g)
    want = generate_multi(InferenceEngine(py, use_cuda_graph=False), prompt, GenerateParams(max_tokens=12))[0].tokens
    got = native.generate(prompt[0].tolist(), max_tokens=12)[0][0]
    assert got == want
    tokens = torch.randint(0, cfg.vocab_size, (2, 64), generator=g)
    nll, argmax, _ = native.score(tokens.numpy())[0]
    lg = py.logits(tokens.cuda())
    ref_argmax = lg.argmax(-1)[0].tolist()
    agree = sum(int(a == b) for a, b in zip(argmax[:63], ref_argmax[:63]))
    assert agree >= 60, agree
    assert native.device_status() == 0


def test_native_cli_trains_on_the_device(tmp_path):
    """`nanochat_cli train --device cuda:0`: one native process, no Python in the loop; the loss on a Zipf stream
    must fall and the checkpoint it writes must load back into the CPU engine."""
    import os
    import re
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "nanochat_cpp_b200", "nanochat_cli")
    ckpt = str(tmp_path / "gpu.ckpt")
    out = subprocess.run([exe, "train", "--device", "cuda:0", "--synthetic-zipf", "1.1", "--layers", "4", "--hidden", "512",
                          "--heads", "4", "--kv-heads", "2", "--seq", "256", "--vocab", "1000", "--padded-vocab", "1024",
                          "--batch", "8", "--grad-accum", "2", "--num-iterations", "30", "--log-every", "5",
                          "--checkpoint", ckpt], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-800:]
    losses = [float(m) for m in re.findall(r"^step \d+ \| loss ([\d.]+)", out.stdout, flags=re.M)]
    assert len(losses) == 6 and losses[-1] < losses[0] - 0.25, losses
    assert "on cuda" in out.stdout
    E.select_device("cpu")
    cfg = _cfg()
    host = E.NativeModel(cfg, seed=0)
    host.load(ckpt)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 64, (2, cfg.seq_len + 1), generator=g)
    assert np.isfinite(host.forward_loss(tok[:, :-1].numpy(), tok[:, 1:].numpy()))
