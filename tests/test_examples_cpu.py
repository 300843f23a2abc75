"""The examples run as a user would run them; the operator dispatcher routes tensor lists."""
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(name, *args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "examples", name), *args], capture_output=True, text=True,
                          timeout=600, env=env, cwd="/")


def test_hello_world_example():
    r = _run("hello_world.py")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "greedy continuation" in r.stdout
    losses = [float(l.split()[-1]) for l in r.stdout.splitlines() if l.startswith("step")]
    assert losses[-1] < losses[0]


def test_checkpoint_roundtrip_example(tmp_path):
    r = _run("checkpoint_roundtrip.py", str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    assert "round trip ok" in r.stdout


def test_dispatch_finds_tensors_inside_lists():
    from nanochat_cpp_b200 import ops
    assert ops._first_tensor(([torch.zeros(2)], 1.0), {}) is not None
    assert ops._first_tensor((1.0,), {"grads": (torch.zeros(1),)}) is not None
    assert ops._first_tensor((1.0, "x"), {}) is None
    g = [torch.full((4,), 3.0), torch.full((9,), 4.0)]
    norm, scale = ops.grad_norm_and_clip(g, 1.0)
    assert abs(float(norm) - (36.0 + 144.0) ** 0.5) < 1e-5 and abs(float(scale) * float(norm) - 1.0) < 1e-6
