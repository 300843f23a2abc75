"""ThreadSanitizer over the host runtime's threaded parts (transports + ring, mesh replicas, loader prefetch)."""
import glob
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "nanochat_cpp_b200", "csrc", "host")


def test_host_runtime_is_race_free_under_tsan(tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    sources = [s for s in glob.glob(os.path.join(HOST, "*.cc")) if not os.path.basename(s).startswith("capi")]
    exe = str(tmp_path / "tsan_host")
    cmd = ["g++", "-std=c++20", "-O1", "-g", "-fsanitize=thread", "-fno-omit-frame-pointer", "-pthread",
           "-Wno-unknown-pragmas", "-I", HOST, "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "native", "tsan_host.cc"), *sources, "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if r.returncode != 0 and "tsan" in (r.stderr or "").lower() and "cannot find" in r.stderr:
        pytest.skip("libtsan is not installed")
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    assert "ThreadSanitizer" not in r.stderr, r.stderr[-4000:]
    assert r.returncode == 0, (r.stdout, r.stderr[-2000:])
    assert "tsan driver: ok" in r.stdout
