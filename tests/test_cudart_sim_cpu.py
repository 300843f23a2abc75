"""The stand-in CUDA runtime (csrc/sim/cudart_sim.cc): on this machine, without a GPU, the native CLI's `--device cuda:0`
path runs the C++ GPU engine against it; every launch, tensor map, copy and allocation is checked against the B200's
limits and written to a trace. A second program makes the mistakes on purpose (through the runtime API, on the host)
and the runtime names each one."""
import json
import os
import subprocess
import textwrap

import pytest

import nanochat_cpp_b200

PKG = os.path.dirname(nanochat_cpp_b200.__file__)
SIM = os.path.join(PKG, "libcudart_sim.so")
CLI = os.path.join(PKG, "nanochat_cli")
GPU = os.path.join(PKG, "libnanochat_gpu.so")


def _trace(path):
    return [json.loads(line) for line in open(path)]


@pytest.mark.skipif(not (os.path.exists(SIM) and os.path.exists(CLI) and os.path.exists(GPU)),
                    reason="native libraries not built")
def test_gpu_engine_host_side_runs_clean_under_the_simulated_runtime(tmp_path):
    trace = str(tmp_path / "trace.jsonl")
    env = dict(os.environ, LD_PRELOAD=SIM, NANOCHAT_SIM_TRACE=trace, NANOCHAT_SIM_STRICT="1")
    cmd = [CLI, "train", "--device", "cuda:0", "--synthetic-zipf", "--layers", "4", "--hidden", "256", "--heads", "2",
           "--kv-heads", "1", "--vocab", "1024", "--seq", "256", "--batch", "2", "--num-iterations", "2"]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert p.returncode == 0, p.stderr[-2000:]
    assert "2 steps on cuda" in p.stdout
    rows = _trace(trace)
    summary = rows[-1]
    assert summary["call"] == "summary" and summary["violations"] == 0
    assert not [r for r in rows if r["call"] == "violation"]
    launches = [r for r in rows if r["call"] == "launch"]
    assert len(launches) == summary["launches"] > 300
    # the engine's own launch counter and the runtime agree
    assert f"kernel launches {summary['launches']}" in p.stdout
    per = summary["per_kernel"]
    for needle in ("gemm_pair_kernel", "attention_fwd2_kernel", "attention_bwd_kernel", "classifier_smem_kernel",
                   "adamw_kernel", "muon_", "rmsnorm_kernel", "embedding_fwd_kernel"):
        assert any(needle in k for k in per), needle
    # CTA pairs are launched as clusters of two, with the grid a multiple of the cluster
    pairs = [r for r in launches if "gemm_pair_kernel" in r["kernel"]]
    assert pairs and all(r["cluster"] == [2, 1, 1] and r["grid"][0] % 2 == 0 for r in pairs)
    assert all(r["smem"] <= 232448 for r in launches)
    maps = [r for r in rows if r["call"] == "tensor_map"]
    assert maps and all(m["box"][0] * m["elem_bytes"] % 16 == 0 for m in maps)
    assert summary["live_streams"] == 0 and summary["live_events"] == 0


@pytest.mark.skipif(not (os.path.exists(SIM) and os.path.exists(CLI) and os.path.exists(GPU)),
                    reason="native libraries not built")
def test_checkpoint_and_paged_generation_run_clean_under_the_simulated_runtime(tmp_path):
    """The inference side of the C++ GPU engine: a checkpoint written by a (simulated) training step is loaded and six
    tokens are decoded over the paged cache: prefill through the flash kernel, decode through the skinny GEMMs, the
    fused prologue and the paged attention kernel. Every launch and tensor map passes the runtime's checks."""
    model = ["--layers", "4", "--hidden", "256", "--heads", "2", "--kv-heads", "1", "--vocab", "1024", "--seq", "256"]
    ck = str(tmp_path / "m.ckpt")
    env = dict(os.environ, LD_PRELOAD=SIM, NANOCHAT_SIM_STRICT="1", NANOCHAT_SIM_TRACE=str(tmp_path / "t1.jsonl"))
    p = subprocess.run([CLI, "train", "--device", "cuda:0", "--synthetic-zipf", *model, "--batch", "2",
                        "--num-iterations", "1", "--checkpoint", ck], env=env, capture_output=True, text=True,
                       timeout=300, cwd=str(tmp_path))
    assert p.returncode == 0 and os.path.getsize(ck) > 1 << 20, p.stderr[-1500:]
    trace = str(tmp_path / "t2.jsonl")
    env["NANOCHAT_SIM_TRACE"] = trace
    p = subprocess.run([CLI, "generate", "--device", "cuda:0", "--model", ck, *model, "--tokens", "1,2,3,4,5",
                        "--max-tokens", "6"], env=env, capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert p.returncode == 0, p.stderr[-1500:]
    assert p.stdout.strip().startswith("1,2,3,4,5,") and len(p.stdout.strip().split(",")) == 11
    rows = _trace(trace)
    summary = rows[-1]
    assert summary["violations"] == 0
    per = summary["per_kernel"]
    for needle in ("paged_decode_kernel", "decode_prep_append_kernel", "gemm_skinny_kernel", "attention_fwd2_kernel",
                   "softcap_logits_kernel"):
        assert any(needle in k for k in per), needle


BAD_PROGRAM = textwrap.dedent("""
    #include <cuda.h>
    #include <cuda_runtime_api.h>
    #include <cstdio>
    typedef CUresult (*Encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static void not_a_kernel() {}
    int main() {
      char* d = nullptr;
      char host[256] = {0};
      cudaStream_t s;
      cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
      cudaMalloc(reinterpret_cast<void**>(&d), 4096);
      cudaMemcpyAsync(d + 4000, host, 256, cudaMemcpyHostToDevice, s);          // 160 bytes past the end
      cudaMemsetAsync(d, 0, 8192, s);                                          // twice the allocation
      cudaLaunchKernel(reinterpret_cast<const void*>(&not_a_kernel), dim3(1), dim3(2048), nullptr, 0, s);
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      CUtensorMap map;
      cuuint64_t dims[2] = {100, 8}, strides[1] = {200};                       // 200-byte rows: not a multiple of 16
      cuuint32_t box[2] = {72, 8}, es[2] = {1, 1};                             // 144-byte inner box under 128B swizzle
      reinterpret_cast<Encode>(fn)(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d + 2, dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      cudaFree(host);                                                          // not an allocation
      cudaStreamDestroy(s);
      cudaStreamSynchronize(s);                                                // destroyed
      std::puts("done");
      return 0;                                                                // d is never freed
    }
""")


@pytest.mark.skipif(not os.path.exists(SIM), reason="simulated runtime not built")
def test_the_runtime_names_each_mistake(tmp_path):
    src, exe, trace = tmp_path / "bad.cc", tmp_path / "bad", str(tmp_path / "trace.jsonl")
    src.write_text(BAD_PROGRAM)
    cuda_inc = "/usr/local/cuda/include"
    subprocess.run(["g++", "-std=c++17", "-I", cuda_inc, str(src), "-o", str(exe), "-L", PKG, "-lcudart_sim",
                    f"-Wl,-rpath,{PKG}"], check=True, capture_output=True)
    p = subprocess.run([str(exe)], env=dict(os.environ, NANOCHAT_SIM_TRACE=trace), capture_output=True, text=True,
                       timeout=60)
    assert p.returncode == 0 and "done" in p.stdout
    rows = _trace(trace)
    said = " | ".join(r["what"] for r in rows if r["call"] == "violation")
    for needle in ("destination of 256 bytes leaves its allocation", "range of 8192 bytes leaves its allocation",
                   "no module registered", "outside (1024, 1024, 64)", "base address not 16-byte aligned",
                   "200 bytes is not a multiple of 16", "exceeds the 128-byte swizzle span",
                   "pointer is not a live allocation", "stream is not live"):
        assert needle in said, (needle, said)
    summary = rows[-1]
    assert summary["violations"] >= 9 and summary["live_allocations"] == 1 and summary["live_bytes"] == 4096
