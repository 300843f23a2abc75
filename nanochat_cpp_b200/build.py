"""In-tree build of the native code.

Two artefacts, both placed next to this file so that they travel with the source tree:

* `_C.so`        - the PyTorch extension: every CUDA kernel of `csrc/cuda` (compiled by nvcc
                   for sm_100a only) plus `csrc/cuda/bindings.cpp`.
* `libnanochat_core.so` - the host runtime of `csrc/host` (formats, tokenizer, BPE trainer, data
                   loader, parquet reader, C ABI); plain C++20, no CUDA, no torch.
* `libnanochat_gpu.so` - the same kernels plus the C++ GPU engine of `csrc/gpu` (no torch): what the C ABI and
                   the native CLI run on when a CUDA device is selected.

`python -m nanochat_cpp_b200.build` builds what is stale. Objects are cached under `_build/`
keyed by a hash of the source, the headers beside it and the flags.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC_CUDA = os.path.join(HERE, "csrc", "cuda")
CSRC_HOST = os.path.join(HERE, "csrc", "host")
BUILD_DIR = os.path.join(HERE, "_build")
EXT_PATH = os.path.join(HERE, "_C.so")
CORE_PATH = os.path.join(HERE, "libnanochat_core.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-fPIC", "-std=c++17", "-Wall", "-Wno-unused-function"]
HOST_FLAGS = ["-O3", "-fPIC", "-std=c++20", "-Wall", "-Wextra", "-pthread", "-fopenmp"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _hash(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd: List[str], log: str) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{r.stdout[-6000:]}")


def _compile_many(jobs) -> List[str]:
    objs = []
    todo = []
    for src, obj, cmd in jobs:
        objs.append(obj)
        if not os.path.exists(obj):
            todo.append((src, obj, cmd))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            futs = [ex.submit(_run, cmd, obj + ".log") for _, obj, cmd in todo]
            for f in futs:
                f.result()
    return objs


def _prune(keep: List[str], prefix: str) -> None:
    """Drop cached objects (and their logs) of sources that have since changed."""
    keep_set = set(keep)
    for path in glob.glob(os.path.join(BUILD_DIR, "*.o")):
        base = os.path.basename(path)
        is_host = base.startswith("host_")
        if base.startswith("gpu_") or (prefix == "host_") != is_host:
            continue
        if path not in keep_set:
            for victim in (path, path + ".log"):
                try:
                    os.remove(victim)
                except OSError:
                    pass


def build_extension(verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the PyTorch extension."""
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(BUILD_DIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC_CUDA, "*.h")) + glob.glob(os.path.join(CSRC_CUDA, "*.cuh"))
    cu_sources = sorted(glob.glob(os.path.join(CSRC_CUDA, "*.cu")))
    cpp_sources = sorted(glob.glob(os.path.join(CSRC_CUDA, "*.cpp")))
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    jobs = []
    for src in cu_sources:
        tag = _hash([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, [nvcc] + NVCC_FLAGS + ["-I", CSRC_CUDA, "-c", src, "-o", obj]))
    inc = []
    for p in ce.include_paths("cuda") if hasattr(ce, "include_paths") else []:
        inc += ["-I", p]
    inc += ["-I", os.path.join(cuda_home, "include"), "-I", sysconfig.get_paths()["include"], "-I", CSRC_CUDA]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI) if hasattr(torch._C, "_GLIBCXX_USE_CXX11_ABI") else 1
    defs = ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    for part in ("rowops", "attention", "optim", "comm", "decode", "fp8"):
        if os.path.exists(os.path.join(CSRC_CUDA, part + "_bind.cpp")):
            defs.append("-DNC_HAVE_" + part.upper())
    for src in cpp_sources:
        tag = _hash([src] + headers, " ".join(CXX_FLAGS) + torch.__version__)
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, ["g++"] + CXX_FLAGS + defs + inc + ["-c", src, "-o", obj]))
    objs = _compile_many(jobs)
    _prune(objs, prefix="")
    stamp = os.path.join(BUILD_DIR, "ext.stamp")
    key = _hash(objs, "link")
    if os.path.exists(EXT_PATH) and os.path.exists(stamp) and open(stamp).read() == key:
        return EXT_PATH
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-shared", "-o", EXT_PATH] + objs + [
        "-L", torch_lib, "-L", os.path.join(cuda_home, "lib64"), "-lc10", "-lc10_cuda", "-ltorch_cpu",
        "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart", f"-Wl,-rpath,{torch_lib}",
        f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}"]
    _run(cmd, os.path.join(BUILD_DIR, "link_ext.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", EXT_PATH)
    return EXT_PATH


CLI_PATH = os.path.join(HERE, "nanochat_cli")
GPU_PATH = os.path.join(HERE, "libnanochat_gpu.so")
CSRC_GPU = os.path.join(HERE, "csrc", "gpu")


def build_gpu_engine(verbose: bool = False) -> str:
    """`libnanochat_gpu.so`: the sm_100a kernels of csrc/cuda (the same objects the extension links, without any of
    its PyTorch bindings) and the C++ engine of csrc/gpu that drives them; no torch, no Python. The core library
    opens it when a CUDA device is selected through the C ABI."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    if not os.path.isdir(CSRC_GPU) or not os.path.exists(CORE_PATH):
        return ""
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    headers = (glob.glob(os.path.join(CSRC_CUDA, "*.h")) + glob.glob(os.path.join(CSRC_CUDA, "*.cuh")) +
               glob.glob(os.path.join(CSRC_HOST, "*.h")) + glob.glob(os.path.join(CSRC_GPU, "*.h")))
    jobs = []
    for src in sorted(glob.glob(os.path.join(CSRC_CUDA, "*.cu"))):      # cache shared with the extension
        tag = _hash([src] + glob.glob(os.path.join(CSRC_CUDA, "*.h")) + glob.glob(os.path.join(CSRC_CUDA, "*.cuh")),
                    " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, [nvcc] + NVCC_FLAGS + ["-I", CSRC_CUDA, "-c", src, "-o", obj]))
    for src in sorted(glob.glob(os.path.join(CSRC_GPU, "*.cu"))):
        tag = _hash([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD_DIR, "gpu_" + os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, [nvcc] + NVCC_FLAGS + ["-I", CSRC_GPU, "-c", src, "-o", obj]))
    for src in sorted(glob.glob(os.path.join(CSRC_GPU, "*.cc"))):
        tag = _hash([src] + headers, " ".join(HOST_FLAGS))
        obj = os.path.join(BUILD_DIR, "gpu_" + os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, ["g++"] + HOST_FLAGS + ["-I", os.path.join(cuda_home, "include"), "-I", CSRC_GPU, "-I",
                                                       CSRC_HOST, "-c", src, "-o", obj]))
    objs = _compile_many(jobs)
    stamp = os.path.join(BUILD_DIR, "gpu.stamp")
    key = _hash(objs + [CORE_PATH], "link-gpu")
    if os.path.exists(GPU_PATH) and os.path.exists(stamp) and open(stamp).read() == key:
        return GPU_PATH
    _run(["g++", "-shared", "-pthread", "-fopenmp", "-o", GPU_PATH] + objs +
         ["-L", HERE, "-lnanochat_core", "-L", os.path.join(cuda_home, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN",
          f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}"], os.path.join(BUILD_DIR, "link_gpu.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", GPU_PATH)
    return GPU_PATH


def build_sim(verbose: bool = False) -> str:
    """`libcudart_sim.so`: the stand-in CUDA runtime of csrc/sim (host code only; needs the CUDA headers, no GPU).
    Preloaded under the native CLI it lets the C++ GPU engine's host side run, checked, on a machine without a GPU."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    src = os.path.join(os.path.dirname(CSRC_HOST), "sim", "cudart_sim.cc")
    if not os.path.exists(src):
        return ""
    out = os.path.join(HERE, "libcudart_sim.so")
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    key = _hash([src], "sim")
    stamp = os.path.join(BUILD_DIR, "sim.stamp")
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == key:
        return out
    _run(["g++", "-shared", "-fPIC", "-O2", "-std=c++17", "-Wall", "-I", os.path.join(cuda_home, "include"), src, "-o",
          out], os.path.join(BUILD_DIR, "sim.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", out)
    return out


def build_emu(verbose: bool = False) -> str:
    """`libnc_emu.so`: the CUDA-core kernels of csrc/cuda compiled by the host compiler over csrc/emu/cuda_emu.h
    (every CUDA thread a fiber). Needs the CUDA headers, no GPU and no nvcc."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    emu_dir = os.path.join(os.path.dirname(CSRC_HOST), "emu")
    srcs = [os.path.join(emu_dir, f) for f in ("emu_kernels.cc", "emu_optim.cc", "emu_decode.cc", "emu_comm.cc", "emu_runtime.cc")]
    if not all(os.path.exists(f) for f in srcs):
        return ""
    out = os.path.join(HERE, "libnc_emu.so")
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    deps = srcs + [os.path.join(emu_dir, "cuda_emu.h")] + glob.glob(os.path.join(CSRC_CUDA, "*.cuh")) + \
        glob.glob(os.path.join(CSRC_CUDA, "*.h")) + \
        [os.path.join(CSRC_CUDA, f) for f in ("rowops.cu", "optim.cu", "decode.cu", "comm.cu")]
    key = _hash(deps, "emu-nsa")
    stamp = os.path.join(BUILD_DIR, "emu.stamp")
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == key:
        return out
    # -fno-strict-aliasing: device code reads a register vector through a pointer of its element type as a matter of
    # course; nvcc gives that the obvious meaning, a host compiler only with this flag
    _run(["g++", "-O2", "-g", "-std=c++20", "-fPIC", "-shared", "-fno-strict-aliasing", "-I",
          os.path.join(cuda_home, "include"), "-I", CSRC_CUDA]
         + srcs + ["-o", out], os.path.join(BUILD_DIR, "emu.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", out)
    return out


def build_core(verbose: bool = False) -> str:
    """Compile the host runtime (no CUDA, no torch)."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC_HOST, "*.cc")))
    if not sources:
        return ""
    headers = glob.glob(os.path.join(CSRC_HOST, "*.h")) + glob.glob(
        os.path.join(os.path.dirname(HERE), "include", "nanochat", "*.h"))
    inc = ["-I", CSRC_HOST, "-I", os.path.join(os.path.dirname(HERE), "include")]
    jobs = []
    for src in sources:
        tag = _hash([src] + headers, " ".join(HOST_FLAGS))
        obj = os.path.join(BUILD_DIR, "host_" + os.path.basename(src) + "." + tag + ".o")
        jobs.append((src, obj, ["g++"] + HOST_FLAGS + inc + ["-c", src, "-o", obj]))
    objs = _compile_many(jobs)
    _prune(objs, prefix="host_")
    stamp = os.path.join(BUILD_DIR, "core.stamp")
    key = _hash(objs, "link-core")
    if os.path.exists(CORE_PATH) and os.path.exists(stamp) and open(stamp).read() == key:
        return CORE_PATH
    _run(["g++", "-shared", "-pthread", "-fopenmp", "-o", CORE_PATH] + objs, os.path.join(BUILD_DIR, "link_core.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", CORE_PATH)
    build_cli(verbose)
    return CORE_PATH


def build_cli(verbose: bool = False) -> str:
    """The native command line (links only the host runtime; finds it beside itself through $ORIGIN)."""
    src = os.path.join(CSRC_HOST, "cli", "nanochat_cli.cc")
    if not os.path.exists(src) or not os.path.exists(CORE_PATH):
        return ""
    stamp = os.path.join(BUILD_DIR, "cli.stamp")
    key = _hash([src, CORE_PATH, os.path.join(os.path.dirname(HERE), "include", "nanochat", "capi.h")], "cli")
    if os.path.exists(CLI_PATH) and os.path.exists(stamp) and open(stamp).read() == key:
        return CLI_PATH
    _run(["g++", "-std=c++20", "-O2", "-I", os.path.join(os.path.dirname(HERE), "include"), src, "-o", CLI_PATH,
          "-L", HERE, "-lnanochat_core", "-Wl,-rpath,$ORIGIN", "-pthread", "-fopenmp"],
         os.path.join(BUILD_DIR, "link_cli.log"))
    with open(stamp, "w") as f:
        f.write(key)
    if verbose:
        print("built", CLI_PATH)
    return CLI_PATH


def build_all(verbose: bool = False) -> None:
    build_core(verbose)
    build_cli(verbose)
    build_extension(verbose)
    build_gpu_engine(verbose)
    build_sim(verbose)
    build_emu(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
    sys.exit(0)
