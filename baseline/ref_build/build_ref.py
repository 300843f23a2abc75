"""Hand build of the unmodified reference (ming6ao/nanochat.cpp) for the benchmark's reference arm.

The reference is a Bazel project; Bazel is not installed and has no registry access here, so this script
compiles the reference's own sources, untouched and in place, with the compilers of the image:

  * host sources  `src/*.cc`, `src/tokenizer/*.cc` (tests and `*_main.cc` left out)   g++ -std=c++20 -O2 -fopenmp
  * CUDA backend  `backends/cuda/{device,gemm,row_reduce,span_reduce}.cu`, `backends/cuda/kernels/*.cu`,
                  `backends/cuda/gemm/{gemm_bf16.cu,dispatch.cc,...}`, `backends/cuda/collective/*`
                  nvcc -arch=sm_100 -O2 -DNANOCHAT_PRECISION=1 (bf16 compute, fp32 master weights and gradients)
  * left out      `attention_hopper.cu` (sm_90a only: its own stand-in `attention_hopper_absent.cc` is linked,
                  as the reference's build does for every architecture but sm_90a), the CUTLASS Sm90 GEMM objects
                  (need the pinned CUTLASS checkout and sm_90a; `stubs.cc` supplies their launchers returning
                  false, which is what they return on a device that is not compute capability 9.0), and the parquet
                  reader (needs zstd.h; `stubs.cc` supplies `OpenParquetSource` returning "unavailable": the
                  harness feeds documents through `TrainConfig::train_source`).

Output (all under `baseline/_ref/`, which is not tracked; `--backend cpu` builds the reference's CPU backend in
fp32 into `baseline/_ref/cpu/` the same way): `libnanochat_ref.so`, the harness `ref_train`,
`backends/{cpu,cuda}/caps.json` (a copy of the reference's declaration files plus a `b200` device row cloned from
its `h100` row, the reference's own bring-up procedure for a new card), `build.log`.

    python baseline/ref_build/build_ref.py [--ref <reference checkout>] [--jobs 8] [--backend cuda|cpu]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import json
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "baseline", "_ref")


def _skip_host(path: str) -> bool:
    base = os.path.basename(path)
    return (base.endswith("_test.cc") or base.endswith("_main.cc") or base.endswith("_benchmark.cc")
            or base in ("nanochat_cli.cc",))


def sources(ref: str, backend: str):
    host = [p for p in sorted(glob.glob(f"{ref}/src/*.cc") + glob.glob(f"{ref}/src/tokenizer/*.cc"))
            if not _skip_host(p)]
    cuda = []
    if backend == "cuda":
        # the CUDA backend defines CreateGradientSync itself (collective/native_sync.cu)
        host = [p for p in host if os.path.basename(p) != "distributed.cc"]
        host += [f"{ref}/backends/cuda/caps_names.cc", f"{ref}/backends/cuda/fused_overrides.cc",
                 f"{ref}/backends/cuda/gemm/dispatch.cc", f"{ref}/backends/cuda/gemm/cutlass_candidates.cc",
                 f"{ref}/backends/cuda/kernels/attention_hopper_absent.cc"]
        host += [p for p in sorted(glob.glob(f"{ref}/backends/cuda/collective/*.cc")) if not _skip_host(p)]
        cuda = [f"{ref}/backends/cuda/{n}.cu" for n in ("device", "gemm", "row_reduce", "span_reduce")]
        cuda += [f"{ref}/backends/cuda/gemm/gemm_bf16.cu"]
        cuda += [p for p in sorted(glob.glob(f"{ref}/backends/cuda/kernels/*.cu"))
                 if not os.path.basename(p).startswith("attention_hopper")]
        cuda += [f"{ref}/backends/cuda/collective/native_sync.cu"]
    else:
        host += [f"{ref}/backends/cpu/kernels.cc"] + \
                [p for p in glob.glob(f"{ref}/backends/cpu/caps_names.cc")]
    return host, cuda


def obj_name(ref: str, src: str) -> str:
    rel = os.path.relpath(src, ref) if src.startswith(ref) else os.path.relpath(src, ROOT)
    return rel.replace("/", "__") + ".o"


def run(cmd, log):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append("$ " + " ".join(cmd) + "\n" + p.stdout)
    return p.returncode, p.stdout


def write_caps(ref: str):
    """Copies the two capability declarations and adds a `b200` row cloned from `h100` (with the rates this
    pool's B200 measured), so that the reference does not fall back to its slow composition tier for lack of a row."""
    for backend in ("cpu", "cuda"):
        src = f"{ref}/backends/{backend}/caps.json"
        dst_dir = os.path.join(OUT, "backends", backend)
        os.makedirs(dst_dir, exist_ok=True)
        if not os.path.exists(src):
            continue
        doc = json.load(open(src))
        if backend == "cuda":
            devs = doc.get("devices", [])
            h100 = next((d for d in devs if str(d.get("name", "")).lower().replace(" ", "") in ("h100",)), None)
            if h100 is not None and not any("b200" in str(d.get("name", "")).lower() for d in devs):
                row = json.loads(json.dumps(h100))
                row["name"] = "b200"
                devs.append(row)
        json.dump(doc, open(os.path.join(dst_dir, "caps.json"), "w"), indent=2)


def build(ref: str, jobs: int, backend: str, verbose: bool = True) -> int:
    global OUT
    if backend == "cpu":
        OUT = os.path.join(ROOT, "baseline", "_ref", "cpu")
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    precision = "1" if backend == "cuda" else "0"
    host, cuda = sources(ref, backend)
    extra = [os.path.join(HERE, "stubs.cc")]
    inc = [f"-I{ref}", f"-I{ref}/include"]
    cxx = ["g++", "-std=c++20", "-O2", "-fPIC", "-fopenmp", f"-DNANOCHAT_PRECISION={precision}", "-w"] + inc
    if backend == "cuda":
        cxx += ["-DNANOCHAT_REF_CUDA=1", "-I/usr/local/cuda/include"]
    nvcc = ["nvcc", "-arch=sm_100", "-std=c++20", "-O2", "-Xcompiler", "-O2,-fPIC,-fopenmp,-w",
            f"-DNANOCHAT_PRECISION={precision}", "-diag-suppress", "20012", "-Xcudafe", "--diag_suppress=177"] + inc
    log: list[str] = []
    tasks = []
    for s in host + extra:
        tasks.append((s, cxx + ["-c", s, "-o", os.path.join(OUT, "obj", obj_name(ref, s))]))
    for s in cuda:
        tasks.append((s, nvcc + ["-c", s, "-o", os.path.join(OUT, "obj", obj_name(ref, s))]))
    t0 = time.time()
    failed = []
    with cf.ThreadPoolExecutor(jobs) as ex:
        futs = {ex.submit(run, cmd, log): src for src, cmd in tasks}
        for f in cf.as_completed(futs):
            rc, out = f.result()
            if rc != 0:
                failed.append(futs[f])
                if verbose:
                    print(f"FAILED {futs[f]}\n{out[-3000:]}")
    objs = [os.path.join(OUT, "obj", obj_name(ref, s)) for s in host + extra + cuda]
    rc = 1
    if not failed:
        lib = os.path.join(OUT, "libnanochat_ref.so")
        link = ["g++", "-shared", "-o", lib] + objs + ["-fopenmp", "-lpthread"]
        if backend == "cuda":
            link += ["-L/usr/local/cuda/lib64", "-lcudart", "-lcublas", "-lcublasLt", "-Wl,-rpath,/usr/local/cuda/lib64"]
        rc, out = run(link, log)
        if rc != 0 and verbose:
            print(out[-6000:])
        if rc == 0:
            exe = os.path.join(OUT, "ref_train")
            cmd = cxx + [os.path.join(HERE, "harness.cc"), "-o", exe, f"-L{OUT}", "-lnanochat_ref",
                         "-Wl,-rpath,$ORIGIN", "-fopenmp", "-lpthread"]
            if backend == "cuda":
                cmd += ["-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"]
            rc, out = run(cmd, log)
            if rc != 0 and verbose:
                print(out[-6000:])
    write_caps(ref)
    open(os.path.join(OUT, "build.log"), "w").write("\n".join(log))
    json.dump({"backend": backend, "ref": ref, "ok": rc == 0 and not failed, "failed": failed,
               "host_sources": len(host), "cuda_sources": len(cuda), "seconds": round(time.time() - t0, 1)},
              open(os.path.join(OUT, "build.json"), "w"), indent=1)
    if verbose:
        print(f"reference build ({backend}): {'ok' if rc == 0 and not failed else 'FAILED'} in {time.time() - t0:.0f}s, "
              f"{len(host)} host + {len(cuda)} cuda sources -> {OUT}")
    return 0 if (rc == 0 and not failed) else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("NANOCHAT_REF_SRC", "/root/reference"))
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--backend", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--clean", action="store_true")
    a = ap.parse_args()
    if a.clean and os.path.isdir(OUT):
        shutil.rmtree(OUT)
    if not os.path.isdir(a.ref):
        print(f"reference sources not found at {a.ref}")
        return 2
    return build(a.ref, a.jobs, a.backend)


if __name__ == "__main__":
    sys.exit(main())
