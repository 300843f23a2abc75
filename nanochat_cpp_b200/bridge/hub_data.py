"""Task datasets hosted on the Hub, and the guarded executor for generated programs.

`DatasetCache.load(repo_id, subset, split)` gives a `HubDataset`: the rows of the dataset's parquet export, read with
pyarrow from a local cache (`<base>/task_data/<owner>--<name>/<subset>/<split>/NNNNN.parquet` + `manifest.json`, the
layout the reference uses in python/nanochat_cpp_bridge/reference_tasks.py, so both share one cache). A missing split is
fetched once: the manifest is written after the last shard, so its presence means the download finished, and a file
lock lets several ranks call `load` at the same time. `HubDataset.shuffle(seed)` orders rows as
`datasets.Dataset.shuffle(seed=seed)` does (a `numpy.random.default_rng(seed)` permutation), which is the order
upstream nanochat evaluates in.

The fetch step is a callable `fetch(repo_id, subset, split) -> iterable of (name, bytes)`; the default asks the Hub's
parquet listing over HTTPS. Tests pass their own.

`run_program(code)` runs a generated Python program in a fresh isolated interpreter (`-I`), in an empty temporary
directory, with a scrubbed environment, resource limits (CPU seconds, address space, file size, open files, no core
dumps) and a wall-clock limit; the child is its own process group and the whole group is ended on time-out. The
result has `.success` like the reference's executor result, so task code reads one shape either way.
"""
from __future__ import annotations

import dataclasses
import json
import os
import signal
import subprocess
import sys
import tempfile
from pathlib import Path
from typing import Callable, Iterable, Optional, Tuple

from .extras import need


def base_dir(environ=None) -> Path:
    env = os.environ if environ is None else environ
    d = Path(env["NANOCHAT_BASE_DIR"]) if env.get("NANOCHAT_BASE_DIR") else Path.home() / ".cache" / "nanochat"
    d.mkdir(parents=True, exist_ok=True)
    return d


class HubDataset:
    """Rows of a pyarrow table as dicts, optionally through a permutation."""

    def __init__(self, table, order=None):
        self.table, self.order = table, order

    def __len__(self) -> int:
        return self.table.num_rows

    def shuffle(self, seed: int) -> "HubDataset":
        np = need("numpy")
        return HubDataset(self.table, np.random.default_rng(seed).permutation(len(self)))

    def __getitem__(self, i: int) -> dict:
        if not -len(self) <= i < len(self):
            raise IndexError(i)
        j = i % len(self)
        j = j if self.order is None else int(self.order[j])
        return {c: self.table[c][j].as_py() for c in self.table.column_names}

    def __iter__(self):
        return (self[i] for i in range(len(self)))


def http_fetch(repo_id: str, subset: str, split: str) -> Iterable[Tuple[str, bytes]]:
    """Default fetch: the Hub's auto-generated parquet export of one split, shard by shard."""
    import urllib.request
    with urllib.request.urlopen(f"https://huggingface.co/api/datasets/{repo_id}/parquet/{subset}/{split}") as r:
        urls = json.loads(r.read())
    for k, url in enumerate(urls):
        with urllib.request.urlopen(url) as r:
            yield f"{k:05d}.parquet", r.read()


class DatasetCache:
    def __init__(self, root: Optional[Path] = None, fetch: Callable[[str, str, str], Iterable] = http_fetch):
        self.root = Path(root) if root else base_dir() / "task_data"
        self.fetch = fetch

    def split_dir(self, repo_id: str, subset: str, split: str) -> Path:
        return self.root / repo_id.replace("/", "--") / subset / split

    def ensure(self, repo_id: str, subset: str = "default", split: str = "train") -> list:
        d = self.split_dir(repo_id, subset, split)
        manifest = d / "manifest.json"
        if not manifest.exists():
            d.mkdir(parents=True, exist_ok=True)
            filelock = need("filelock")
            with filelock.FileLock(str(manifest) + ".lock"):
                if not manifest.exists():           # the rank that got the lock first downloads; the rest skip
                    names = []
                    for name, blob in self.fetch(repo_id, subset, split):
                        tmp = d / (name + ".part")
                        tmp.write_bytes(blob)
                        os.replace(tmp, d / name)
                        names.append(name)
                    if not names:
                        raise RuntimeError(f"{repo_id} {subset}/{split}: the listing is empty")
                    tmp = d / "manifest.json.part"
                    tmp.write_text(json.dumps(names))
                    os.replace(tmp, manifest)
        return [d / n for n in json.loads(manifest.read_text())]

    def load(self, repo_id: str, subset: str = "default", split: str = "train") -> HubDataset:
        pa = need("pyarrow")
        pq = need("pyarrow.parquet")
        return HubDataset(pa.concat_tables([pq.read_table(str(p)) for p in self.ensure(repo_id, subset, split)]))


def hub_loader(cache: Optional[DatasetCache] = None) -> Callable[..., HubDataset]:
    """The loader as one callable `(repo_id, subset="default", split="train") -> HubDataset`, the form the task
    classes and the mixture builders take."""
    c = cache or DatasetCache()
    return c.load


# --------------------------------------------------------------------------------------------- guarded execution
@dataclasses.dataclass
class ProgramResult:
    success: bool
    stdout: str = ""
    stderr: str = ""
    timed_out: bool = False
    returncode: Optional[int] = None
    error: str = ""


def _limits(cpu_seconds: int, memory_bytes: int):
    def apply():
        import resource
        os.setsid()
        for what, value in ((resource.RLIMIT_CPU, cpu_seconds), (resource.RLIMIT_AS, memory_bytes),
                            (resource.RLIMIT_FSIZE, 16 << 20), (resource.RLIMIT_NOFILE, 64),
                            (resource.RLIMIT_CORE, 0)):
            try:
                resource.setrlimit(what, (value, value))
            except (ValueError, OSError):
                pass
    return apply


def run_program(code: str, *, timeout: float = 5.0, memory_bytes: int = 1 << 30, max_output: int = 1 << 16) -> ProgramResult:
    with tempfile.TemporaryDirectory(prefix="nc_exec_") as cwd:
        env = {"PATH": "/usr/bin:/bin", "HOME": cwd, "TMPDIR": cwd, "LANG": "C.UTF-8", "PYTHONHASHSEED": "0",
               "OMP_NUM_THREADS": "1", "TOKENIZERS_PARALLELISM": "false"}
        try:
            p = subprocess.Popen([sys.executable, "-I", "-c", code], cwd=cwd, env=env, stdin=subprocess.DEVNULL,
                                 stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                 preexec_fn=_limits(int(timeout) + 1, memory_bytes))
        except OSError as e:
            return ProgramResult(False, error=str(e))
        try:
            out, err = p.communicate(timeout=timeout)
            timed_out = False
        except subprocess.TimeoutExpired:
            try:
                os.killpg(p.pid, signal.SIGKILL)      # the child called setsid: its pid is its group
            except ProcessLookupError:
                pass
            out, err = p.communicate()
            timed_out = True
        return ProgramResult(success=(not timed_out and p.returncode == 0),
                             stdout=out.decode(errors="replace")[:max_output],
                             stderr=err.decode(errors="replace")[:max_output], timed_out=timed_out,
                             returncode=p.returncode)


def code_executor(**limits) -> Callable[[str], ProgramResult]:
    return lambda code: run_program(code, **limits)
