"""Checkpoint stages on the Hugging Face Hub.

A *stage* is one point of the recipe (base, sft, rl) published as a folder `<stage>/` of a model repository:

    checkpoint.ckpt     the NCHKPT01 container
    model.json          the model configuration
    tokenizer.nctoken   the NCTOKEN1 artefact the stage was trained with
    train.json          the training configuration
    run.json            provenance: stage, run, source revision, build, parent stage, step, time
    metrics.jsonl, summary.json, README.md   (optional extras and the card)

Tokenizers shared by several runs live in a repository of their own as `vocab-<N>.nctoken`; pretraining shards come
from a dataset repository. File names, the record's keys and the repository naming (`<namespace>/nanochat-<run>`)
follow the reference (python/nanochat_cpp_bridge/hf_hub.py) so that a stage written by either loads in the other.

Nothing here imports `huggingface_hub` at module level. `HubClient` takes the two objects that talk to the network,
an `HfApi`-like `api` (create_repo / upload_folder / upload_file / create_tag / whoami) and a
`snapshot_download`-like `download`; without them it builds the real ones on first use. Tests hand in fakes.
"""
from __future__ import annotations

import dataclasses
import datetime
import json
import os
import shutil
from pathlib import Path
from typing import Any, Callable, Iterable, Optional, Sequence

from .extras import need

CONTAINER_MAGIC = b"NCHKPT01"
TOKENIZER_MAGIC = b"NCTOKEN1"
REPO_PREFIX = "nanochat"
LOAD_FILES = ("checkpoint.ckpt", "model.json", "tokenizer.nctoken")
ALL_FILES = LOAD_FILES + ("train.json", "run.json", "metrics.jsonl", "summary.json", "README.md")
PRETRAIN_DATASET = "karpathy/climbmix-400b-shuffle"
PRETRAIN_SHARDS = ("shard_00000.parquet", "shard_06542.parquet")      # the training and the validation shard


def tokenizer_file(vocab_size: int) -> str:
    return f"vocab-{int(vocab_size)}.nctoken"


def now_utc() -> str:
    return datetime.datetime.now(datetime.timezone.utc).isoformat()


@dataclasses.dataclass
class RunRecord:
    """Provenance of one stage (`run.json`)."""
    stage: str
    run_name: str
    git_revision: str = ""
    build_key: str = ""
    cuda_arch: str = "sm_100a"
    container: str = CONTAINER_MAGIC.decode()
    parent_repo_id: str = ""
    parent_revision: str = ""
    step: int = 0
    created_utc: str = ""

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1, sort_keys=True) + "\n"

    @classmethod
    def from_json(cls, text: str) -> "RunRecord":
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in json.loads(text).items() if k in known})

    def card(self, description: str = "") -> str:
        out = [f"# {self.run_name}", ""]
        if description:
            out += [description, ""]
        out += [f"- stage: `{self.stage}`", f"- container: `{self.container}`",
                f"- source revision: `{self.git_revision}`", f"- step: {self.step}"]
        if self.parent_repo_id:
            out.append(f"- parent: `{self.parent_repo_id}` at `{self.parent_revision}`")
        return "\n".join(out) + "\n"


def _check_magic(path: Path, magic: bytes, what: str) -> None:
    with open(path, "rb") as f:
        head = f.read(len(magic))
    if head != magic:
        raise ValueError(f"{path}: not {what} (starts with {head!r})")


def _as_json_text(obj) -> str:
    if isinstance(obj, str):
        return obj if obj.endswith("\n") else obj + "\n"
    if hasattr(obj, "to_dict"):
        obj = obj.to_dict()
    elif dataclasses.is_dataclass(obj):
        obj = dataclasses.asdict(obj)
    return json.dumps(obj, indent=1, sort_keys=True) + "\n"


def write_stage(folder, record: RunRecord, *, model_json, train_json, tokenizer, checkpoint=None,
                description: str = "", extras: Iterable = ()) -> Path:
    """Lay out one stage folder. `model_json` / `train_json`: text, a dict, a dataclass or an object with `to_dict`.
    `tokenizer` and `checkpoint` are paths of artefacts (copied; their magic is checked); `extras` are more files to
    copy under their own names (metrics.jsonl, summary.json)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "model.json").write_text(_as_json_text(model_json), encoding="utf-8")
    (folder / "train.json").write_text(_as_json_text(train_json), encoding="utf-8")
    _check_magic(Path(tokenizer), TOKENIZER_MAGIC, "an NCTOKEN1 tokenizer")
    shutil.copyfile(tokenizer, folder / "tokenizer.nctoken")
    if checkpoint is not None:
        _check_magic(Path(checkpoint), CONTAINER_MAGIC, "an NCHKPT01 container")
        if Path(checkpoint).resolve() != (folder / "checkpoint.ckpt").resolve():
            shutil.copyfile(checkpoint, folder / "checkpoint.ckpt")
    for path in extras:
        shutil.copyfile(path, folder / Path(path).name)
    if not record.created_utc:
        record.created_utc = now_utc()
    (folder / "run.json").write_text(record.to_json(), encoding="utf-8")
    (folder / "README.md").write_text(record.card(description), encoding="utf-8")
    return folder


def read_stage(folder) -> dict:
    """What a loader needs from a stage folder: paths of the container and tokenizer, the parsed model config, the
    record if present. Raises if a required file is missing or has the wrong magic."""
    folder = Path(folder)
    for name in LOAD_FILES:
        if not (folder / name).is_file():
            raise FileNotFoundError(f"stage folder {folder} has no {name}")
    _check_magic(folder / "checkpoint.ckpt", CONTAINER_MAGIC, "an NCHKPT01 container")
    _check_magic(folder / "tokenizer.nctoken", TOKENIZER_MAGIC, "an NCTOKEN1 tokenizer")
    rec = folder / "run.json"
    return {"checkpoint": folder / "checkpoint.ckpt", "tokenizer": folder / "tokenizer.nctoken",
            "model": json.loads((folder / "model.json").read_text(encoding="utf-8")),
            "record": RunRecord.from_json(rec.read_text(encoding="utf-8")) if rec.is_file() else None}


def load_stage(folder, device: str = "cpu", dtype=None):
    """(model, tokenizer, record) of a stage folder through this package's own loaders."""
    from ..data.native import Tokenizer
    from ..train.checkpointer import load_checkpoint
    info = read_stage(folder)
    kw = {} if dtype is None else {"dtype": dtype}
    model, _ = load_checkpoint(str(info["checkpoint"]), device=device, **kw)
    return model, Tokenizer.load(str(info["tokenizer"])), info["record"]


class HubClient:
    """The network side. `api` and `download` default to `huggingface_hub.HfApi(token)` and
    `huggingface_hub.snapshot_download`, built on first use."""

    def __init__(self, api: Any = None, download: Optional[Callable[..., Any]] = None, token: Optional[str] = None,
                 environ=None):
        self._api, self._download, self.token = api, download, token
        self.environ = os.environ if environ is None else environ

    @property
    def api(self):
        if self._api is None:
            self._api = need("huggingface_hub", "publishing to the Hub").HfApi(token=self.token)
        return self._api

    @property
    def download(self):
        if self._download is None:
            self._download = need("huggingface_hub", "downloading from the Hub").snapshot_download
        return self._download

    # -- naming
    def namespace(self) -> str:
        name = self.environ.get("HF_USERNAME")
        if name:
            return name
        info = self.api.whoami() or {}
        name = info.get("name") or info.get("user")
        if not name:
            raise RuntimeError("cannot resolve the Hub namespace; set HF_USERNAME")
        return name

    def repo_id(self, run_name: str, namespace: Optional[str] = None, prefix: str = REPO_PREFIX) -> str:
        return f"{namespace or self.namespace()}/{prefix}-{run_name}"

    # -- stages
    def publish_stage(self, repo_id: str, stage: str, folder, *, private: bool = False, message: str = "",
                      tag: Optional[str] = None) -> str:
        if (Path(folder) / "checkpoint.ckpt").exists():
            read_stage(folder)          # refuse to publish a folder whose artefacts do not carry their magic
        self.api.create_repo(repo_id=repo_id, repo_type="model", private=private, exist_ok=True)
        self.api.upload_folder(repo_id=repo_id, repo_type="model", folder_path=str(folder), path_in_repo=str(stage),
                               commit_message=message or f"stage {stage}", token=self.token)
        if tag:
            self.api.create_tag(repo_id=repo_id, tag=tag, repo_type="model", token=self.token)
        return str(stage)

    def publish_file(self, repo_id: str, path_in_repo: str, local_path, message: str = "") -> str:
        self.api.upload_file(repo_id=repo_id, repo_type="model", path_or_fileobj=str(local_path),
                             path_in_repo=str(path_in_repo), commit_message=message or f"add {path_in_repo}",
                             token=self.token)
        return str(path_in_repo)

    def fetch_stage(self, repo_id: str, stage: str, dest, *, revision: str = "main",
                    files: Sequence[str] = LOAD_FILES) -> Path:
        local = self.download(repo_id=repo_id, repo_type="model", revision=revision, local_dir=str(dest),
                              token=self.token, allow_patterns=[f"{stage}/{n}" for n in files])
        return Path(local) / str(stage)

    # -- tokenizers
    def publish_tokenizer(self, repo_id: str, vocab_size: int, local_path, message: str = "") -> str:
        _check_magic(Path(local_path), TOKENIZER_MAGIC, "an NCTOKEN1 tokenizer")
        self.api.create_repo(repo_id=repo_id, repo_type="model", exist_ok=True)
        return self.publish_file(repo_id, tokenizer_file(vocab_size), local_path, message)

    def fetch_tokenizer(self, repo_id: str, vocab_size: int, dest, *, revision: str = "main") -> Optional[Path]:
        """The local path, or None when the repository does not have that vocabulary size (the caller trains one)."""
        name = tokenizer_file(vocab_size)
        try:
            local = self.download(repo_id=repo_id, repo_type="model", revision=revision, local_dir=str(dest),
                                  token=self.token, allow_patterns=[name])
        except Exception:       # any miss (no repository, no file, no network) means "train it"
            return None
        path = Path(local) / name
        return path if path.is_file() else None

    # -- pretraining shards
    def fetch_shards(self, dest, *, repo_id: str = PRETRAIN_DATASET, shards: Sequence[str] = PRETRAIN_SHARDS) -> Path:
        """Download the shards that are not in `dest` yet; cheap to call on every run."""
        dest = Path(dest)
        wanted = [s for s in shards if not (dest / s).is_file()]
        if wanted:
            self.download(repo_id=repo_id, repo_type="dataset", local_dir=str(dest), allow_patterns=wanted,
                          token=self.token)
        return dest
