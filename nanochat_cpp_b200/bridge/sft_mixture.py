"""The supervised fine-tuning mixture over hub datasets: SmolTalk once, MMLU auxiliary-train three times, GSM8K train
four times (upstream nanochat's `scripts/chat_sft.py` multipliers); validation = the matching test splits capped at
5,200 MMLU and 420 GSM8K rows so the task ratios stay those of training.

The task classes here only add the dataset access to `chat.tasks` (prompt format, tool-call parts and scoring are
inherited); every dataset is shuffled with seed 42 as upstream does, and rows stay in the parquet table until they are
asked for. `MixtureBuilder(loader)` takes the loader callable (`hub_data.hub_loader()` or a fake), so nothing here
touches the network by itself. Counterpart of the reference's python/nanochat_cpp_bridge/sft_reference.py.
"""
from __future__ import annotations

from typing import Callable, Optional

from ..chat.sft_data import TaskMixture
from ..chat.tasks import GSM8K, MMLU, Task

SMOLTALK_REPO = "HuggingFaceTB/smol-smoltalk"
MMLU_REPO = "cais/mmlu"
GSM8K_REPO = "openai/gsm8k"
MMLU_EPOCHS, GSM8K_EPOCHS = 3, 4
VAL_MMLU_ROWS, VAL_GSM8K_ROWS = 5200, 420
SHUFFLE_SEED = 42


class LazyRows:
    """A strided window over an indexable dataset; rows are materialised one at a time."""

    def __init__(self, source, start: int = 0, stop: Optional[int] = None, step: int = 1):
        self.source = source
        self.index = range(len(source))[start:stop:step]

    def lazy_slice(self, start, stop, step):
        view = LazyRows(self.source)
        view.index = self.index[start:stop:step]
        return view

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int) -> dict:
        return self.source[self.index[i]]


def _rows(loader, repo, subset, split):
    return LazyRows(loader(repo, subset, split).shuffle(SHUFFLE_SEED))


class SmolTalk(Task):
    """General conversations. A conversation must be (optional system,) user, assistant, user, ... with string
    contents; a malformed one fails here, with its index, not inside the renderer."""

    def __init__(self, loader: Callable, split: str = "train", **kw):
        if split not in ("train", "test"):
            raise ValueError("SmolTalk split must be train or test")
        super().__init__(_rows(loader, SMOLTALK_REPO, "default", split), **kw)

    def get_example(self, i):
        messages = self.rows[i]["messages"]
        body = messages[1:] if messages and messages[0]["role"] == "system" else messages
        if len(body) < 2:
            raise ValueError(f"SmolTalk row {i}: fewer than two turns")
        for k, m in enumerate(body):
            want = "user" if k % 2 == 0 else "assistant"
            if m["role"] != want or not isinstance(m["content"], str):
                raise ValueError(f"SmolTalk row {i}: turn {k} is {m['role']!r}, expected {want!r} with text content")
        return {"messages": messages}


class HubMMLU(MMLU):
    def __init__(self, loader: Callable, subset: str = "all", split: str = "test", **kw):
        if subset != "all" or split not in ("auxiliary_train", "validation", "dev", "test"):
            raise ValueError("MMLU: subset all; split auxiliary_train, validation, dev or test")
        Task.__init__(self, _rows(loader, MMLU_REPO, subset, split), **kw)


class HubGSM8K(GSM8K):
    def __init__(self, loader: Callable, subset: str = "main", split: str = "train", **kw):
        if subset not in ("main", "socratic") or split not in ("train", "test"):
            raise ValueError("GSM8K: subset main or socratic; split train or test")
        Task.__init__(self, _rows(loader, GSM8K_REPO, subset, split), **kw)


class MixtureBuilder:
    """`builder("train" | "val" | "demo", **options)` -> TaskMixture."""

    def __init__(self, loader: Optional[Callable] = None):
        if loader is None:
            from .hub_data import hub_loader
            loader = hub_loader()
        self.loader = loader

    def train(self, mmlu_epochs: int = MMLU_EPOCHS, gsm8k_epochs: int = GSM8K_EPOCHS) -> TaskMixture:
        ld = self.loader
        return TaskMixture([SmolTalk(ld, "train")] + [HubMMLU(ld, "all", "auxiliary_train") for _ in range(mmlu_epochs)]
                           + [HubGSM8K(ld, "main", "train") for _ in range(gsm8k_epochs)])

    def val(self) -> TaskMixture:
        ld = self.loader
        return TaskMixture([SmolTalk(ld, "test"), HubMMLU(ld, "all", "test", stop=VAL_MMLU_ROWS),
                            HubGSM8K(ld, "main", "test", stop=VAL_GSM8K_ROWS)])

    def demo(self, limit: int = 64) -> TaskMixture:
        """The first `limit` rows of each training task (the shards still download whole)."""
        ld = self.loader
        return TaskMixture([SmolTalk(ld, "train", stop=limit), HubMMLU(ld, "all", "auxiliary_train", stop=limit),
                            HubGSM8K(ld, "main", "train", stop=limit)])

    def __call__(self, kind: str = "train", **options) -> TaskMixture:
        if kind not in ("train", "val", "demo"):
            raise ValueError(f"unknown mixture '{kind}' (train, val, demo)")
        return getattr(self, kind)(**options)
