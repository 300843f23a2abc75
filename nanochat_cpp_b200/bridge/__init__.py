"""Adapters to things outside this package: the Hugging Face Hub, hub-hosted task datasets, tiktoken, upstream
PyTorch checkpoints.

The core (`api`, `chat`, `post`, `train`) imports none of this: it takes callables (a dataset loader, a code executor,
a mixture builder) and these modules provide them. Every module here imports its optional dependency inside the call
that needs it, so the package imports on a machine that has none of them, and each network-facing function accepts
the object that does the transfer (`api=`, `download=`), so the tests run with fakes and no network.

Counterpart of the reference's adapter distribution (python/nanochat_cpp_bridge/: `hf_hub.py`, `reference_data.py`,
`reference_tasks.py`, `sft_reference.py`, `torch_checkpoint.py`).

    extras.py          which optional package a feature needs, and the error that says so
    hub.py             checkpoint stages as Hub folders: write / publish / fetch, tokenizer and dataset files
    hub_data.py        parquet-backed hub datasets with the `datasets` shuffle order; sandboxed code executor
    sft_mixture.py     the SmolTalk + MMLU + GSM8K supervised mixture over hub datasets
    tiktoken_tok.py    a tiktoken encoding built from an NCTOKEN1 artefact
    torch_checkpoint   = `nanochat_cpp_b200.train.convert` (upstream `.pt` <-> NCHKPT01), re-exported here
"""
from ..train import convert as torch_checkpoint  # noqa: F401
from .extras import MissingExtra  # noqa: F401
