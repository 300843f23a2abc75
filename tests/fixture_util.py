"""Helpers shared by the fixture-parity tests: build a model / optimizer from the records of a fixture."""
import os

import numpy as np
import torch

from nanochat_cpp_b200.config import Config
from nanochat_cpp_b200.data.record_file import read_records
from nanochat_cpp_b200.models import GPT
from nanochat_cpp_b200.optim import OptimizerConfig, SchedulerConfig


def load(data_dir, name):
    return read_records(os.path.join(data_dir, name))[1]


def config_of(recs, pre="config/") -> Config:
    g = lambda k: int(recs[pre + k][0])
    return Config(num_layers=g("layers"), num_heads=g("heads"), num_kv_heads=g("kv_heads"), hidden_dim=g("embd"),
                  seq_len=g("seq"), vocab_size=g("vocab"), padded_vocab_size=g("padded_vocab"), rope_base=100000.0,
                  window_pattern=bytes(recs[pre + "window_pattern"]).decode())


def model_of(recs, prefix="param/", cfg=None):
    cfg = cfg or config_of(recs)
    m = GPT(cfg, "cpu", torch.float32, init=False)
    sd = {}
    for s in m.params.specs:
        a = np.array(recs[prefix + s.name])
        sd[s.name] = torch.from_numpy(a).reshape(s.shape)
    m.load_state_dict(sd)
    return cfg, m


def optim_of(recs, pre="config/"):
    o = lambda k, d=None: float(recs[pre + "opt/" + k][0]) if pre + "opt/" + k in recs else d
    s = lambda k, d=None: float(recs[pre + "sched/" + k][0]) if pre + "sched/" + k in recs else d
    oc = OptimizerConfig(unembedding_lr=o("unembedding_lr"), embedding_lr=o("embedding_lr"), matrix_lr=o("matrix_lr"),
                         scalar_lr=o("scalar_lr"), weight_decay=o("weight_decay", 0.0), clip=o("clip", 0.0),
                         adam_eps=o("adam_eps"), muon_ns_steps=int(o("muon_ns_steps", 5)),
                         muon_beta2=o("muon_beta2", 0.9))
    sc = SchedulerConfig(num_iterations=int(s("num_iterations", 0)), warmup_steps=int(s("warmup_steps", 0)),
                         warmdown_ratio=s("warmdown_ratio", 0.0), final_lr_frac=s("final_lr_frac", 0.0),
                         weight_decay_base=s("weight_decay_base", 0.0),
                         muon_momentum_warmup_steps=s("muon_momentum_warmup_steps", 0.0),
                         muon_momentum_start=s("muon_momentum_start", 0.95),
                         muon_momentum_peak=s("muon_momentum_peak", 0.95),
                         muon_momentum_final=s("muon_momentum_final", 0.95))
    return oc, sc
