from .gpt import GPT  # noqa: F401
from .params import ParamStore, init_weights, param_specs  # noqa: F401
