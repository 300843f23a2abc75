from .engine import (GeneratedSequence, GenerateParams, InferenceEngine, PagedKVCache, generate,  # noqa: F401
                     generate_multi, sample)
