"""B200-native (sm_100a) implementation of TriAttention's quantised attention path.

Same public names as the reference package (``triattention/__init__.py:1-3``); the model glue is
imported lazily so that the kernels can be used without transformers.
"""
__all__ = ["TriAttention", "eos_ids", "load_model", "load_tokenizer", "render_prompt"]


def __getattr__(name):
    if name in __all__:
        from triattention_b200 import models
        return getattr(models, name)
    raise AttributeError(name)
