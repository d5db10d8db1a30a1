"""The reference's package name over the sm_100a implementation.

Code written against the reference (``from triattention import TriAttention``, ``python -m triattention.infer``,
``from triattention.kernels.prefill import Prefill``, ``from triattention.maps import uniform`` ...) resolves here to
the modules of ``triattention_b200``: every submodule of this package IS the module of the same name there (the same
module object), so classes compare equal and attributes set on one are seen through the other.
Public names as in ``triattention/__init__.py:1-3`` of the reference; the model glue is imported lazily.
"""
__all__ = ["TriAttention", "eos_ids", "load_model", "load_tokenizer", "render_prompt"]


def __getattr__(name):
    if name in __all__:
        from triattention_b200 import models
        return getattr(models, name)
    raise AttributeError(name)
