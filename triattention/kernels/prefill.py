"""``triattention.kernels.prefill`` (kernels/prefill.py of the reference): the module object of ``triattention_b200.kernels.prefill``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("triattention_b200.kernels.prefill")
