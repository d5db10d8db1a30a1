"""``triattention.kernels.extension`` (kernels/extension.py of the reference): the module object of ``triattention_b200.kernels.extension``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("triattention_b200.kernels.extension")
