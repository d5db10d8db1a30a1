"""``triattention.kernels.decode`` (kernels/decode.py of the reference): the module object of ``triattention_b200.kernels.decode``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("triattention_b200.kernels.decode")
