"""``triattention.models`` (models.py of the reference): the module object of ``triattention_b200.models``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("triattention_b200.models")
