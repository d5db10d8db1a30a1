"""Band-map loading (``triattention-map-v1``).

Same behaviour as ``triattention/maps.py:1-41``: the loader reads only ``["bands"]`` —
``{"<layer>": [[w8, w4] per Q head]}`` in tile-distance units with ``INF = 1 << 20`` — and validates
it against the model's layer and head counts (``ValueError`` on mismatch).  One optional extension
field is understood and ignored by older readers: ``"bf16_kv_heads": {"<layer>": [kv head, ...]}``
marks KV heads that stay un-quantised (BF16); v1 maps without it load exactly as before.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

INF = 1 << 20
DATA = Path(os.environ.get("TRIATTENTION_MAP_DIR", Path(__file__).resolve().parent / "data"))
PRESETS = {"llama": "llama-3.2-3b-instruct", "qwen2": "qwen2-7b-instruct", "mistral3": "ministral-3-8b-instruct-2512"}


def preset(model):
    """maps.py:10-17.  The selected maps are data files of the reference project; they are looked up in
    ``TRIATTENTION_MAP_DIR`` (default: this package's ``data/`` directory)."""
    name = PRESETS.get(model.config.model_type)
    if name is None:
        raise ValueError(f"no bundled map for model type {model.config.model_type!r}; pass --map")
    path = DATA / f"{name}.json"
    if not path.is_file():
        raise ValueError(f"map {path} not found; pass --map or set TRIATTENTION_MAP_DIR")
    return path


def load_map(path, model=None):
    doc = json.loads(Path(path).read_text())
    return from_bands(doc["bands"], model, doc.get("bf16_kv_heads"))


def from_bands(bands, model=None, bf16_kv_heads=None):
    if model is not None:
        text = getattr(model.config, "text_config", model.config)
        if len(bands) != text.num_hidden_layers or len(bands["0"]) != text.num_attention_heads:
            raise ValueError("the map does not match the model's layers and heads")

    def bands_fn(layer, heads):
        return torch.tensor(bands[str(layer)], dtype=torch.int32)

    if bf16_kv_heads:
        bands_fn.bf16_kv_heads = lambda layer: tuple(int(h) for h in bf16_kv_heads.get(str(layer), ()))
    return bands_fn


def uniform(w8, w4):
    def bands_fn(layer, heads):
        return torch.tensor([[w8, w4]] * heads, dtype=torch.int32)

    bands_fn.layer_independent = True
    return bands_fn


def per_kv_head(kinds, group):
    """Map in the vocabulary of the benchmark configurations: one of "int8" / "int4" / "bf16" per KV head, expanded to Q-head bands
    (INT8 -> [INF, INF], INT4 -> [1, INF]) plus the BF16 head list.  Layer independent."""
    table = {"int8": [INF, INF], "int4": [1, INF], "bf16": [INF, INF]}
    rows = [table[kind] for kind in kinds for _ in range(group)]
    bf16 = tuple(i for i, kind in enumerate(kinds) if kind == "bf16")

    def bands_fn(layer, heads):
        if heads != len(rows):
            raise ValueError("the map does not match the model's layers and heads")
        return torch.tensor(rows, dtype=torch.int32)

    bands_fn.layer_independent = True
    if bf16:
        bands_fn.bf16_kv_heads = lambda layer: bf16
    return bands_fn
