"""Code written against the reference's import paths resolves to this implementation.

Only names of the reference project are used here (`triattention`, `triattention.infer`, `.models`, `.maps`,
`.kernels.prefill`, `.kernels.decode`, `.kernels.extension`; reference files triattention/__init__.py:1-3, infer.py:8-18,
maps.py:8-41, kernels/prefill.py:7-40, kernels/decode.py:9-22)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_package_and_submodules_resolve():
    import triattention
    from triattention import TriAttention, eos_ids, load_model, load_tokenizer, render_prompt   # noqa: F401
    from triattention.kernels.decode import NEAR_V8, DecodeCache
    from triattention.kernels.extension import load_extension
    from triattention.kernels.prefill import F16, I4, I8, Q4, SKIP, BandTable, Prefill
    from triattention.maps import INF, PRESETS, from_bands, load_map, preset, uniform   # noqa: F401
    from triattention.models import exact_attention, use_attention   # noqa: F401
    assert triattention.__all__ == ["TriAttention", "eos_ids", "load_model", "load_tokenizer", "render_prompt"]
    assert (SKIP, F16, I8, I4, Q4) == (0, 1, 2, 3, 4) and NEAR_V8 == 16 and INF == 1 << 20
    assert set(PRESETS) == {"llama", "qwen2", "mistral3"}
    assert callable(load_extension) and callable(Prefill) and callable(DecodeCache) and callable(BandTable.build)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="requires a CUDA GPU"):      # extension.py:15-16 of the reference
            load_extension()


def test_calibrate_style_callers_on_cpu():
    """`Prefill(module, uniform(w8, w4))` with a shared `.buffers` dict, `uniform`'s layer_independent flag, and
    `BandTable.build` (calibrate.py:44-48 and select.py:36-39 of the reference use exactly these)."""
    from triattention.kernels.decode import DecodeCache
    from triattention.kernels.prefill import Q4, BandTable, Prefill
    from triattention.maps import INF, uniform
    fn = uniform(2, 5)
    assert fn.layer_independent and fn(3, 4).tolist() == [[2, 5]] * 4
    shared = {}
    a, b = Prefill(None, uniform(INF, INF)), Prefill(None, fn)
    a.buffers = shared
    b.buffers = shared
    assert a.buffers is b.buffers and a.decode_cache is None
    table = BandTable.build(fn(0, 4), 12, 2, "cpu")
    assert Q4 in table.formats and table.order.numel() == 4 * 12 and table.bands.tolist() == [[2, 5]] * 4
    cache = DecodeCache(None, 8)
    codes, formats = cache.codes(40)
    assert codes.tolist()[:2] == [2, 3] and formats == frozenset({2, 3}) and not cache.stored(0)


def test_calibrate_entry_point_flags():
    """python -m triattention.calibrate takes the reference tool's flags (calibrate.py:33-39)."""
    from triattention.calibrate import W4, W8, grid
    assert len(W8) == 11 and len(W4) == 12 and len(grid()) == 86
    out = subprocess.run([sys.executable, "-m", "triattention.calibrate", "--help"], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    for flag in ("--model", "--samples", "--output", "--rows", "--response-tokens"):
        assert flag in out.stdout


def test_infer_entry_point_flags():
    out = subprocess.run([sys.executable, "-m", "triattention.infer", "--help"], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0
    for flag in ("--model", "--prompt", "--map", "--max-new-tokens"):
        assert flag in out.stdout
