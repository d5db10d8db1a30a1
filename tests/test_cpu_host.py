"""CPU checks of the host side: blob layouts, map loading, band tables, cache planning, and that the
C-ABI library loads and exports every symbol the header declares (no compute calls)."""
import ctypes
import json
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import triattention_oracle as orc
from triattention_b200 import maps
from triattention_b200.kernels import decode as dec
import layouts
from triattention_b200.kernels.extension import SIGNATURES, load_library
from triattention_b200.kernels.prefill import F16, I8, Q4, BandTable

ROOT = Path(__file__).resolve().parent.parent


# ---- blob layouts: the numpy packers follow the index formulas of csrc/kv_write.cu -----------------------
def test_k8_blob_formula():
    codes = np.random.default_rng(0).integers(-127, 128, (64, 128), dtype=np.int8)
    blob = layouts.pack_k8(codes).view(np.int8)
    for r, c in ((0, 0), (5, 17), (63, 127), (40, 96), (9, 15)):
        assert blob[(r // 8) * 1024 + (c // 16) * 128 + (r % 8) * 16 + c % 16] == codes[r, c]
    assert (layouts.unpack_k8(layouts.pack_k8(codes)) == codes).all()


def test_k4_blob_formula():
    rng = np.random.default_rng(1)
    blob = rng.integers(0, 256, 4096, dtype=np.uint8)
    codes = layouts.unpack_k4(blob)
    for r, c in ((0, 0), (5, 17), (63, 127), (40, 96), (9, 47)):
        byte = int(blob[(r // 8) * 512 + (r % 8) * 64 + (c // 32) * 16 + ((c % 32) // 8) * 4 + c % 4])
        nib = (byte >> 4) if (c % 8) >= 4 else (byte & 0xF)
        assert codes[r, c] == (nib - 16 if nib > 7 else nib)


def test_v_blob_formulas():
    rng = np.random.default_rng(2)
    v = rng.integers(-127, 128, (64, 128), dtype=np.int8)        # [key][channel]
    blob = layouts.pack_v8(v).view(np.int8)
    for key, ch in ((0, 0), (13, 5), (63, 127), (34, 77)):
        blk, k16 = key // 16, key % 16
        pos = int(np.nonzero(layouts.KPERM == k16)[0][0])
        assert blob[(ch // 8) * 512 + blk * 128 + (ch % 8) * 16 + pos] == v[key, ch]
    assert (layouts.unpack_v8(layouts.pack_v8(v)) == v).all()
    b4 = rng.integers(0, 256, 4096, dtype=np.uint8)
    v4 = layouts.unpack_v4(b4)
    for key, ch in ((0, 0), (13, 5), (63, 127), (34, 77), (50, 3)):
        kc, k32 = key // 32, key % 32
        pos = int(np.nonzero(layouts.KPERM == k32 % 16)[0][0])
        byte = int(b4[(ch // 8) * 256 + kc * 128 + (ch % 8) * 16 + pos])
        nib = (byte >> 4) if k32 >= 16 else (byte & 0xF)
        assert v4[key, ch] == (nib - 16 if nib > 7 else nib)
    h = rng.standard_normal((64, 128)).astype(np.float16)
    assert (layouts.unpack_v16(layouts.pack_v16(h)) == h).all()
    b16 = layouts.pack_v16(h).view(np.float16)
    assert b16[(77 // 8) * 512 + (34 // 8) * 64 + (77 % 8) * 8 + 34 % 8] == h[34, 77]
    assert sorted(layouts.KPERM.tolist()) == list(range(16))


def test_swizzle128_is_an_involution_per_row_group():
    rows = np.arange(16 * 128, dtype=np.uint8).reshape(16, 128)
    img = layouts.swizzle128(rows)
    assert (layouts.swizzle128(img) == rows).all()
    assert (img[0] == rows[0]).all() and (img[1, :16] == rows[1, 16:32]).all()


# ---- maps --------------------------------------------------------------------------------------------
class _Cfg:
    def __init__(self, layers, heads, model_type="llama"):
        self.num_hidden_layers, self.num_attention_heads, self.model_type = layers, heads, model_type


class _Model:
    def __init__(self, layers, heads, model_type="llama"):
        self.config = _Cfg(layers, heads, model_type)


def test_load_map_v1(tmp_path):
    doc = dict(format="triattention-map-v1", model_type="llama", length=65536, c4=0.905, point=0.8, cost=0.79,
               bands={"0": [[maps.INF, maps.INF], [2, 16]], "1": [[1, 4], [8, maps.INF]]})
    path = tmp_path / "m.json"
    path.write_text(json.dumps(doc))
    fn = maps.load_map(path, _Model(2, 2))
    assert fn(1, 2).tolist() == [[1, 4], [8, maps.INF]] and fn(0, 2).dtype == torch.int32
    assert not hasattr(fn, "bf16_kv_heads")
    with pytest.raises(ValueError):
        maps.load_map(path, _Model(3, 2))
    with pytest.raises(ValueError):
        maps.load_map(path, _Model(2, 4))
    doc["bf16_kv_heads"] = {"1": [0]}
    path.write_text(json.dumps(doc))
    fn = maps.load_map(path, _Model(2, 2))
    assert fn.bf16_kv_heads(1) == (0,) and fn.bf16_kv_heads(0) == ()


def test_uniform_and_presets():
    fn = maps.uniform(4, 8)
    assert fn.layer_independent and fn(3, 5).tolist() == [[4, 8]] * 5
    with pytest.raises(ValueError):
        maps.preset(_Model(1, 1, "gpt2"))
    fn = maps.per_kv_head(["int8", "int4", "bf16"], 2)
    assert fn(0, 6).tolist() == [[maps.INF, maps.INF]] * 2 + [[1, maps.INF]] * 2 + [[maps.INF, maps.INF]] * 2
    assert fn.bf16_kv_heads(0) == (2,)


# ---- band table ----------------------------------------------------------------------------------------
def test_band_table_matches_oracle():
    bands = [[maps.INF, maps.INF], [2, 3], [1, maps.INF], [1, 1]]
    for rows in (1, 2, 5, 40):
        table = BandTable.build(bands, rows, 2, "cpu")
        assert set(table.formats) == orc.band_formats(np.asarray(bands), rows)
        assert (table.order.numpy() == orc.cta_order(4, 2, rows)).all()
        assert table.bands.tolist() == bands
    assert BandTable.build([[1, 1]] * 2, 9, 1, "cpu").formats == frozenset({F16})
    assert BandTable.build([[2, 2]] * 2, 9, 1, "cpu").formats == frozenset({F16, I8})
    assert Q4 in BandTable.build([[1, 2]] * 2, 9, 1, "cpu").formats
    with pytest.raises(ValueError):
        BandTable.build([[0, 4]] * 2, 9, 1, "cpu")
    t = BandTable.build(bands, 5, 2, "cpu", bf16_kv=(1,))
    assert t.bands.tolist() == bands[:2] + [[0, 0], [0, 0]] and t.host.tolist() == bands


# ---- cache planning ---------------------------------------------------------------------------------------
def test_plan_matches_reference_tile_rules():
    bands = np.array([[2, 5], [1, 3], [maps.INF, maps.INF], [1, 1]])
    prompt = 64 * 40 - 7
    plan = dec.plan_streams(bands, 2, prompt, batch=3, ctas=16)
    tabs = orc.decode_tables(bands, 2, prompt)
    for kh in range(2):
        rows = plan["tmeta"][plan["tab_begin"][kh]:plan["tab_begin"][kh] + plan["count"][kh]]
        info = rows[:, 1].astype(np.int64)
        assert (info & 0xFFF).tolist() == tabs[kh]["tiles"].tolist()
        assert ((info >> 12) & 0xFF).tolist() == tabs[kh]["rowmask"].tolist()
        assert (((info >> 20) & 1) == (tabs[kh]["state"] == 4)).all()
        assert (((info >> 21) & 1) == (tabs[kh]["vfmt"] == orc.I4)).all()
        size = np.where(tabs[kh]["state"] == 4, 4096, 8192) + np.where(tabs[kh]["vfmt"] == orc.I4, 4096, 8192) + 16
        assert (rows[:, 0].astype(np.int64) * 16 == np.concatenate([[0], np.cumsum(size)[:-1]])).all()


def test_plan_work_list_covers_every_tile_once():
    bands = np.array([[maps.INF, maps.INF]] * 4 + [[1, maps.INF]] * 2 + [[4, 9]] * 2)
    for bf16 in ((), (1,), (0, 3)):
        plan = dec.plan_streams(bands, 4, 8192, batch=5, bf16_kv=bf16, ctas=64)
        units = 20
        seen = [np.zeros(plan["unit_count"][u], int) for u in range(units)]
        slots = set()
        for u, first, cnt, slot in plan["segments"]:
            seen[u][first:first + cnt] += 1
            assert cnt > 0 and slot not in slots
            slots.add(slot)
            lo, n = plan["unit_slots"][u]
            assert lo <= slot < lo + n
        assert all((s == 1).all() for s in seen) and len(slots) == plan["slots"]
        # every CTA owns a contiguous run of segments, and the runs are balanced by cost
        cs = plan["cta_segments"]
        assert cs[0] == 0 and cs[-1] == len(plan["segments"]) and (np.diff(cs) >= 0).all() and len(cs) == 65
        sizes = {u: None for u in range(units)}
        cost = np.zeros(64)
        for c in range(64):
            for u, first, cnt, slot in plan["segments"][cs[c]:cs[c + 1]]:
                rows = plan["tmeta"][plan["unit_tab"][u] + first:plan["unit_tab"][u] + first + cnt]
                info = rows[:, 1].astype(np.int64)
                bf, k4, v4 = info >> 22 & 1, info >> 20 & 1, info >> 21 & 1
                cost[c] += np.where(bf == 1, dec.TILE_COSTS[0], np.where((k4 == 0) & (v4 == 0), dec.TILE_COSTS[1], dec.TILE_COSTS[2])).sum()
        assert cost.max() - cost.min() <= 2 * max(dec.TILE_COSTS)
        # streams do not overlap and stay inside the pool
        ends = plan["unit_base"] + plan["head_bytes"][np.arange(units) % 4]
        order = np.argsort(plan["unit_base"])
        assert (plan["unit_base"][order][1:] >= ends[order][:-1]).all() and ends.max() <= plan["pool_bytes"]
        assert (plan["unit_flags"] == np.isin(np.arange(units) % 4, list(bf16))).all()


def test_plan_c2_byte_model():
    """benchmark configuration 2: 8 KV heads (4 INT8, 2 INT4, 2 BF16), cache of 8192 tokens, batch 32."""
    bands = np.array([[maps.INF, maps.INF]] * 12 + [[1, maps.INF]] * 6 + [[maps.INF, maps.INF]] * 6)
    plan = dec.plan_streams(bands, 8, 8192, batch=32, bf16_kv=(6, 7), ctas=444)
    assert plan["head_bytes"].tolist() == [1644544] * 4 + [1128448] * 2 + [4194304] * 2
    assert plan["payload_bytes"] == 551157760


def test_needs_k4():
    assert dec.DecodeCache.needs_k4(np.array([[1, maps.INF]] * 2), 1, 5)
    assert not dec.DecodeCache.needs_k4(np.array([[maps.INF, maps.INF]] * 2), 1, 5)
    assert not dec.DecodeCache.needs_k4(np.array([[1, maps.INF]] * 2), 1, 1)


# ---- C ABI ------------------------------------------------------------------------------------------------
def header_functions():
    text = (ROOT / "include" / "triattention_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    found = {}
    for m in re.finditer(r"\b(?:int|const char\*)\s+(tri_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        found[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return found


def test_library_exports_every_declared_symbol():
    lib = load_library()
    declared = header_functions()
    assert set(SIGNATURES) | {"tri_last_error"} == set(declared), set(SIGNATURES) ^ set(declared)
    for name, nargs in declared.items():
        assert hasattr(lib, name), name
        if name in SIGNATURES:
            assert len(SIGNATURES[name]) == nargs, (name, len(SIGNATURES[name]), nargs)
    assert lib.tri_abi_version() == 5
    assert isinstance(lib.tri_last_error(), bytes)


def test_argument_errors_without_gpu():
    """Validation happens before any CUDA call, so it can be exercised on CPU."""
    lib = load_library()
    assert lib.tri_prepare_qk(*([None] * 2), 1, 8, 2, 64, *([0] * 6), *([None] * 13)) == -1
    assert b"null" in lib.tri_last_error()
    assert lib.tri_pack_v(None, 1, 2, 64, 0, 0, 0, *([None] * 8)) == -1


def test_error_word_is_keyed_by_the_device_that_ran_the_kernel(monkeypatch):
    """"cuda" without an index means the current device, not device 0: on rank r > 0 the kernels write the word of
    cuda:r, and the check must read that one."""
    import torch
    from triattention_b200.kernels.extension import Module
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 3)
    assert Module._device_index("cuda") == 3 and Module._device_index(torch.device("cuda")) == 3
    assert Module._device_index("cuda:1") == 1 and Module._device_index(torch.device("cuda", 5)) == 5
    assert Module._device_index(2) == 2
    m = Module(lib=None)
    m._errors = {0: torch.zeros(1, dtype=torch.int32), 3: torch.full((1,), 4, dtype=torch.int32)}
    with pytest.raises(RuntimeError, match="device error 4 on cuda:3"):
        m.check_device_error()                  # no argument: every device this process launched on
    assert int(m._errors[3].item()) == 0        # reported once, then cleared
    m.check_device_error()
    m._errors[3].fill_(1)
    m.check_device_error("cuda:0")              # another device's word is not this call's business
    with pytest.raises(RuntimeError, match="device error 1"):
        m.check_device_error("cuda")            # the current device (3)
    # a prefill wait that ran out leaves its site (and the tile's step) in the upper bits: 1 | 11 << 8 | 37 << 16
    m._errors[0].fill_(1 | (11 << 8) | (37 << 16))
    with pytest.raises(RuntimeError, match="device error 1 on cuda:0, wait site 11 at step 37 of the prefill kernel"):
        m.check_device_error()


def test_decode_entry_points_validate_before_any_cuda_call():
    lib = load_library()
    assert lib.tri_decode_merge(None, 0, 0, *([None] * 3), 0, None, None, None, 0, None, 0, 0, None, 0, None,
                                *([None] * 5), 0, 0, None, None, 0, 0, None, None, 0, 0, 1, 8, 2, 4, 0.088, None, None) == -1
    assert b"decode_merge" in lib.tri_last_error()
    assert lib.tri_decode_partials(None, 0, 0, *([None] * 7), 4, *([None] * 8), None, 0, 0, None, 1, 8, 2, 64, 0.088,
                                   None, None) == -1
    assert b"decode_partials" in lib.tri_last_error()
    assert lib.tri_gather_wait(None, 0, None, 0, None, None) == -1 and b"gather_wait" in lib.tri_last_error()


def test_plan_streams_appended_tiles():
    """Tiles appended behind the prompt (DecodeCache(fold_tail=...)): the streams keep their place, the new tiles sit
    where append_off says, are flagged as full and seen by every Q head, and every tile is in exactly one segment."""
    dm, dm_inf = dec, maps.INF
    bands = np.asarray([[dm_inf, dm_inf]] * 2 + [[1, dm_inf]] * 2 + [[dm_inf, dm_inf]] * 2, np.int64)
    plans = [dm.plan_streams(bands, 3, 200, 2, bf16_kv=(2,), ctas=8, extra=e, reserve=3) for e in range(4)]
    tile = dm.K8_BYTES + dm.V8_BYTES + 16
    for e, p in enumerate(plans):
        assert np.array_equal(p["unit_base"], plans[0]["unit_base"]) and p["pool_bytes"] == plans[0]["pool_bytes"]
        assert np.array_equal(p["append_off"], plans[0]["append_off"])
        assert list(p["count"]) == [4 + e, 4 + e, 7 + 2 * e]
        for kh in range(3):
            rows = p["tmeta"][p["tab_begin"][kh]:p["tab_begin"][kh] + p["count"][kh]]
            old = plans[0]["tmeta"][plans[0]["tab_begin"][kh]:plans[0]["tab_begin"][kh] + plans[0]["count"][kh]]
            assert np.array_equal(rows[:len(old)], old)
            new = rows[len(old):]
            step = 2 * dm.BF16_CHUNK_BYTES if kh == 2 else tile
            assert all(int(r[1]) & dm.INFO_FULL and (int(r[1]) >> dm.INFO_ROW_SHIFT) & 0xFF == 0xFF for r in new)
            assert all(bool(int(r[1]) & dm.INFO_BF16) == (kh == 2) and not int(r[1]) & (dm.INFO_K4 | dm.INFO_V4) for r in new)
            offs = [int(r[0]) * 16 for r in new]
            per = step // (2 if kh == 2 else 1)
            assert offs == [int(p["append_off"][kh]) + i * per for i in range(len(new))]
            assert not len(offs) or offs[-1] + per <= p["head_bytes"][kh]
        covered = np.zeros((6, 16), np.int64)
        for unit, first, n, _ in p["segments"]:
            covered[unit, first:first + n] += 1
        for unit in range(6):
            assert (covered[unit, :p["unit_count"][unit]] == 1).all() and not covered[unit, p["unit_count"][unit]:].any()
    with pytest.raises(ValueError):
        dm.plan_streams(bands, 3, 200, 2, ctas=8, extra=1, split=(0, 2))


def test_band_table_q_modes():
    """Which Q codes the attention reads per head: INT8 codes for every quantised head, INT4 codes only where the band
    has an INT4 part for some query block, nothing for heads of un-quantised KV groups."""
    bands = [[maps.INF, maps.INF]] * 2 + [[1, maps.INF]] * 2 + [[2, 2]] * 2 + [[3, 9]] * 2
    table = BandTable.build(bands, 40, 4, "cpu", bf16_kv=(0,))
    assert table.q_modes.tolist() == [0, 0, 3, 3, 1, 1, 3, 3]
    assert BandTable.build(bands, 3, 4, "cpu").q_modes.tolist() == [1, 1, 3, 3, 1, 1, 1, 1]   # 3 tiles: [3, 9] never gets past w8


def test_calibration_grid_and_error_measure():
    """The grid has the reference's 86 points in its order (calibrate.py:13-18), and the batched error measure equals the
    definition evaluated one configuration and one head at a time (calibrate.py:53-62)."""
    from triattention_b200.calibrate import W4, W8, grid, head_errors
    from triattention_b200.maps import INF
    points = grid()
    assert len(points) == 86 and points[0] == (1, 1) and points[-1] == (INF, INF)
    assert points == sorted(points) and len(set(points)) == 86
    assert all(w4 >= w8 and w8 in W8 and (w4 in W4 or w4 == w8) for w8, w4 in points)
    assert [p for p in points if p[0] == INF] == [(INF, INF)]
    assert {w4 for w8, w4 in points if w8 == 4} == {4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, INF}
    g = torch.Generator().manual_seed(5)
    c, h, r, hidden = 11, 3, 7, 40
    exact = torch.randn(h, r, 128, generator=g)
    outputs = (exact[None] + 0.01 * torch.randn(c, h, r, 128, generator=g)).to(torch.bfloat16)
    weight = torch.randn(hidden, h * 128, generator=g).to(torch.bfloat16)
    got = head_errors(outputs, exact, weight, chunk=4)
    assert got.shape == (h, c) and got.dtype == torch.float64
    w = weight.double()
    energy = (exact.double().transpose(0, 1).reshape(r, h * 128) @ w.T).square().sum()
    for ci in range(c):
        for hi in range(h):
            delta = outputs[ci, hi].double() - exact[hi].double()
            want = (delta @ w[:, hi * 128:(hi + 1) * 128].T).square().sum() / energy
            assert abs(got[hi, ci] - want) <= 1e-4 * want


def test_calibration_sample_loader(tmp_path):
    import json
    from triattention_b200.calibrate import load_samples

    class Tokens:
        chat_template = None

        def __call__(self, text, add_special_tokens=False):
            assert add_special_tokens is False
            return type("Enc", (), {"input_ids": [ord(ch) for ch in text]})()

        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
            return "<" + messages[0]["content"] + ">"

    path = tmp_path / "samples.jsonl"
    path.write_text(json.dumps({"prompt": "ab", "response": "wxyz"}) + "\n" + json.dumps({"prompt": "c", "response": "q"}) + "\n")
    samples = load_samples(path, Tokens(), 3)
    assert [n for _, n in samples] == [3, 1]
    assert samples[0][0][-3:] == [ord("w"), ord("x"), ord("y")] and samples[1][0][-1] == ord("q")
    assert len(samples[0][0]) > 3


def test_tail_row_count_for_the_merge_kernel_hint():
    """DecodeCache counts generated tokens on the host for tri_decode_tail_hint: the next call's tail holds one row more
    than tokens generated so far, at most max_tail (the tail saturates), starts again at every fold of 64 rows, and a
    caller that captures the step in a CUDA graph can pin the value."""
    import torch
    from triattention_b200.kernels.decode import DecodeCache
    from triattention_b200.kernels.extension import LONG_TAIL_ROWS
    cache = DecodeCache(None, 8)
    cache.step = torch.zeros(1, dtype=torch.int64)
    seen = []
    for _ in range(12):
        seen.append(cache.tail_rows())
        cache.advance()
    assert seen == [1, 2, 3, 4, 5, 6, 7, 8, 8, 8, 8, 8] and int(cache.step) == 12
    folding = DecodeCache(None, 64, fold_tail=128)
    folding.step = torch.zeros(1, dtype=torch.int64)
    rows = []
    for _ in range(130):
        rows.append(folding.tail_rows())
        folding.advance()
    assert rows[:64] == list(range(1, 65)) and rows[64:128] == list(range(1, 65)) and rows[128:] == [1, 2]
    cache.hint_rows = -1
    assert cache.tail_rows() == -1
    cache.hint_rows = None
    assert cache.tail_rows() == 8 and 1 <= LONG_TAIL_ROWS < 64
