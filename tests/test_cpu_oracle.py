"""CPU checks of the oracle: internal consistency, the reference's packed layouts, and the golden vectors
recorded from the reference's own CUDA extension on a B200 (tests/golden/*.npz)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import scipy.linalg

import triattention_oracle as orc
from util import ABS_TOL, code_mismatch, fp_report, from_bits, ulp_diff

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))


def test_rotation_is_signed_hadamard():
    x = orc.synth((3, 5, 128), 0).astype(np.float64)
    h = scipy.linalg.hadamard(128).astype(np.float64)
    want = (x * orc.SIGNS) @ h / np.sqrt(128.0)
    assert np.abs(orc.rotate128(x.astype(np.float32)) - want).max() < 2e-6
    assert int((orc.SIGNS < 0).sum()) == 66


def test_rotation_preserves_norm_and_inverts():
    x = orc.synth((2, 7, 128), 1)
    y = orc.rotate128(x)
    assert np.allclose(np.linalg.norm(x, axis=-1), np.linalg.norm(y, axis=-1), rtol=1e-5)
    back = orc.rotate128(y * orc.SIGNS) * orc.SIGNS     # H is symmetric and orthogonal
    assert np.abs(back - x).max() < 1e-5


@pytest.mark.parametrize("words,unpack,signed4", [(2048, orc.unpack_ref_k8, False), (1024, orc.unpack_ref_k4, True),
                                                  (2048, orc.unpack_ref_v8, False), (1024, orc.unpack_ref_v4, True)])
def test_reference_layouts_are_bijections(words, unpack, signed4):
    rng = np.random.default_rng(words)
    raw = rng.integers(0, 2 ** 32, (1, 2, words), dtype=np.uint64).astype(np.uint32)
    out = unpack(raw)
    assert out.shape == (1, 2, 64, 128)
    # every packed element lands on a distinct logical position: changing one word changes exactly its elements
    raw2 = raw.copy()
    raw2[0, 1, 7] ^= np.uint32(0xFFFFFFFF)
    diff = (unpack(raw2) != out).sum()
    assert diff == (8 if signed4 else 4)


def test_q_quantisation_properties():
    q = orc.synth((2, 9, 128), 3, outlier_dims=(7, 42), outlier_scale=16.0)
    q[0, 0] = 0                                       # an all-zero row keeps zero codes and a zero scale
    q8, qa, q4, qa4 = orc.quantize_q(q)
    assert np.abs(q8).max() == 127 and np.abs(q4).max() == 7
    assert (q8[0, 0] == 0).all() and qa[0, 0] == 0
    x = orc.rotate128(q)
    assert np.abs(q8 * qa[..., None] - x).max() <= qa.max() * 0.5001
    assert np.allclose(qa * 127, qa4 * 7, rtol=1e-6)


def test_stats_order_and_ragged_lengths():
    for t in (1, 63, 64, 65, 200):
        x = orc.synth((2, t, 128), 4)
        stat = orc.channel_stats(x)
        assert np.allclose(stat[:, 0], x.mean(1), atol=1e-5)
        rng = np.maximum(x.max(1) - stat[:, 0], stat[:, 0] - x.min(1))
        assert np.allclose(stat[:, 1], np.where(rng > 0, rng / 127, 1), rtol=1e-6)
    ident = orc.channel_stats(x, identity=True)
    assert (ident[:, 0] == 0).all() and (ident[:, 1] == 1).all() and (ident[:, 2] == 1).all()


def test_band_tiles_match_the_band_definition():
    for qb in range(0, 40):
        for w8, w4 in ((1, 1), (1, 3), (2, 3), (4, 8), (8, 8), (1, orc.INF), (orc.INF, orc.INF)):
            f16, t8, t4 = orc.band_tiles(qb, w8, w4)
            assert f16 == ([0] if qb == 0 else [0, qb])
            assert t8 == [t for t in range(1, qb) if qb - t < w8]
            assert t4 == [t for t in range(1, qb) if w8 <= qb - t < w4]


def test_prefill_close_to_exact_attention_on_mild_inputs():
    q, k, v = orc.synth((4, 150, 128), 5), orc.synth((2, 150, 128), 6), orc.synth((2, 150, 128), 7)
    out = orc.prefill(q, k, v, np.array([[orc.INF, orc.INF]] * 4), 0.0884)
    ex = orc.exact_attention(q, k, v, 0.0884)
    assert np.abs(out - ex).max() < 0.05


def test_decode_is_split_invariant_and_close_to_exact():
    hq, hk, t = 4, 2, 300
    q, k, v = orc.synth((hq, t, 128), 8), orc.synth((hk, t, 128), 9), orc.synth((hk, t, 128), 10)
    bands = np.array([[orc.INF, orc.INF]] * hq)
    _, ops = orc.prefill(q, k, v, bands, 0.0884, return_operands=True)
    qd, kc, vc = orc.synth((hq, 1, 128), 11)[:, 0], orc.synth((hk, 1, 128), 12)[:, 0], orc.synth((hk, 1, 128), 13)[:, 0]
    outs = []
    for per in (None, 1, 3):
        tk, tv = np.zeros((hk, 4, 128), np.float32), np.zeros((hk, 4, 128), np.float32)
        outs.append(orc.decode_step(qd, ops, bands, t, 0.0884, tk, tv, kc, vc, 0, 4, per))
    assert np.abs(outs[0] - outs[1]).max() < 1e-4 and np.abs(outs[0] - outs[2]).max() < 1e-4
    kk, vv = np.concatenate([k, kc[:, None]], 1), np.concatenate([v, vc[:, None]], 1)
    ex = np.stack([orc.exact_decode(qd[h], kk[h // 2], vv[h // 2], 0.0884) for h in range(hq)])
    assert np.abs(outs[0] - ex).max() < 0.05


def test_folded_tail_tiles_stay_close_to_exact_attention():
    """64 generated tokens quantised into one more tile (fold_tail): the result stays an attention over all keys."""
    hq, hk, t = 4, 2, 130
    q, k, v = orc.synth((hq, t, 128), 14), orc.synth((hk, t, 128), 15), orc.synth((hk, t, 128), 16)
    bands = np.array([[orc.INF, orc.INF]] * 2 + [[1, orc.INF]] * 2)
    _, ops = orc.prefill(q, k, v, bands, 0.0884, return_operands=True)
    qd, kd, vd = orc.synth((hq, 66, 128), 17), orc.synth((hk, 66, 128), 18), orc.synth((hk, 66, 128), 19)
    tk, tv = np.zeros((hk, 64, 128), np.float32), np.zeros((hk, 64, 128), np.float32)
    tk[:], tv[:] = kd[:, :64], vd[:, :64]
    tile = orc.fold_tail(ops, tk.copy(), tv.copy())
    assert tile["k8"].shape == (hk, 64, 128) and tile["ka"].shape == (hk, 4) and np.abs(tile["v8"]).max() <= 127
    outs = [orc.decode_step(qd[:, 64 + s], ops, bands, t, 0.0884, tk, tv, kd[:, 64 + s], vd[:, 64 + s], s, 64,
                            appended=[tile]) for s in range(2)]
    for s in range(2):
        kk, vv = np.concatenate([k, kd[:, :65 + s]], 1), np.concatenate([v, vd[:, :65 + s]], 1)
        ex = np.stack([orc.exact_decode(qd[h, 64 + s], kk[h // 2], vv[h // 2], 0.0884) for h in range(hq)])
        assert np.abs(outs[s] - ex).max() < 0.06
    # the split of the tile list must not matter with an appended tile either
    tk2, tv2 = tk.copy(), tv.copy()
    one = orc.decode_step(qd[:, 65], ops, bands, t, 0.0884, tk2, tv2, kd[:, 65], vd[:, 65], 1, 64, per=1, appended=[tile])
    assert np.abs(one - outs[1]).max() < 1e-4


def test_task_table_passes_cover_exact_attention():
    """Task-table mode: when the four passes together name every causal tile once, the block is an attention over all
    keys (sink in the fp16 pass, the others spread over the INT8, INT4-V and INT4-score passes, diagonal last)."""
    hq, hk, t = 2, 1, 330
    q, k, v = orc.synth((hq, t, 128), 31), orc.synth((hk, t, 128), 32), orc.synth((hk, t, 128), 33)
    _, o = orc.prefill(q, k, v, np.array([[orc.INF, orc.INF]] * hq), 0.0884, return_operands=True)
    vstat = orc.channel_stats(v)
    v16, v8, v4 = orc.pack_v(v, vstat)
    ex = orc.exact_attention(q, k, v, 0.0884)
    sl2, qb = orc.sm_log2(0.0884), 4
    rows = slice(qb * 64, (qb + 1) * 64)
    for h in range(hq):
        res = orc.prefill_block(o["q8"][h, rows], o["qa"][h, rows] * sl2, o["k8"][0], o["ka"][0], v16[0], v8[0], vstat[0], t, qb,
                                [0], [1], [3, 4], o["q4"][h, rows], o["qa4"][h, rows] * sl2, o["k4"][0], o["ka4"][0],
                                tiles_i4=[2], v4=v4[0])
        assert np.abs(res - ex[h, rows]).max() < 0.12      # 4-bit weights and 4-bit V on one tile, 4-bit scores on two


def test_decode_tables_rules():
    bands = np.array([[2, 5], [1, 3], [orc.INF, orc.INF], [1, 1]])
    tabs = orc.decode_tables(bands, 2, 64 * 10)
    # head group 0: Q heads 0,1.  tile 0 always kept; d<2 -> 8; d<5 -> 4 for head 0, d<3 -> 4 for head 1
    t0 = dict(zip(tabs[0]["tiles"].tolist(), zip(tabs[0]["state"].tolist(), tabs[0]["rowmask"].tolist())))
    assert t0[0] == (8, 3) and t0[9] == (8, 3) and t0[8] == (8, 1 | 2) and t0[7] == (4, 3) and t0[5] == (4, 1)
    assert 4 not in t0 and 1 not in t0
    assert tabs[1]["tiles"].tolist() == list(range(10)) and (tabs[1]["state"] == 8).all()
    assert tabs[1]["rowmask"].tolist() == [3] + [1] * 8 + [3]
    codes = orc.decode_v_codes(40)
    assert codes[0] == orc.I8 and (codes[1:24] == orc.I4).all() and (codes[24:] == orc.I8).all()


# ---- golden vectors from the reference's CUDA extension ------------------------------------------------
# Allowance of this IEEE restatement against the fast-math kernels, frozen from the recorded vectors:
# measured: scales within 2 ulp, no differing code in the recorded cases.  Bound: 4 ulp, and codes may
# differ by one level on at most 0.05 % of the elements (a scale that moved by an ulp flips a rounding tie).
SCALE_ULP, CODE_RATE = 4, 5e-4


@pytest.mark.parametrize("name", ["small", "c1"])
def test_oracle_matches_reference_golden(name):
    path = GOLDEN / f"{name}.npz"
    if not path.is_file():
        pytest.skip(f"{path.name} has not been recorded yet")
    import make_golden
    g = np.load(path)
    hq, hk, t, _, _, _, keep = make_golden.CASES[name]
    q, k, v, bands, qd, kd, vd = make_golden.inputs(name)
    scale = 1.0 / np.sqrt(128.0)
    out, ops = orc.prefill(q, k, v, bands, scale, return_operands=True)
    for key in ("qa", "qa4", "ka", "ka4"):
        assert ulp_diff(ops[key], g[key]).max() <= SCALE_ULP, key
    assert ulp_diff(ops["kstat"][:, 0], g["kstat"][:, 0]).max() <= SCALE_ULP
    assert ulp_diff(ops["vstat"], g["vstat"]).max() <= SCALE_ULP
    for key, mine in (("q8", ops["q8"][:, ::keep]), ("q4", ops["q4"][:, ::keep]), ("k8", ops["k8"]), ("k4", ops["k4"]),
                      ("v8", ops["v8"]), ("v4", ops["v4"])):
        if key in g:
            rate, big = code_mismatch(mine, g[key])
            assert big <= 1 and rate <= CODE_RATE, (key, rate, big)
    r = fp_report(orc.to_bf16(out)[:, ::keep], from_bits(g["out_bits"]))
    assert r["worst_excess"] <= 0 and r["cos"] >= 0.9999 and r["mean_abs"] <= ABS_TOL / 4, r
    for per in (2, 1000):
        tk, tv = np.zeros((hk, 8, 128), np.float32), np.zeros((hk, 8, 128), np.float32)
        for step in range(3):
            od = orc.decode_step(qd[:, step], ops, bands, t, scale, tk, tv, kd[:, step], vd[:, step], step, 8, per)
            r = fp_report(orc.to_bf16(od), from_bits(g[f"decode_bits_per{per}"][step]))
            assert r["worst_excess"] <= 0 and r["cos"] >= 0.9999 and r["mean_abs"] <= ABS_TOL / 4, (per, step, r)


@pytest.mark.parametrize("name", ["small", "c1"])
def test_decode_partials_match_reference_golden(name):
    """The split partials (m, l, o) that the reference's decode_kernel left behind after the third recorded step at two
    kept tiles per split (pm, pl, po of common_device.cuh:355-370): the restatement's decode_partials gives the same
    triples, so the split pass is pinned on its own and not only through the merged output."""
    path = GOLDEN / f"{name}.npz"
    if not path.is_file():
        pytest.skip(f"{path.name} has not been recorded yet")
    import make_golden
    g = np.load(path)
    hq, hk, t, _, _, _, _ = make_golden.CASES[name]
    q, k, v, bands, qd, _, _ = make_golden.inputs(name)
    scale, per, splits = 1.0 / np.sqrt(128.0), 2, int(g["splits"])
    _, ops = orc.prefill(q, k, v, bands, scale, return_operands=True)
    tables = orc.decode_tables(bands, hk, t)
    parts = orc.decode_partials(qd[:, 2], ops, tables, t, scale,
                                lambda kh, n: [(a, min(n, a + per)) for a in range(0, n, per)])
    pm, pl, po = g["pm"].reshape(hq, splits), g["pl"].reshape(hq, splits), g["po"].reshape(hq, splits, 128)
    for h in range(hq):
        assert len(parts[h]) == splits
        for s, (m, l, o) in enumerate(parts[h]):
            assert abs(m - pm[h, s]) <= 1e-4 * max(1.0, abs(m)), (h, s, m, pm[h, s])
            assert abs(l - pl[h, s]) <= 1e-4 * abs(l), (h, s, l, pl[h, s])
            assert np.abs(o - po[h, s]).max() <= 1e-3 * np.abs(o).max(), (h, s)


def test_reference_accumulator_noise_floor():
    """How reproducible the reference kernel's outputs are at all.  It accumulates every tile's integer P.V sums, biased
    by 12582912, into a float32 register and removes the bias at the end (prefill_sm80.cu:416-449,466-487): near
    2^27 that register resolves 16 units while a tile contributes a few thousand.  Here the restatement evaluates one
    query block twice over the same codes, maxima and float32 scales: once with the reference's float32 accumulation
    and once in float64 without the bias.  The difference is the reference's own rounding noise.  In a V channel
    scaled x20 (a benchmark outlier channel) it exceeds the flat 2e-3 of the parity contract, so no implementation that
    sums the same products can agree with the reference kernel to 2e-3 there; scaled by the channel's range it is
    small, and in ordinary channels it is far below 2e-3.  This is why the full-size GPU comparisons scale the absolute
    bound by range / 8 in wide channels (tests/test_gpu_7_full_size.py)."""
    t, wide = 4096, 93
    mk = lambda seed, dims: orc.synth((1, t, 128), seed, outlier_dims=dims, outlier_scale=20.0)
    q, k, v = mk(1, (5,)), mk(2, (77,)), mk(3, (wide,))
    sl2 = orc.sm_log2(1.0 / np.sqrt(128.0))
    q8, qa, _, _ = orc.quantize_q(q)
    kstat = orc.channel_stats(k)
    k8, ka, _, _ = orc.quantize_k(k, kstat[:, 0])
    vstat = orc.channel_stats(v)
    v16, v8, _ = orc.pack_v(v, vstat)
    qb = t // 64 - 1
    rows = slice(qb * 64, (qb + 1) * 64)
    tf, t8, t4 = orc.band_tiles(qb, orc.INF, orc.INF)
    args = (q8[0, rows], (qa[0, rows] * sl2).astype(np.float32), k8[0], ka[0], v16[0], v8[0], vstat[0], t, qb, tf, t8, t4)
    noise = np.abs(orc.prefill_block(*args) - orc.prefill_block(*args, precise=True))
    span = float(v[0, :, wide].max() - v[0, :, wide].min())
    others = np.delete(noise, wide, axis=1)
    assert span > 100 and noise[:, wide].max() > 2e-3, (span, noise[:, wide].max())        # the flat bound is out of reach
    assert noise[:, wide].max() < 2e-3 * span / 8 / 4                                       # a quarter of the scaled bound
    assert others.max() < 1e-3 and np.sqrt((others ** 2).mean()) < 1e-4                     # ordinary channels: far below
