"""CPU restatement of the reference's quantised-attention arithmetic.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this
module, and only as the checker.  The product (``triattention_b200``) never imports it and has no
CPU fallback.

Parity status: the reference ships no tests, fixtures or golden vectors and has no CPU code path,
so this restatement is pinned against outputs of the reference's own CUDA extension recorded on a
B200 (``tests/golden/*.npz``, produced by ``tests/golden/make_golden.py``) and, in the GPU tests,
against that extension run live on the same inputs.  Where no such fixture covers a function its
docstring says "parity unpinned".

All arithmetic is IEEE float32 (numpy).  The reference is compiled with ``--use_fast_math``
(``triattention/kernels/extension.py:52``): its ``/``, ``1/x`` and ``exp2f`` are hardware
approximations, so scales may differ from this file by a few ulp and codes by one level at rounding
ties.  ``fma32`` emulates a single-rounding fused multiply-add through float64.

Reference files restated here (paths inside the reference project):
  triattention/kernels/cuda/prefill_sm80.cu   :27,78-115 (constants, P rounding, dither, rotation)
                                              :158-257  (QK fragments, masks, scaled row max, margin)
                                              :259-488  (tile lists, passes, online softmax, epilogue)
  triattention/kernels/cuda/common_device.cuh :1-172    (Q/K/V quantise, statistics, packed layouts)
                                              :178-469  (decode tile, partials, merge, BF16 tail)
  triattention/kernels/prefill.py             :10-28,87-108 (band table, CTA order, executor)
  triattention/kernels/decode.py              :17-67    (V format per tile, kept-tile compaction)
"""
from __future__ import annotations

import numpy as np

D, BM, BN = 128, 64, 64
INF = 1 << 20                      # maps.py:8
SKIP, F16, I8, I4, Q4 = 0, 1, 2, 3, 4  # kernels/prefill.py:7
NEAR_V8 = 16                       # kernels/decode.py:9
STAT_BLOCKS = 64                   # common_device.cuh:30
MAGIC_I = 0x4B400000               # prefill_sm80.cu:27
MAGIC_F = np.float32(12582912.0)
LOG2E = 1.4426950408889634
SIGN_WORDS = (0x9A3B5E71, 0x2C6D8F13, 0xE41B7A95, 0x5F02C3D8)  # prefill_sm80.cu:95
ROT_SCALE = np.float32(0.08838834764831845)                     # prefill_sm80.cu:114
C7_127 = np.array([0x3D61C387], dtype=np.uint32).view(np.float32)[0]  # 7.f/127.f folded by nvcc
FLT_MAX = np.float32(np.finfo(np.float32).max)
FLT_MIN = np.float32(np.finfo(np.float32).tiny)
f32 = np.float32


def _signs() -> np.ndarray:
    c = np.arange(D)
    words = np.array(SIGN_WORDS, dtype=np.uint64)
    bit = (words[c >> 5] >> (c & 31).astype(np.uint64)) & np.uint64(1)
    return np.where(bit == 1, -1.0, 1.0).astype(np.float32)


SIGNS = _signs()


def fma32(a, b, c):
    """round32(a*b+c): the product of two float32 is exact in float64; one extra rounding is rare."""
    return (np.asarray(a, np.float64) * np.asarray(b, np.float64) + np.asarray(c, np.float64)).astype(np.float32)


def exp2_32(x):
    with np.errstate(under="ignore", over="ignore"):
        return np.exp2(np.asarray(x, np.float32)).astype(np.float32)


def sm_log2(scale: float) -> np.float32:
    """prefill_sm80.cu:538, common_host.cuh:65: (float)(double(scale)*log2(e))."""
    return np.float32(float(scale) * LOG2E)


# ---------------------------------------------------------------------------------------------
# rotation and quantisation (write path)
# ---------------------------------------------------------------------------------------------
def rotate128(x) -> np.ndarray:
    """prefill_sm80.cu:95-115.  Sign flip, natural-order radix-2 WHT over feature bits 0..6 in that
    order (lower = lo+hi, upper = lo-hi), then one multiply by 1/sqrt(128)."""
    x = np.asarray(x, np.float32) * SIGNS
    shape = x.shape
    for b in range(7):
        y = x.reshape(-1, D >> (b + 1), 2, 1 << b)
        lo, hi = y[:, :, 0, :], y[:, :, 1, :]
        x = np.stack([lo + hi, lo - hi], axis=2).reshape(shape)
    return x * ROT_SCALE


def quantize_q(q):
    """common_device.cuh:1-28.  q [...,T,128] float32 (bf16 values) -> q8, qa, q4 (values -7..7), qa4."""
    x = rotate128(q)
    m = np.abs(x).max(-1, keepdims=True)
    with np.errstate(divide="ignore"):
        inv = np.where(m > 0, f32(127) / m, f32(0)).astype(np.float32)
        inv4 = np.where(m > 0, f32(7) / m, f32(0)).astype(np.float32)
    q8 = np.rint(x * inv).astype(np.int8)
    q4 = np.rint(x * inv4).astype(np.int8)
    return q8, (m / f32(127))[..., 0], q4, (m / f32(7))[..., 0]


def channel_stats(x, identity: bool = False) -> np.ndarray:
    """common_device.cuh:32-56.  x [H,T,128] -> stat [H,3,128] = (mean, scale, 1/scale).
    64 strided partial sums (block b takes tokens b, b+64, ...) added in token order, then the 64
    partials added in block order."""
    x = np.asarray(x, np.float32)
    h, t, _ = x.shape
    stat = np.empty((h, 3, D), np.float32)
    if identity:  # common_host.cuh:39-41
        stat[:, 0], stat[:, 1], stat[:, 2] = 0, 1, 1
        return stat
    rows = (t + STAT_BLOCKS - 1) // STAT_BLOCKS
    pad = rows * STAT_BLOCKS - t
    xs = np.concatenate([x, np.zeros((h, pad, D), np.float32)], 1).reshape(h, rows, STAT_BLOCKS, D)
    xh = np.concatenate([x, np.full((h, pad, D), -FLT_MAX, np.float32)], 1).reshape(h, rows, STAT_BLOCKS, D)
    xl = np.concatenate([x, np.full((h, pad, D), FLT_MAX, np.float32)], 1).reshape(h, rows, STAT_BLOCKS, D)
    psum = np.zeros((h, STAT_BLOCKS, D), np.float32)
    for r in range(rows):
        psum = psum + xs[:, r]
    hi = np.maximum(xh.max(1), -FLT_MAX).max(1)
    lo = np.minimum(xl.min(1), FLT_MAX).min(1)
    total = np.zeros((h, D), np.float32)
    for b in range(STAT_BLOCKS):
        total = total + psum[:, b]
    mean = total / f32(t)
    rng = np.maximum(hi - mean, mean - lo)
    scale = np.where(rng > 0, rng / f32(127), f32(1)).astype(np.float32)
    stat[:, 0], stat[:, 1], stat[:, 2] = mean, scale, f32(1) / scale
    return stat


def quantize_k(k, mean):
    """common_device.cuh:58-131.  k [H,T,128], mean [H,128] ->
    k8 int8 [H,tiles,64,128], ka [H,tiles,4], k4 int8 (-7..7) same shape, ka4.  Rows >= T are zero."""
    k = np.asarray(k, np.float32)
    h, t, _ = k.shape
    tiles = (t + BN - 1) // BN
    y = np.zeros((h, tiles * BN, D), np.float32)
    y[:, :t] = rotate128(k - mean[:, None, :])
    g = y.reshape(h, tiles, 4, 16, D)
    cm = np.abs(g).max((3, 4))
    with np.errstate(divide="ignore"):
        inv = np.where(cm > 0, f32(127) / cm, f32(0)).astype(np.float32)
        inv4 = np.where(cm > 0, f32(7) / cm, f32(0)).astype(np.float32)
    ka = np.where(cm > 0, cm / f32(127), f32(1)).astype(np.float32)
    ka4 = np.where(cm > 0, cm / f32(7), f32(1)).astype(np.float32)
    k8 = np.rint(g * inv[..., None, None]).astype(np.int8).reshape(h, tiles, BN, D)
    k4 = np.rint(g * inv4[..., None, None]).astype(np.int8).reshape(h, tiles, BN, D)
    return k8, ka, k4, ka4


def normalize_v(v, vstat) -> np.ndarray:
    """vnorm, common_device.cuh:132-134.  -> V' float32 [H,tiles*64,128], rows >= T zero."""
    v = np.asarray(v, np.float32)
    h, t, _ = v.shape
    tiles = (t + BN - 1) // BN
    out = np.zeros((h, tiles * BN, D), np.float32)
    out[:, :t] = (v - vstat[:, 0][:, None, :]) * vstat[:, 2][:, None, :]
    return out


def pack_v(v, vstat):
    """common_device.cuh:136-172 (values only).  -> v16 float16, v8 int8, v4 int8 (-7..7), each
    [H,tiles,64,128] indexed [key][channel]."""
    vn = normalize_v(v, vstat)
    h = vn.shape[0]
    v16 = vn.astype(np.float16)
    v8 = np.clip(np.rint(vn), -127, 127).astype(np.int8)
    v4 = np.clip(np.rint(vn * C7_127), -7, 7).astype(np.int8)
    shape = (h, -1, BN, D)
    return v16.reshape(shape), v8.reshape(shape), v4.reshape(shape)


# ---------------------------------------------------------------------------------------------
# the reference extension's packed layouts -> logical [key][feature] arrays (for GPU-side compares)
# ---------------------------------------------------------------------------------------------
def _kic(s, j):
    return 2 * s + np.where(j < 2, j, j + 6)  # key_in_col, prefill_sm80.cu:93


def unpack_ref_k8(kp) -> np.ndarray:
    """uint32 [H,tiles,2048] (common_device.cuh:101-114) -> int8 [H,tiles,64,128]."""
    kp = np.ascontiguousarray(kp).view(np.uint8).reshape(kp.shape[0], kp.shape[1], 8192)
    p = np.arange(8192)
    b, h, i = p % 4, (p // 4) % 2, p // 8
    lane, pair, col, chunk = i % 32, (i // 32) % 2, (i // 64) % 4, i // 256
    row = col * 16 + lane // 4 + pair * 8
    feat = chunk * 32 + (lane % 4) * 4 + h * 16 + b
    out = np.empty(kp.shape[:2] + (BN, D), np.int8)
    out[:, :, row, feat] = kp.view(np.int8)
    return out


def _nibbles(words) -> np.ndarray:
    """uint32 [...,W] -> signed 4-bit values [...,W*8], nibble e of word w at index 8w+e."""
    w = np.ascontiguousarray(words).astype(np.uint32)
    n = (w[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & np.uint32(0xF)
    n = n.astype(np.int8)
    return np.where(n > 7, n - 16, n).astype(np.int8).reshape(w.shape[:-1] + (-1,))


def unpack_ref_k4(k4p) -> np.ndarray:
    """uint32 [H,tiles,1024] (common_device.cuh:117-130) -> int8 [H,tiles,64,128] in -8..7."""
    nib = _nibbles(k4p)
    p = np.arange(8192)
    e, h, i = p % 8, (p // 8) % 2, p // 16
    lane, pair, col, step = i % 32, (i // 32) % 2, (i // 64) % 4, i // 256
    row = col * 16 + lane // 4 + pair * 8
    feat = step * 64 + (lane % 4) * 8 + h * 32 + e
    out = np.empty(nib.shape[:2] + (BN, D), np.int8)
    out[:, :, row, feat] = nib
    return out


def unpack_ref_q4(q4) -> np.ndarray:
    """uint8 [...,T,64] (common_device.cuh:22-25; even feature in the low nibble) -> int8 [...,T,128]."""
    q4 = np.asarray(q4, np.uint8)
    lo, hi = (q4 & 0xF).astype(np.int8), (q4 >> 4).astype(np.int8)
    both = np.stack([lo, hi], -1).reshape(q4.shape[:-1] + (D,))
    return np.where(both > 7, both - 16, both).astype(np.int8)


def unpack_ref_v8(v8p) -> np.ndarray:
    """uint32 [H,tiles,2048] (common_device.cuh:149-159) -> int8 [H,tiles,64 keys,128 channels]."""
    raw = np.ascontiguousarray(v8p).view(np.int8).reshape(v8p.shape[0], v8p.shape[1], 8192)
    p = np.arange(8192)
    b, i = p % 4, p // 4
    word, lane, n8 = i % 4, (i // 4) % 32, i // 128
    key = word * 16 + _kic(lane % 4, b)
    ch = n8 * 8 + lane // 4
    out = np.empty(raw.shape[:2] + (BN, D), np.int8)
    out[:, :, key, ch] = raw
    return out


def unpack_ref_v4(v4p) -> np.ndarray:
    """uint32 [H,tiles,1024] (common_device.cuh:160-171) -> int8 [H,tiles,64,128] in -7..7."""
    nib = _nibbles(v4p)
    p = np.arange(8192)
    j, i = p % 8, p // 8
    h, lane, n8 = i % 2, (i // 2) % 32, i // 64
    key = (2 * h + j % 2) * 16 + _kic(lane % 4, j // 2)
    ch = n8 * 8 + lane // 4
    out = np.empty(nib.shape[:2] + (BN, D), np.int8)
    out[:, :, key, ch] = nib
    return out


def unpack_ref_v16(v16p) -> np.ndarray:
    """uint32 [H,tiles,4096] (common_device.cuh:142-148) -> float16 [H,tiles,64,128]."""
    raw = np.ascontiguousarray(v16p).view(np.float16).reshape(v16p.shape[0], v16p.shape[1], 8192)
    p = np.arange(8192)
    half, i = p % 2, p // 2
    word, lane, col16, key16 = i % 4, (i // 4) % 32, (i // 128) % 8, i // 1024
    key = key16 * 16 + 2 * (lane % 4) + (word % 2) * 8 + half
    ch = col16 * 16 + lane // 4 + (word // 2) * 8
    out = np.empty(raw.shape[:2] + (BN, D), np.float16)
    out[:, :, key, ch] = raw
    return out


# ---------------------------------------------------------------------------------------------
# band table and tile lists
# ---------------------------------------------------------------------------------------------
def band_tiles(qb: int, w8: int, w4: int):
    """prefill_sm80.cu:279-286: (FP16-PV tiles, INT8-QK/INT8-PV tiles, INT4-QK/INT8-PV tiles)."""
    f16 = [0] if qb == 0 else [0, qb]
    lo8 = max(1, qb - w8 + 1)
    lo4 = max(1, qb - w4 + 1)
    n8 = max(0, qb - lo8)
    n4 = max(0, qb - w8 - lo4 + 1)
    return f16, list(range(lo8, lo8 + n8)), list(range(lo4, lo4 + n4))


def cta_order(heads_q: int, heads_kv: int, rows: int) -> np.ndarray:
    """kernels/prefill.py:24-25: (KV head, query block descending, Q head in group)."""
    heads = np.arange(heads_q).reshape(heads_kv, -1)
    qb = np.arange(rows)[::-1]
    return (heads[:, None, :] * rows + qb[None, :, None]).reshape(-1).astype(np.int32)


def band_formats(bands, rows: int):
    """kernels/prefill.py:19-26: which operand formats a band table needs at this length."""
    b = np.asarray(bands, np.int64)
    w8, w4 = b[:, :1], b[:, 1:]
    qb = np.arange(rows)[None, :]
    n8 = np.clip(qb - np.clip(qb - w8 + 1, 1, None), 0, None)
    n4 = np.clip(qb - w8 - np.clip(qb - w4 + 1, 1, None) + 1, 0, None)
    return {F16} | ({I8} if (n8 > 0).any() else set()) | ({Q4} if (n4 > 0).any() else set())


# ---------------------------------------------------------------------------------------------
# prefill attention (band mode)
# ---------------------------------------------------------------------------------------------
def _margin(slope, base):
    """tile_base_margin, prefill_sm80.cu:255-257."""
    return fma32(slope, f32(0.75), np.abs(base).astype(np.float32) * f32(2.4e-7))


def prefill_block(qc, qs, kc, ks, v16, v8, vstat_h, tokens, qb, tiles_f16, tiles_i8, tiles_q4,
                  qc4=None, qs4=None, kc4=None, ks4=None, return_acc=False, tiles_i4=(), v4=None, precise=False):
    """One (Q head, query block): prefill_sm80.cu:259-488.  Band mode gives three tile lists; the task-table mode
    (:287-292, :478-481) gives four, the extra one (tiles_i4, run third) being INT8 scores with 4-bit P codes
    against the INT4 V codes v4.  In every pass only the LAST tile is masked, and only if it is the diagonal one.

    qc int8 [64,128] Q codes of the block (rows >= T zero), qs float32 [64] = qa*sm_log2 (FLT_MIN for
    rows >= T); kc int8 [tiles,64,128], ks [tiles,4]; v16 float16 / v8 int8 [tiles,64,128];
    vstat_h [3,128].  Returns float32 [64,128] before the output cast.

    precise=True keeps every code, maximum and float32 scale exactly as above but carries the running output and
    denominator in float64 without the 12582912 bias on the integer P.V sums (the reference adds float_bits(d) * bq to
    a float32 accumulator and removes the bias at the end, :416-449,466-487): the difference between the two modes
    is the float32 rounding noise of the reference's own accumulation scheme, which bounds how closely any
    implementation that sums the same products can agree with it.
    """
    qbeg = qb * BM
    rows = np.arange(BM)
    acc_t = np.float64 if precise else np.float32
    out = np.zeros((BM, D), acc_t)
    m = np.full(BM, -FLT_MAX, np.float32)
    denom = np.zeros(BM, acc_t)
    corr = np.zeros(BM, np.float32)
    accs = {}
    pv8_done = 0

    def visit(tile, q_codes, q_scale, k_codes, k_scale, pv, last_masked, flush, q4pass):
        nonlocal out, m, denom, corr
        acc = q_codes.astype(np.int32) @ k_codes[tile].astype(np.int32).T  # [64 rows, 64 keys], exact
        if return_acc:
            accs[(tile, 4 if q4pass else 8)] = acc
        keys = tile * BN + np.arange(BN)
        if last_masked:  # :191 — only the diagonal tile is masked
            dead = (keys[None, :] >= tokens) | (keys[None, :] > (qbeg + rows)[:, None]) | ((qbeg + rows)[:, None] >= tokens)
        else:
            dead = np.zeros((BM, BN), bool)
        ksc = k_scale[tile].astype(np.float32)                       # [4]
        accf = acc.astype(np.float32)                               # exact (|acc| < 2^24)
        slope_col = (q_scale[:, None] * ksc[None, :]).astype(np.float32)  # qs*ks[col]
        # scaled_row_max :244-253
        am = np.where(dead, np.int64(-(1 << 40)), acc).reshape(BM, 4, 16).max(2)
        has = am > -(1 << 39)
        cand = np.where(has, slope_col * am.astype(np.float32), -np.inf).astype(np.float32)
        tile_max = cand.max(1)
        n = np.maximum(m, tile_max)
        alpha = exp2_32(m - n)
        m = n
        # the reference folds corr into out when any alpha != 1 in the warp (or on flush); doing it
        # per row whenever alpha != 1 (or on flush) is the same arithmetic up to when the fold happens
        fold = flush | (alpha != 1)
        if precise:
            out = out * alpha.astype(np.float64)[:, None]
        else:
            out = np.where(fold[:, None], fma32(out, alpha[:, None], (-corr * alpha)[:, None]), out)
            corr = np.where(fold, f32(0), corr)
        slope = np.repeat(slope_col, 16, axis=1)                    # [64,64]
        if pv == F16:
            denom = denom * alpha
            if q4pass:
                arg = fma32(slope, accf, -m[:, None])
            else:
                arg = fma32(slope, accf + MAGIC_F, fma32(-slope, MAGIC_F, -m[:, None]))
            p = np.where(dead, f32(0), exp2_32(arg)).astype(np.float16)
            denom = denom + p.astype(acc_t).sum(1, dtype=acc_t)
            out = out + p.astype(acc_t) @ v16[tile].astype(acc_t)
            return
        ks_max = ksc.max()
        base = np.where(tile_max > -np.inf, tile_max, m).astype(np.float32)
        base = base + _margin(q_scale * ks_max, base)
        if pv == I4:   # :392-441 with levels = 15: no bias on the integer sums, restore factor 127/7
            bq = exp2_32(base - m) / f32(15)
            arg = fma32(slope, accf + MAGIC_F, fma32(-slope, MAGIC_F, -base[:, None]))
            e = np.where(dead, f32(0), exp2_32(arg))
            p4 = (np.floor(fma32(e, f32(15), f32(49152.5)).astype(np.float64) - 49152.0).astype(np.int64)) & 0xFF
            d = p4 @ v4[tile].astype(np.int64)
            if precise:
                out = out + d.astype(np.float64) * (bq * (f32(127) / f32(7))).astype(np.float64)[:, None]
                denom = denom * alpha.astype(np.float64) + p4.sum(1).astype(np.float64) * bq.astype(np.float64)
                return
            out = fma32(d.astype(np.float32), (bq * (f32(127) / f32(7))).astype(np.float32)[:, None], out)
            denom = fma32(p4.sum(1).astype(np.float32), bq, denom * alpha)
            return
        bq = exp2_32(base - m) / f32(255)
        if q4pass:
            arg = fma32(slope, accf, -base[:, None])
        else:
            arg = fma32(slope, accf + MAGIC_F, fma32(-slope, MAGIC_F, -base[:, None]))
        e = np.where(dead, f32(0), exp2_32(arg))
        w = fma32(e, f32(255), f32(49152.5))
        p8 = (np.floor(w.astype(np.float64) - 49152.0).astype(np.int64)) & 0xFF
        d = p8 @ v8[tile].astype(np.int64)                           # [64,128] exact
        if precise:
            out = out + d.astype(np.float64) * bq.astype(np.float64)[:, None]
            denom = denom * alpha.astype(np.float64) + p8.sum(1).astype(np.float64) * bq.astype(np.float64)
            return
        out = fma32((d + 12582912).astype(np.float32), bq[:, None], out)
        corr = fma32(MAGIC_F, bq, corr)
        denom = fma32(p8.sum(1).astype(np.float32), bq, denom * alpha)

    none = np.zeros(BM, bool)
    for i, t in enumerate(tiles_f16):
        visit(t, qc, qs, kc, ks, F16, t == qb and i == len(tiles_f16) - 1, none, False)
    for i, t in enumerate(tiles_i8):
        last = i == len(tiles_i8) - 1
        flush = (not last) and (pv8_done + i) % 16 == 15
        visit(t, qc, qs, kc, ks, I8, t == qb and last, np.full(BM, flush), False)
    pv8_done += len(tiles_i8)
    for i, t in enumerate(tiles_i4):
        visit(t, qc, qs, kc, ks, I4, t == qb and i == len(tiles_i4) - 1, none, False)
    for i, t in enumerate(tiles_q4):
        last = i == len(tiles_q4) - 1
        flush = (not last) and (pv8_done + i) % 16 == 15
        visit(t, qc4, qs4, kc4, ks4, I8, t == qb and last, np.full(BM, flush), True)
    if precise:
        with np.errstate(divide="ignore", invalid="ignore"):
            res = np.where(denom[:, None] > 0, out / denom[:, None], 0.0) * vstat_h[1][None, :].astype(np.float64) + vstat_h[0][None, :]
        return (res.astype(np.float32), accs) if return_acc else res.astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(denom > 0, f32(1) / denom, f32(0)).astype(np.float32)
    res = fma32((out - corr[:, None]) * inv[:, None], vstat_h[1][None, :], vstat_h[0][None, :])
    return (res, accs) if return_acc else res


def prefill(q, k, v, bands, scale, return_operands=False):
    """One sequence: kernels/prefill.py:87-108 over common_host.cuh:1-45 and prefill_sm80.cu:510-543.
    q [Hq,T,128], k/v [Hkv,T,128] float32 holding bf16 values; bands [Hq,2].
    Returns float32 [Hq,T,128] (before the bf16 cast) and, optionally, the operand dict."""
    q, k, v = (np.asarray(x, np.float32) for x in (q, k, v))
    hq, t, _ = q.shape
    hk = k.shape[0]
    g = hq // hk
    rows = (t + BM - 1) // BM
    sl2 = sm_log2(scale)
    q8, qa, q4, qa4 = quantize_q(q)
    kstat = channel_stats(k)
    k8, ka, k4, ka4 = quantize_k(k, kstat[:, 0])
    fm = band_formats(bands, rows)
    vstat = channel_stats(v, identity=(I8 not in fm and Q4 not in fm))
    v16, v8, v4 = pack_v(v, vstat)
    out = np.zeros((hq, rows * BM, D), np.float32)
    pad = rows * BM - t
    q8p = np.concatenate([q8, np.zeros((hq, pad, D), np.int8)], 1)
    q4p = np.concatenate([q4, np.zeros((hq, pad, D), np.int8)], 1)
    qsp = np.concatenate([qa * sl2, np.full((hq, pad), FLT_MIN, np.float32)], 1).astype(np.float32)
    qs4p = np.concatenate([qa4 * sl2, np.full((hq, pad), FLT_MIN, np.float32)], 1).astype(np.float32)
    for h in range(hq):
        kh = h // g
        w8, w4 = int(bands[h][0]), int(bands[h][1])
        for qb in range(rows):
            tf, t8, t4 = band_tiles(qb, w8, w4)
            sl = slice(qb * BM, (qb + 1) * BM)
            out[h, sl] = prefill_block(q8p[h, sl], qsp[h, sl], k8[kh], ka[kh], v16[kh], v8[kh], vstat[kh], t, qb,
                                       tf, t8, t4, q4p[h, sl], qs4p[h, sl], k4[kh], ka4[kh])
    res = out[:, :t]
    if return_operands:
        return res, dict(q8=q8, qa=qa, q4=q4, qa4=qa4, kstat=kstat, k8=k8, ka=ka, k4=k4, ka4=ka4, vstat=vstat,
                         v16=v16, v8=v8, v4=v4)
    return res


def exact_attention(q, k, v, scale):
    """models.py:45-47 (torch SDPA, causal, GQA) restated in float32 for the BF16-head extension.
    parity unpinned: the reference only calls the library kernel."""
    q, k, v = (np.asarray(x, np.float32) for x in (q, k, v))
    hq, t, _ = q.shape
    g = hq // k.shape[0]
    out = np.empty_like(q)
    mask = np.triu(np.ones((t, t), bool), 1)
    for h in range(hq):
        s = (q[h] @ k[h // g].T) * f32(scale)
        s = np.where(mask, -np.inf, s)
        p = np.exp(s - s.max(1, keepdims=True))
        out[h] = (p / p.sum(1, keepdims=True)) @ v[h // g]
    return out


# ---------------------------------------------------------------------------------------------
# decode cache tables and decode step
# ---------------------------------------------------------------------------------------------
def decode_v_codes(tiles: int) -> np.ndarray:
    """kernels/decode.py:17-22: V format per prompt tile for decode (I8 for tile 0 and the last 16)."""
    j = np.arange(tiles)
    return np.where((tiles - 1 - j < NEAR_V8) | (j == 0), I8, I4)


def decode_tables(bands, heads_kv: int, prompt: int):
    """kernels/decode.py:24-45: per KV head the kept tiles (ascending), their K state (8 or 4) and the
    row mask of Q heads that attend to them.  Returns a list (one per KV head) of dicts."""
    b = np.asarray(bands, np.int64)
    tiles = (prompt + BN - 1) // BN
    j = np.arange(tiles)
    w8, w4, d = b[:, :1], b[:, 1:], (tiles - 1) - j[None, :]
    state = np.where((j[None, :] == 0) | (d < w8), 8, np.where(d < w4, 4, 0))
    state = state.reshape(heads_kv, -1, tiles)
    kv = state.max(1)
    rowmask = ((state > 0).astype(np.int64) << np.arange(state.shape[1])[None, :, None]).sum(1)
    vfmt = decode_v_codes(tiles)
    res = []
    for kh in range(heads_kv):
        kept = np.nonzero(kv[kh] > 0)[0]
        res.append(dict(tiles=kept, state=kv[kh][kept], rowmask=rowmask[kh][kept] & 0xFF, vfmt=vfmt[kept]))
    return res


def _decode_tile(qcodes, qscale, kcodes, kt, vcodes, pv, kq, key_begin, prompt, rowmask, st):
    """decode_tile, common_device.cuh:178-273, for the g live rows of one KV head."""
    g = qcodes.shape[0]
    acc = qcodes.astype(np.int64) @ kcodes.astype(np.int64).T          # [g,64]
    keys = key_begin + np.arange(BN)
    row_on = ((rowmask >> np.arange(g)) & 1).astype(bool)
    live = row_on[:, None] & (keys[None, :] < prompt)
    accf = acc.astype(np.float32)
    slope0 = (qscale[:, None] * kt[None, :]).astype(np.float32)        # [g,4] per warp/col
    slope1 = (qscale * kt.max()).astype(np.float32)
    am = np.where(live, acc, -(1 << 40)).reshape(g, 4, 16).max(2)
    has = am > -(1 << 39)
    rowmax = np.where(has, slope0 * am.astype(np.float32), -np.inf).astype(np.float32)
    tile = rowmax.max(1)
    n = np.maximum(st["m"], tile)
    alpha = exp2_32(st["m"] - n)
    st["m"] = n
    st["out"] = st["out"] * alpha[:, None]
    st["corr"] = st["corr"] * alpha
    levels = f32(255) if pv == I8 else f32(15)
    anyk = tile > -np.inf
    base = np.where(anyk, tile, n).astype(np.float32)
    base = base + _margin(slope1, base)
    bq = np.where(anyk, exp2_32(base - n) / levels, f32(0)).astype(np.float32)
    restore = bq if pv == I8 else (bq * (f32(127) / f32(7))).astype(np.float32)
    slope = np.repeat(slope0, 16, axis=1)
    if kq == 8:
        # nvcc contracts bias-base = (-slope*Magic)-base into one fma (common_device.cuh:225,243)
        arg = fma32(slope, accf + MAGIC_F, fma32(-slope, MAGIC_F, -base[:, None]))
    else:
        arg = fma32(slope, accf, -base[:, None])
    e = np.where(live, exp2_32(arg), f32(0))
    dither = (f32(49152.0) + (acc & 0xFF).astype(np.float32) / f32(256)).astype(np.float32)
    dither = np.where(live, dither, f32(49152.0))
    w = fma32(e, levels, dither)
    p = np.floor(w.astype(np.float64) - 49152.0).astype(np.int64) & 0xFF
    # per-warp denominators: lane sub holds keys {2s,2s+1,8+2s,9+2s} of the warp's 16 (:213-216,248-251)
    pw = p.reshape(g, 4, 2, 4, 2)                                       # [g, warp, half, sub, parity]
    lane = pw.sum((2, 4)).astype(np.float32) * bq[:, None, None]        # [g, warp, sub]
    part = (lane[..., 0] + lane[..., 1]) + (lane[..., 2] + lane[..., 3])
    st["denom"] = fma32(st["denom"], alpha[:, None], part)
    d = p @ vcodes.astype(np.int64)                                     # [g,128]
    if pv == I8:
        st["corr"] = fma32(MAGIC_F, restore, st["corr"])
        st["out"] = fma32((d + 12582912).astype(np.float32), restore[:, None], st["out"])
    else:
        st["out"] = fma32(d.astype(np.float32), restore[:, None], st["out"])


def decode_quantize_q(q, sl2):
    """decode_kernel prologue, common_device.cuh:291-315: codes and qscale = qa*sm_log2 (FLT_MIN if 0)."""
    q8, qa, q4, qa4 = quantize_q(q)
    live = qa > 0
    qs = np.where(live, qa * sl2, FLT_MIN).astype(np.float32)
    qs4 = np.where(live, qa4 * sl2, FLT_MIN).astype(np.float32)
    return q8, qs, q4, qs4


def fold_tail(ops, tail_k, tail_v):
    """Not in the reference (its tail of generated tokens is capped, common_host.cuh:56): 64 tail rows become one
    more cached tile, quantised with the prompt's statistics by the prompt's own rules (common_device.cuh:58-172).
    tail_k, tail_v [Hkv,64,128] -> dict(k8 [Hkv,64,128], ka [Hkv,4], v8 [Hkv,64,128]).  parity unpinned."""
    k8, ka, _, _ = quantize_k(tail_k, ops["kstat"][:, 0])
    _, v8, _ = pack_v(tail_v, ops["vstat"])
    return dict(k8=k8[:, 0], ka=ka[:, 0], v8=v8[:, 0])


def decode_partials(q, ops, tables, prompt, scale, splits_of, appended=()):
    """decode_kernel, common_device.cuh:275-371.  q [Hq,128]; ops = logical operand dict from
    ``prefill(..., return_operands=True)``; tables from ``decode_tables``; ``splits_of(kh, n)`` returns
    the list of (first, last) index ranges over that head's kept tiles.  Returns per Q head a list of
    (m, l, o[128]) partials in split order.  appended = tiles from ``fold_tail`` in order: they follow the
    head's kept tiles, INT8 K and V, every Q head of the group attends, all 64 keys live."""
    hq = q.shape[0]
    hk = len(tables)
    g = hq // hk
    sl2 = sm_log2(scale)
    q8, qs, q4, qs4 = decode_quantize_q(np.asarray(q, np.float32), sl2)
    parts = [[] for _ in range(hq)]
    for kh in range(hk):
        tb = tables[kh]
        rows = slice(kh * g, (kh + 1) * g)
        kept = len(tb["tiles"])
        for first, last in splits_of(kh, kept + len(appended)):
            st = dict(m=np.full(g, -FLT_MAX, np.float32), denom=np.zeros((g, 4), np.float32),
                      out=np.zeros((g, D), np.float32), corr=np.zeros(g, np.float32))
            for i in range(first, last):
                if i >= kept:
                    extra = appended[i - kept]
                    _decode_tile(q8[rows], qs[rows], extra["k8"][kh], extra["ka"][kh], extra["v8"][kh], I8, 8,
                                 0, 1 << 30, 0xFF, st)
                    continue
                tile, state, pv = int(tb["tiles"][i]), int(tb["state"][i]), int(tb["vfmt"][i])
                vcodes = ops["v8"][kh, tile] if pv == I8 else ops["v4"][kh, tile]
                if state == 4:
                    _decode_tile(q4[rows], qs4[rows], ops["k4"][kh, tile], ops["ka4"][kh, tile], vcodes, pv, 4,
                                 tile * BN, prompt, int(tb["rowmask"][i]), st)
                else:
                    _decode_tile(q8[rows], qs[rows], ops["k8"][kh, tile], ops["ka"][kh, tile], vcodes, pv, 8,
                                 tile * BN, prompt, int(tb["rowmask"][i]), st)
            pl = ((st["denom"][:, 0] + st["denom"][:, 1]) + st["denom"][:, 2]) + st["denom"][:, 3]
            po = st["out"] - st["corr"][:, None]
            for r in range(g):
                parts[kh * g + r].append((st["m"][r], pl[r], po[r]))
    return parts


def decode_merge(q, parts, kmean, vstat, tail_k, tail_v, kcur, vcur, step, max_tail, scale):
    """decode_merge_kernel, common_device.cuh:373-469.  tail_k/tail_v [Hkv,max_tail,128] are updated in
    place (the current token is appended at min(step, max_tail-1)).  Returns float32 [Hq,128]."""
    q = np.asarray(q, np.float32)
    hq, hk = q.shape[0], kmean.shape[0]
    g = hq // hk
    sl2 = sm_log2(scale)
    prior = min(int(step), max_tail - 1)
    tail_k[:, prior] = kcur
    tail_v[:, prior] = vcur
    out = np.empty((hq, D), np.float32)
    for h in range(hq):
        kh = h // g
        kt = tail_k[kh, :prior + 1].astype(np.float32) - kmean[kh][None, :]
        ts = ((kt * q[h][None, :]).sum(1, dtype=np.float32) * sl2).astype(np.float32)
        pm = np.array([p[0] for p in parts[h]], np.float32)
        pl = np.array([p[1] for p in parts[h]], np.float32)
        po = np.stack([p[2] for p in parts[h]]) if parts[h] else np.zeros((0, D), np.float32)
        big = max(float(pm.max()) if len(pm) else -np.inf, float(ts.max()), float(-FLT_MAX))
        big = f32(big)
        w = exp2_32(pm - big)
        total = (pl * w).sum(dtype=np.float32)
        acc = (po * w[:, None]).sum(0, dtype=np.float32)
        acc = acc * vstat[kh, 1] + total * vstat[kh, 0]
        e = exp2_32(ts - big)
        total = total + e.sum(dtype=np.float32)
        acc = acc + (e[:, None] * tail_v[kh, :prior + 1].astype(np.float32)).sum(0, dtype=np.float32)
        out[h] = acc / total
    return out


def decode_step(q, ops, bands, prompt, scale, tail_k, tail_v, kcur, vcur, step, max_tail, per=None, appended=()):
    """One decode step of one sequence (kernels/decode.py:69-80).  ``per`` = kept tiles per split
    (kernels/decode.py:54-55); None = one split per head."""
    hk = ops["kstat"].shape[0]
    tables = decode_tables(bands, hk, prompt)

    def splits_of(kh, n):
        step_ = n if per is None else per
        return [(a, min(n, a + step_)) for a in range(0, max(n, 1), max(step_, 1)) if a < n] or []

    parts = decode_partials(q, ops, tables, prompt, scale, splits_of, appended)
    return decode_merge(q, parts, ops["kstat"][:, 0], ops["vstat"], tail_k, tail_v, kcur, vcur, step, max_tail, scale)


def exact_decode(q, k_all, v_all, scale):
    """BF16-head extension in decode: softmax(q k^T scale) v over prompt + tail keys, float32.
    parity unpinned (no counterpart in the reference's kernels)."""
    q, k_all, v_all = (np.asarray(x, np.float32) for x in (q, k_all, v_all))
    s = (k_all @ q) * f32(scale)
    p = np.exp(s - s.max())
    return (p[:, None] * v_all).sum(0) / p.sum()


# ---------------------------------------------------------------------------------------------
# synthetic inputs shared by tests, golden generation and the bench
# ---------------------------------------------------------------------------------------------
def synth(shape, seed, outlier_dims=None, outlier_scale=16.0, outlier_fraction=None):
    """N(0,1) tensor [H,T,128] rounded to bf16 values (returned as float32).  Either fixed outlier
    feature indices per head, or a seeded fraction of the H*128 channels, scaled for all tokens."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape, dtype=np.float32)
    h = shape[0]
    if outlier_dims is not None:
        x[..., list(outlier_dims)] *= f32(outlier_scale)
    if outlier_fraction:
        n = int(round(outlier_fraction * h * D))
        pick = rng.permutation(h * D)[:n]
        x.reshape(h, -1, D)[pick // D, :, pick % D] *= f32(outlier_scale)
    return to_bf16(x)


def to_bf16(x) -> np.ndarray:
    """Round float32 to the nearest bf16 value (ties to even), keeping float32 storage."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)
