"""Loader and thin Python shim over the sm_100a C-ABI library.

Mirrors ``triattention/kernels/extension.py:28-54`` (``load_extension()`` returns an object with
``prepare_qk``, ``pack_v``, ``attention``, ``decode`` and ``decode_occupancy``), but the library is built
ahead of time for sm_100a only (``python -m triattention_b200.build``) and bound with ctypes: no JIT, no
architecture dispatch, no CPU fallback.  A missing library or a missing GPU is an error, raised as
``RuntimeError`` like the reference does (``extension.py:15-19``).
"""
from __future__ import annotations

import ctypes
import functools
from pathlib import Path

import torch

LIBRARY = Path(__file__).resolve().parent.parent / "libtriattn_sm100a.so"

_P, _I, _L, _D, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_double, ctypes.c_uint32

# name -> argtypes, in the order of include/triattention_b200.h
SIGNATURES = {
    "tri_prepare_qk": [_P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "tri_pack_v": [_P, _I, _I, _I, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P],
    "tri_write_kv": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                     _P, _P, _P, _P, _P, _P, _P, _P],
    "tri_requantize_kv": [_P, _P, _I, _I, _I, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P],
    "tri_attention": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _I, _I, _I, _I, _D,
                      _P, _L, _L, _L, _P, _L, _L, _L, _P, _P],
    "tri_attention_sweep": [_P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _I, _I, _I, _I, _D, _P, _P],
    "tri_attention_tasks": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _I, _I, _I, _I, _D, _P, _P],
    "tri_cache_store": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P],
    "tri_cache_store_bf16": [_P, _P, _P, _I, _P, _P, _I, _I, _L, _L, _L, _L, _L, _L, _I, _I, _P],
    "tri_decode": [_P, _L, _L, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _L, _L, _P, _P, _L, _L, _P, _P, _L, _L,
                   _P, _P, _P, _P, _I, _I, _I, _I, _I, _D, _I, _P, _P],
    "tri_decode_static": [_P, _L, _L, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _L, _L, _P, _P, _L, _L, _P, _P,
                          _L, _L, _I, _I, _I, _I, _I, _D, _P, _P],
    "tri_decode_fold": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "tri_decode_partials": [_P, _L, _L, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P,
                            _I, _I, _I, _I, _D, _P, _P],
    "tri_decode_split": [_P, _L, _L, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _L, _L, _P, _P, _L, _L, _P, _P, _L, _L,
                         _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _D, _P, _P],
    "tri_decode_merge": [_P, _L, _L, _P, _P, _P, _L, _P, _P, _P, _I, _P, _I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _L, _L, _P, _P,
                         _L, _L, _P, _P, _L, _L, _I, _I, _I, _I, _D, _P, _P],
    "tri_gather_wait": [_P, _L, _P, _I, _P, _P],
    "tri_decode_occupancy": [],
    "tri_decode_tail_hint": [_I],
    "tri_qk_accumulators": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "tri_abi_version": [],
}


ABI_VERSION = 5         # tri_abi_version() of the library these signatures describe
LONG_TAIL_ROWS = 8      # tri_decode_tail_hint: above this many rows (or without a hint) the unrolled merge kernel runs


def load_library() -> ctypes.CDLL:
    """dlopen the library and declare every entry point (no GPU needed for this)."""
    if not LIBRARY.is_file():
        raise RuntimeError(f"{LIBRARY.name} is missing: build it with `python -m triattention_b200.build` "
                           "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(LIBRARY))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, ctypes.c_int
    lib.tri_last_error.argtypes, lib.tri_last_error.restype = [], ctypes.c_char_p
    if lib.tri_abi_version() != ABI_VERSION:     # a library built from older sources takes other arguments
        raise RuntimeError(f"{LIBRARY.name} has ABI version {lib.tri_abi_version()}, this package wants {ABI_VERSION}: "
                           "rebuild it with `python -m triattention_b200.build`")
    return lib


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Module:
    """The five reference method names (batched), plus the cache-store and parity helpers."""

    def __init__(self, lib):
        self.lib = lib
        self._errors = {}

    # -- plumbing ------------------------------------------------------------------------------
    def _check(self, status):
        if status < 0:
            raise RuntimeError(self.lib.tri_last_error().decode())
        return status

    @staticmethod
    def _device_index(device):
        """Index of a CUDA device given as torch.device / str / int; "cuda" means the current device."""
        d = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        return torch.cuda.current_device() if d.index is None else d.index

    def error_word(self, device):
        """The int32 word on `device` that kernels with bounded waits write their error code to (one per GPU)."""
        key = self._device_index(device)
        if key not in self._errors:
            self._errors[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        return self._errors[key]

    def check_device_error(self, device=None):
        """Synchronise and raise if a kernel reported an error (a bounded wait that ran out, a bad table entry).
        device=None checks the word of every GPU this process has launched on."""
        keys = sorted(self._errors) if device is None else [self._device_index(device)]
        for key in keys:
            if key not in self._errors:
                continue
            word = int(self._errors[key].item())
            if word:
                self._errors[key].zero_()
                where = f", wait site {(word >> 8) & 0xff} at step {word >> 16} of the prefill kernel" if word >> 8 else ""
                raise RuntimeError(f"TriAttention kernel reported device error {word & 0xff} on cuda:{key}{where} (1 = "
                                   "barrier wait ran out, 3 = tile number outside the prompt in a task table, 4 = partial "
                                   "slot outside the buffer)")

    @staticmethod
    def _bhtd(x, name):
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[3] == 128 and x.stride(3) == 1):
            raise RuntimeError(f"BF16 {name} [B,H,T,128] with contiguous features")
        return x

    # -- reference surface ---------------------------------------------------------------------
    def prepare_qk(self, q, k, q8, qa, k8, ka, partial, kstat, q4x=None, qa4=None, k4x=None, ka4=None, k4=None,
                   q_modes=None):
        self._bhtd(q, "Q"), self._bhtd(k, "K")
        b, hq, t, _ = q.shape
        hk, tiles = k.shape[1], (t + 63) // 64
        if k.shape[0] != b or k.shape[2] != t or hq % hk:
            raise RuntimeError("BF16 Q/K [B,H,T,128] with contiguous features")
        if not (q8.numel() == b * hq * t * 128 and qa.numel() == b * hq * t and k8.numel() == b * hk * tiles * 8192 and
                ka.numel() == b * hk * tiles * 4 and partial.numel() >= b * hk * 64 * 3 * 128 and
                kstat.numel() == b * hk * 3 * 128):
            raise RuntimeError("Q/K buffers")
        int4 = q4x is not None
        if not (int4 == (qa4 is not None) == (k4x is not None) == (ka4 is not None)) or (k4 is not None and not int4):
            raise RuntimeError("INT4 Q/K buffers (all or none)")
        if q_modes is not None and not (q_modes.is_cuda and q_modes.dtype == torch.int32 and q_modes.numel() == hq
                                        and q_modes.is_contiguous()):
            raise RuntimeError("q_modes int32 [Hq] on the device")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_prepare_qk(q.data_ptr(), k.data_ptr(), b, hq, hk, t, q.stride(0), q.stride(1),
                                                q.stride(2), k.stride(0), k.stride(1), k.stride(2), q8.data_ptr(),
                                                qa.data_ptr(), k8.data_ptr(), ka.data_ptr(), partial.data_ptr(),
                                                kstat.data_ptr(), _ptr(q4x), _ptr(qa4), _ptr(k4x), _ptr(k4), _ptr(ka4),
                                                _ptr(q_modes), _stream()))

    def write_kv(self, q, k, v, q8, qa, k8, ka, partial_k, kstat, partial_v, vstat, q4x=None, qa4=None, k4x=None, ka4=None,
                 k4=None, q_modes=None, v16=None, v8=None, v4=None, v8h=None, raw_heads=None):
        """prepare_qk and pack_v in one call whose Q, K and V chains run side by side (tri_write_kv); same results."""
        self._bhtd(q, "Q"), self._bhtd(k, "K"), self._bhtd(v, "V")
        b, hq, t, _ = q.shape
        hk, tiles = k.shape[1], (t + 63) // 64
        if k.shape[0] != b or k.shape[2] != t or hq % hk or tuple(v.shape) != tuple(k.shape):
            raise RuntimeError("BF16 Q/K/V [B,H,T,128] with contiguous features")
        if not (q8.numel() == b * hq * t * 128 and qa.numel() == b * hq * t and k8.numel() == b * hk * tiles * 8192 and
                ka.numel() == b * hk * tiles * 4 and partial_k.numel() >= b * hk * 64 * 3 * 128 and
                partial_v.numel() >= b * hk * 64 * 3 * 128 and kstat.numel() == b * hk * 3 * 128 and
                vstat.numel() == b * hk * 3 * 128 and partial_k.data_ptr() != partial_v.data_ptr()):
            raise RuntimeError("Q/K/V buffers")
        int4 = q4x is not None
        if not (int4 == (qa4 is not None) == (k4x is not None) == (ka4 is not None)) or (k4 is not None and not int4):
            raise RuntimeError("INT4 Q/K buffers (all or none)")
        for name, buf, size in (("v16", v16, 16384), ("v8", v8, 8192), ("v4", v4, 4096), ("v8h", v8h, 16384)):
            if buf is not None and buf.numel() * buf.element_size() != b * hk * tiles * size:
                raise RuntimeError(f"{name} buffer")
        for name, tab, n in (("q_modes", q_modes, hq), ("raw_heads", raw_heads, hk)):
            if tab is not None and not (tab.is_cuda and tab.dtype == torch.int32 and tab.numel() == n and tab.is_contiguous()):
                raise RuntimeError(f"{name} int32 [{n}] on the device")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_write_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), b, hq, hk, t, q.stride(0), q.stride(1),
                                              q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                              v.stride(2), q8.data_ptr(), qa.data_ptr(), k8.data_ptr(), ka.data_ptr(),
                                              partial_k.data_ptr(), kstat.data_ptr(), _ptr(q4x), _ptr(qa4), _ptr(k4x), _ptr(k4),
                                              _ptr(ka4), _ptr(q_modes), partial_v.data_ptr(), vstat.data_ptr(), _ptr(v16),
                                              _ptr(v8), _ptr(v4), _ptr(v8h), _ptr(raw_heads), _stream()))

    def pack_v(self, v, partial, vstat, v16=None, v8=None, v4=None, v8h=None, raw_heads=None):
        """raw_heads int32 [Hkv] on the device (or None): non-zero = un-quantised KV head (identity statistics, fp16 blob
        of V itself only)."""
        self._bhtd(v, "V")
        if raw_heads is not None and not (raw_heads.is_cuda and raw_heads.dtype == torch.int32 and
                                          raw_heads.numel() == v.shape[1] and raw_heads.is_contiguous()):
            raise RuntimeError("raw_heads int32 [Hkv] on the device")
        b, hk, t, _ = v.shape
        tiles = (t + 63) // 64
        for buf, size in ((v16, 16384), (v8, 8192), (v4, 4096), (v8h, 16384)):
            if buf is not None and buf.numel() * buf.element_size() != b * hk * tiles * size:
                raise RuntimeError("packed V size")
        if partial.numel() < b * hk * 64 * 3 * 128 or vstat.numel() != b * hk * 3 * 128:
            raise RuntimeError("V statistics buffers")
        with torch.cuda.device(v.device):
            self._check(self.lib.tri_pack_v(v.data_ptr(), b, hk, t, v.stride(0), v.stride(1), v.stride(2),
                                            partial.data_ptr(), vstat.data_ptr(), _ptr(v16), _ptr(v8), _ptr(v4), _ptr(v8h),
                                            _ptr(raw_heads), _stream()))

    def requantize_kv(self, k, v, kstat, vstat, k8, ka, v8):
        """K8 / V8 blobs of rows that came after the prompt, with the prompt's statistics."""
        self._bhtd(k, "K"), self._bhtd(v, "V")
        b, hk, t, _ = k.shape
        tiles = (t + 63) // 64
        if v.shape != k.shape or k8.numel() != b * hk * tiles * 8192 or v8.numel() != b * hk * tiles * 8192 or \
                ka.numel() != b * hk * tiles * 4 or kstat.numel() != b * hk * 384 or vstat.numel() != b * hk * 384:
            raise RuntimeError("requantize_kv buffers")
        with torch.cuda.device(k.device):
            self._check(self.lib.tri_requantize_kv(k.data_ptr(), v.data_ptr(), b, hk, t, k.stride(0), k.stride(1), k.stride(2),
                                                   v.stride(0), v.stride(1), v.stride(2), kstat.data_ptr(), vstat.data_ptr(),
                                                   k8.data_ptr(), ka.data_ptr(), v8.data_ptr(), _stream()))

    def attention(self, bands, v16, v8h, vstat, q8, k8, qa8, ka8, q4x, k4x, qa4, ka4, out, scale, heads_kv, q_raw=None,
                  k_raw=None):
        """q_raw / k_raw: the caller's bf16 Q [B,Hq,T,128] and K [B,Hkv,T,128] when the map has un-quantised heads (bands
        rows of zeros); those heads are then computed as exact attention from these rows and their fp16 V blobs."""
        if not (out.dim() == 4 and out.stride(3) == 1 and out.dtype in (torch.bfloat16, torch.float16)):
            raise RuntimeError("output [B,Hq,T,128] aligned")
        b, hq, t, _ = out.shape
        if (q_raw is None) != (k_raw is None):
            raise RuntimeError("raw Q and K rows of un-quantised heads (both or none)")
        raw = (0, 0, 0, 0, 0, 0, 0, 0)
        if q_raw is not None:
            self._bhtd(q_raw, "Q"), self._bhtd(k_raw, "K")
            if q_raw.shape != (b, hq, t, 128) or k_raw.shape != (b, heads_kv, t, 128):
                raise RuntimeError("BF16 Q/K [B,H,T,128] with contiguous features")
            raw = (q_raw.data_ptr(), q_raw.stride(0), q_raw.stride(1), q_raw.stride(2),
                   k_raw.data_ptr(), k_raw.stride(0), k_raw.stride(1), k_raw.stride(2))
        if bands.dtype != torch.int32 or bands.numel() != hq * 2 or not bands.is_contiguous():
            raise RuntimeError("bands [Hq,2] or task tables")
        with torch.cuda.device(out.device):
            self._check(self.lib.tri_attention(bands.data_ptr(), _ptr(v16), _ptr(v8h), vstat.data_ptr(), q8.data_ptr(),
                                               k8.data_ptr(), qa8.data_ptr(), ka8.data_ptr(), _ptr(q4x), _ptr(k4x),
                                               _ptr(qa4), _ptr(ka4), out.data_ptr(), int(out.dtype == torch.float16),
                                               out.stride(0), out.stride(1), out.stride(2), b, hq, heads_kv, t,
                                               float(scale), *raw, self.error_word(out.device).data_ptr(), _stream()))
        return out

    def attention_sweep(self, bands, first_block, v16, v8h, vstat, q8, k8, qa8, ka8, q4x, k4x, qa4, ka4, out, row0, scale, heads_kv,
                        tokens):
        """bands int32 [C,Hq,2] on the device; out [C,B,Hq,R,128] holds query rows row0 .. row0+R-1 (row0 = the first row of
        the four-block group that contains first_block); one launch evaluates every configuration on the same operands."""
        if not (out.dim() == 5 and out.stride(4) == 1 and out.dtype in (torch.bfloat16, torch.float16)):
            raise RuntimeError("output [C,B,Hq,R,128] aligned")
        c, b, hq, r, _ = out.shape
        if bands.dtype != torch.int32 or tuple(bands.shape) != (c, hq, 2) or not bands.is_contiguous():
            raise RuntimeError("bands [C,Hq,2]")
        if row0 != (first_block // 4) * 256 or row0 + r != tokens:
            raise RuntimeError("the output holds the rows from the first computed group of query blocks to the end")
        origin = out.data_ptr() - row0 * out.stride(3) * out.element_size()     # where row 0 would lie
        with torch.cuda.device(out.device):
            self._check(self.lib.tri_attention_sweep(bands.data_ptr(), c, int(first_block), _ptr(v16), _ptr(v8h), vstat.data_ptr(),
                                                     q8.data_ptr(), k8.data_ptr(), qa8.data_ptr(), ka8.data_ptr(), _ptr(q4x),
                                                     _ptr(k4x), _ptr(qa4), _ptr(ka4), origin, int(out.dtype == torch.float16),
                                                     out.stride(0), out.stride(1), out.stride(2), out.stride(3), b, hq, heads_kv,
                                                     int(tokens), float(scale), self.error_word(out.device).data_ptr(), _stream()))
        return out

    def attention_tasks(self, groups, entries, v16, v8, v4, vstat, q8, k8, qa8, ka8, q4x, k4x, qa4, ka4, out, scale, heads_kv):
        """Task-table mode (the reference's attention(order, None, groups, entries, ...)): four explicit tile lists per
        (Q head, query block).  groups / entries int32 on the device."""
        if not (out.dim() == 4 and out.stride(3) == 1 and out.dtype in (torch.bfloat16, torch.float16)):
            raise RuntimeError("output [B,Hq,T,128] aligned")
        b, hq, t, _ = out.shape
        rows = (t + 63) // 64
        if groups.dtype != torch.int32 or entries.dtype != torch.int32 or groups.numel() != hq * rows * 4 + 1:
            raise RuntimeError("bands [Hq,2] or task tables")
        with torch.cuda.device(out.device):
            self._check(self.lib.tri_attention_tasks(groups.data_ptr(), entries.data_ptr(), _ptr(v16), _ptr(v8), _ptr(v4),
                                                     vstat.data_ptr(), q8.data_ptr(), k8.data_ptr(), qa8.data_ptr(),
                                                     ka8.data_ptr(), _ptr(q4x), _ptr(k4x), _ptr(qa4), _ptr(ka4),
                                                     out.data_ptr(), int(out.dtype == torch.float16), out.stride(0),
                                                     out.stride(1), out.stride(2), b, hq, heads_kv, t, float(scale),
                                                     self.error_word(out.device).data_ptr(), _stream()))
        return out

    def cache_store(self, pool, unit_base, unit_tab, unit_count, unit_flags, tmeta, units, max_count, k8, k4, ka, ka4,
                    v8, v4, tiles):
        with torch.cuda.device(pool.device):
            self._check(self.lib.tri_cache_store(pool.data_ptr(), unit_base.data_ptr(), unit_tab.data_ptr(),
                                                 unit_count.data_ptr(), unit_flags.data_ptr(), tmeta.data_ptr(), units,
                                                 max_count, k8.data_ptr(), _ptr(k4), ka.data_ptr(), _ptr(ka4),
                                                 v8.data_ptr(), _ptr(v4), tiles, _stream()))

    def cache_store_bf16(self, pool, unit_base, units, k, v, chunk_begin=0, chunk_count=None):
        self._bhtd(k, "K"), self._bhtd(v, "V")
        if chunk_count is None:
            chunk_count = (k.shape[2] + 31) // 32 - chunk_begin
        with torch.cuda.device(pool.device):
            self._check(self.lib.tri_cache_store_bf16(pool.data_ptr(), unit_base.data_ptr(), units.data_ptr(),
                                                      units.numel(), k.data_ptr(), v.data_ptr(), k.shape[2], k.shape[1],
                                                      k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                                      v.stride(2), int(chunk_begin), int(chunk_count), _stream()))

    def decode(self, q, pool, unit_base, unit_tab, unit_flags, tmeta, segments, cta_segments, unit_slots, kstat, vstat,
               tail_k, tail_v, kcur, vcur, step, out, pm, pl, po, prompt, scale, phases=3, unit_done=None):
        if not (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[2] == 1 and q.shape[3] == 128 and q.stride(3) == 1):
            raise RuntimeError("q [B,Hq,1,128]")
        b, hq = q.shape[0], q.shape[1]
        hk, max_tail = kcur.shape[1], tail_k.shape[1]
        if not (hq % hk == 0 and hq // hk <= 8 and max_tail <= 1024 and step.dtype == torch.int64 and step.is_cuda and
                kcur.stride(3) == 1 and vcur.stride(1) == kcur.stride(1) and vcur.stride(0) == kcur.stride(0) and
                segments.dtype == torch.int32 and cta_segments.dtype == torch.int32 and tmeta.dtype == torch.int32 and
                unit_base.dtype == torch.int64 and
                tail_v.stride() == tail_k.stride() and out.stride(3) == 1):
            raise RuntimeError("decode geometry/buffers")
        if unit_done is not None and not (unit_done.dtype == torch.int32 and unit_done.is_cuda and
                                          unit_done.numel() >= b * hk):
            raise RuntimeError("unit_done int32 [units] on the device")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_decode(q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), unit_base.data_ptr(),
                                            unit_tab.data_ptr(), unit_flags.data_ptr(), tmeta.data_ptr(), segments.data_ptr(),
                                            cta_segments.data_ptr(), cta_segments.numel() - 1, unit_slots.data_ptr(), kstat.data_ptr(), vstat.data_ptr(),
                                            tail_k.data_ptr(), tail_v.data_ptr(), tail_k.stride(0), tail_k.stride(1),
                                            kcur.data_ptr(), vcur.data_ptr(), kcur.stride(0), kcur.stride(1),
                                            step.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), pm.data_ptr(),
                                            pl.data_ptr(), po.data_ptr(), unit_done.data_ptr() if unit_done is not None else None,
                                            b, hq, hk, int(prompt), max_tail, float(scale), int(phases),
                                            self.error_word(q.device).data_ptr(), _stream()))
        return out

    def decode_static(self, q, pool, unit_base, unit_tab, unit_flags, tmeta, segments, cta_segments, unit_slots, kstat,
                      vstat, tail_k, tail_v, kcur, vcur, step, out, prompt, scale):
        """Decode step whose split-KV partials live in the library's own fixed device array, for callers that
        cannot allocate GPU memory.  Refuses plans with more than 1024 segments; calls that may overlap on the
        GPU must not share a device."""
        if not (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[2] == 1 and q.shape[3] == 128 and q.stride(3) == 1):
            raise RuntimeError("q [B,Hq,1,128]")
        b, hq, hk = q.shape[0], q.shape[1], kcur.shape[1]
        if not (hq % hk == 0 and hq // hk <= 8 and tail_k.shape[1] <= 1024 and step.dtype == torch.int64 and step.is_cuda and
                kcur.stride(3) == 1 and vcur.stride(1) == kcur.stride(1) and vcur.stride(0) == kcur.stride(0) and
                segments.dtype == torch.int32 and cta_segments.dtype == torch.int32 and tmeta.dtype == torch.int32 and
                unit_base.dtype == torch.int64 and unit_slots.dtype == torch.int32 and
                tail_v.stride() == tail_k.stride() and out.stride(3) == 1):
            raise RuntimeError("decode geometry/buffers")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_decode_static(
                q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), unit_base.data_ptr(), unit_tab.data_ptr(),
                unit_flags.data_ptr(), tmeta.data_ptr(), segments.data_ptr(), cta_segments.data_ptr(),
                cta_segments.numel() - 1, segments.shape[0], unit_slots.data_ptr(), kstat.data_ptr(), vstat.data_ptr(),
                tail_k.data_ptr(), tail_v.data_ptr(), tail_k.stride(0), tail_k.stride(1), kcur.data_ptr(), vcur.data_ptr(),
                kcur.stride(0), kcur.stride(1), step.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), b, hq, hk,
                int(prompt), tail_k.shape[1], float(scale), self.error_word(q.device).data_ptr(), _stream()))
        return out

    def decode_fold(self, pm, pl, po, unit_slots, fm, fl, fo, group):
        with torch.cuda.device(pm.device):
            self._check(self.lib.tri_decode_fold(pm.data_ptr(), pl.data_ptr(), po.data_ptr(), unit_slots.data_ptr(),
                                                 fm.data_ptr(), fl.data_ptr(), fo.data_ptr(), unit_slots.shape[0], group,
                                                 _stream()))

    def decode_partials(self, q, pool, unit_base, unit_tab, unit_flags, tmeta, segments, cta_segments, unit_slots, pm, pl, po,
                        unit_done, fm, fl, fo, heads_kv, prompt, scale, peers=None, rank=0, epoch=None):
        """This GPU's part of a sequence-split decode step: split pass + in-kernel fold to one triple per (unit, Q head),
        into fm / fl / fo, or (those None; peers = int64 device tensor of every rank's exchange-buffer address as mapped
        here, epoch = int32 [units]) by peer stores into every GPU's exchange buffer."""
        if not (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[2] == 1 and q.shape[3] == 128 and q.stride(3) == 1 and
                unit_done.dtype == torch.int32):
            raise RuntimeError("decode geometry/buffers")
        if peers is None:
            if not (fm.dtype == torch.float32 and fo.is_contiguous()):
                raise RuntimeError("decode geometry/buffers")
        elif not (peers.dtype == torch.int64 and peers.is_cuda and epoch is not None and epoch.dtype == torch.int32 and
                  epoch.numel() >= q.shape[0] * heads_kv and fm is None and fl is None and fo is None):
            raise RuntimeError("decode_partials: exchange group")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_decode_partials(
                q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), unit_base.data_ptr(), unit_tab.data_ptr(),
                unit_flags.data_ptr(), tmeta.data_ptr(), segments.data_ptr(), cta_segments.data_ptr(), cta_segments.numel() - 1,
                unit_slots.data_ptr(), pm.data_ptr(), pl.data_ptr(), po.data_ptr(), unit_done.data_ptr(), _ptr(fm),
                _ptr(fl), _ptr(fo), _ptr(peers), 0 if peers is None else peers.numel(), int(rank), _ptr(epoch),
                q.shape[0], q.shape[1], heads_kv, int(prompt), float(scale),
                self.error_word(q.device).data_ptr(), _stream()))

    def decode_split(self, q, pool, unit_base, unit_tab, unit_flags, tmeta, segments, cta_segments, unit_slots, kstat, vstat,
                     tail_k, tail_v, kcur, vcur, step, out, pm, pl, po, unit_done, peers, rank, epoch, present, prompt, scale):
        """A whole sequence-split decode step on this GPU as one kernel: split pass, fold, delivery of the triples into every
        GPU's exchange buffer, wait for the others' and merge.  Buffers as decode / decode_partials."""
        if not (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[2] == 1 and q.shape[3] == 128 and q.stride(3) == 1 and
                kcur.stride(3) == 1 and vcur.stride(0) == kcur.stride(0) and vcur.stride(1) == kcur.stride(1) and
                tail_v.stride() == tail_k.stride() and out.stride(3) == 1 and step.dtype == torch.int64 and
                peers.dtype == torch.int64 and epoch.dtype == torch.int32 and present.dtype == torch.int32 and
                present.numel() == peers.numel() * q.shape[0] * kcur.shape[1]):
            raise RuntimeError("decode geometry/buffers")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_decode_split(
                q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), unit_base.data_ptr(), unit_tab.data_ptr(),
                unit_flags.data_ptr(), tmeta.data_ptr(), segments.data_ptr(), cta_segments.data_ptr(), cta_segments.numel() - 1,
                unit_slots.data_ptr(), kstat.data_ptr(), vstat.data_ptr(), tail_k.data_ptr(), tail_v.data_ptr(),
                tail_k.stride(0), tail_k.stride(1), kcur.data_ptr(), vcur.data_ptr(), kcur.stride(0), kcur.stride(1),
                step.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), pm.data_ptr(), pl.data_ptr(), po.data_ptr(),
                unit_done.data_ptr(), peers.data_ptr(), peers.numel(), int(rank), epoch.data_ptr(), present.data_ptr(),
                q.shape[0], q.shape[1], kcur.shape[1], int(prompt), tail_k.shape[1], float(scale),
                self.error_word(q.device).data_ptr(), _stream()))
        return out

    def decode_merge(self, q, pm, pl, po, split_stride, unit_slots, kstat, vstat, tail_k, tail_v, kcur, vcur, step, out, scale,
                     exchange=None, present=None, seen=None, world=0, gather=None):
        """The merge alone, over partials that may lie strided (triples gathered from several GPUs, merged in place), or
        (exchange = this rank's exchange buffer, present int32 [world, units], seen int32 [units]) over the triples that
        the peer-memory exchange of decode_partials delivers, waiting for them per unit."""
        if not (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[2] == 1 and q.shape[3] == 128 and q.stride(3) == 1 and
                kcur.stride(3) == 1 and vcur.stride(0) == kcur.stride(0) and vcur.stride(1) == kcur.stride(1) and
                tail_v.stride() == tail_k.stride() and out.stride(3) == 1 and step.dtype == torch.int64):
            raise RuntimeError("decode geometry/buffers")
        with torch.cuda.device(q.device):
            self._check(self.lib.tri_decode_merge(
                q.data_ptr(), q.stride(0), q.stride(1), _ptr(pm), _ptr(pl), _ptr(po), int(split_stride),
                _ptr(exchange), _ptr(present), _ptr(seen), int(world),
                *((None, 0, 0, None, 0, None) if gather is None else
                  (gather["peers"].data_ptr(), gather["peers"].numel(), int(gather["rank"]), gather["unit_row"].data_ptr(),
                   int(gather["rows_total"]), gather["sync"].data_ptr())),
                unit_slots.data_ptr(), kstat.data_ptr(), vstat.data_ptr(), tail_k.data_ptr(), tail_v.data_ptr(),
                tail_k.stride(0), tail_k.stride(1), kcur.data_ptr(), vcur.data_ptr(), kcur.stride(0), kcur.stride(1),
                step.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), q.shape[0], q.shape[1], kcur.shape[1],
                tail_k.shape[1], float(scale), self.error_word(q.device).data_ptr(), _stream()))
        return out

    def gather_wait(self, buffer, rows_total, seen, world):
        """Wait (on the device, bounded) until every rank's rows of the next step have arrived in this GPU's gather buffer."""
        with torch.cuda.device(buffer.device):
            self._check(self.lib.tri_gather_wait(buffer.data_ptr(), int(rows_total), seen.data_ptr(), int(world),
                                                 self.error_word(buffer.device).data_ptr(), _stream()))

    def decode_tail_hint(self, rows):
        """Rows in the BF16 tails for the decode launches that follow on this thread: picks the merge kernel's instantiation
        (plain or unrolled row loops, bit-equal results; LONG_TAIL_ROWS is where the library switches; negative = not
        known)."""
        self._check(self.lib.tri_decode_tail_hint(int(rows)))

    def decode_occupancy(self):
        return self._check(self.lib.tri_decode_occupancy())

    # -- parity helpers --------------------------------------------------------------------------
    def qk_accumulators(self, requests, q8, q4x, k8, k4x, batch, heads_q, heads_kv, tokens):
        acc = torch.empty((requests.shape[0], 128, 64), dtype=torch.int32, device=q8.device)
        with torch.cuda.device(q8.device):
            self._check(self.lib.tri_qk_accumulators(requests.data_ptr(), requests.shape[0], q8.data_ptr(), _ptr(q4x),
                                                     k8.data_ptr(), _ptr(k4x), acc.data_ptr(), batch, heads_q, heads_kv,
                                                     tokens, self.error_word(q8.device).data_ptr(), _stream()))
        return acc


@functools.cache
def load_extension() -> Module:
    if not torch.cuda.is_available():
        raise RuntimeError("TriAttention requires a CUDA GPU.")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise RuntimeError(f"this build targets sm_100a (B200) only; found compute capability {major}.{minor}")
    return Module(load_library())
