"""Prefill executor: KV-cache write (rotate + quantise + pack) and banded attention, batched.

Mirrors ``triattention/kernels/prefill.py`` (``BandTable``, ``Prefill`` with the same constructor,
``buffers`` attribute and ``__call__(layer, q, k, v, scale)``), on top of the sm_100a C-ABI library.
Differences from the reference, all additive:
  * q/k/v carry a batch dimension ``[B,H,T,128]`` (the reference asserts batch 1);
  * operands live in the tile blob layouts of ``csrc/common.cuh`` instead of mma.sync fragment order;
  * a map may mark KV heads as un-quantised BF16 (``bands_fn.bf16_kv_heads(layer)``); their groups are
    computed as exact attention by the same kernel launch (bf16 QK^T, exact online softmax), which is what the
    reference's ``exact_attention`` baseline computes with torch's SDPA (``triattention/models.py:45-47``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

SKIP, F16, I8, I4, Q4 = 0, 1, 2, 3, 4
K8_BYTES, K4_BYTES, V16_BYTES, V8_BYTES, V4_BYTES = 8192, 4096, 16384, 8192, 4096


@dataclass
class BandTable:
    order: torch.Tensor      # reference CTA order (kernels/prefill.py:24-25); informational, the kernel orders itself
    bands: torch.Tensor      # int32 [Hq,2] on the device; (0,0) for heads of BF16 KV groups (skipped by the kernel)
    formats: frozenset
    host: torch.Tensor       # int32 [Hq,2] as given by the map
    bf16_kv: tuple = ()
    q_modes: torch.Tensor = None   # int32 [Hq] on the device: bit 0 = the head's INT8 Q codes are read, bit 1 = its INT4 codes
    raw_kv: torch.Tensor = None    # int32 [Hkv] on the device, 1 = un-quantised KV head; None when the map has none

    @classmethod
    def build(cls, bands, rows, kv_heads, device, bf16_kv=()):
        b = torch.as_tensor(bands, dtype=torch.int64).cpu()
        if b.dim() != 2 or b.shape[1] != 2 or b.shape[0] % kv_heads:
            raise ValueError("bands must be [Hq,2] with Hq a multiple of the KV heads")
        group = b.shape[0] // kv_heads
        quant = torch.ones(b.shape[0], dtype=torch.bool)
        for kh in bf16_kv:
            quant[kh * group:(kh + 1) * group] = False
        if bool((b[quant, 0] < 1).any()):
            raise ValueError("band width w8 must be at least 1 tile")
        w8, w4 = b[:, :1], b[:, 1:]
        qb = torch.arange(rows)[None, :]
        n8 = (qb - torch.clamp(qb - w8 + 1, min=1)).clamp(min=0)[quant]
        n4 = (qb - w8 - torch.clamp(qb - w4 + 1, min=1) + 1).clamp(min=0)[quant]
        heads = torch.arange(b.shape[0]).view(kv_heads, -1)
        order = (heads[:, None, :] * rows + qb.flip(1)[0][None, :, None]).flatten()
        formats = {F16} | ({I8} if bool((n8 > 0).any()) else set()) | ({Q4} if bool((n4 > 0).any()) else set())
        host = b.to(torch.int32).contiguous()
        dev = host.clone()
        dev[~quant] = 0
        modes = torch.zeros(b.shape[0], dtype=torch.int32)
        modes[quant] = 1 + 2 * (n4 > 0).any(dim=1).to(torch.int32)
        raw_kv = None
        if bf16_kv:
            raw_kv = torch.zeros(kv_heads, dtype=torch.int32)
            raw_kv[list(bf16_kv)] = 1
            raw_kv = raw_kv.to(device)
        return cls(order.to(torch.int32).to(device), dev.to(device), frozenset(formats), host, tuple(sorted(bf16_kv)),
                   modes.to(device), raw_kv)


class Prefill:
    def __init__(self, module, bands_fn, decode_cache=None):
        self.module, self.bands_fn, self.decode_cache = module, bands_fn, decode_cache
        self.tables, self.buffers, self.views = {}, {}, {}

    def table(self, layer, heads, kv_heads, rows, device):
        key = (None if getattr(self.bands_fn, "layer_independent", False) else layer, heads, rows)
        if key not in self.tables:
            bf16 = getattr(self.bands_fn, "bf16_kv_heads", None)
            self.tables[key] = BandTable.build(self.bands_fn(layer, heads), rows, kv_heads, device,
                                               tuple(bf16(layer)) if bf16 else ())
        return self.tables[key]

    def buffer(self, name, nbytes, device):
        """Scratch shared by all layers (and by executors that share ``buffers``), grown on demand."""
        current = self.buffers.get(name)
        if current is None or current.numel() < nbytes or current.device != torch.device(device):
            current = self.buffers[name] = torch.empty(nbytes, dtype=torch.uint8, device=device)
            self.views.clear()
        return current[:nbytes]

    def operands(self, b, hq, hk, t, int4, need_k4, formats, device):
        key = (b, hq, hk, t, int4, need_k4, formats, str(device))
        if key in self.views:
            return self.views[key]
        rows = (t + 63) // 64
        raw = lambda name, n: self.buffer(name, n, device)
        f32 = lambda name, n: self.buffer(name, 4 * n, device).view(torch.float32)
        ops = dict(
            q8=raw("q8", b * hq * t * 128).view(torch.int8).view(b * hq, t, 128),
            qa=f32("qa", b * hq * t),
            k8=raw("k8", b * hk * rows * K8_BYTES),
            ka=f32("ka", b * hk * rows * 4),
            partial=f32("partial", b * hk * 64 * 3 * 128),
            partial_v=f32("partial_v", b * hk * 64 * 3 * 128),
            kstat=f32("kstat", b * hk * 3 * 128).view(b * hk, 3, 128),
            vstat=f32("vstat", b * hk * 3 * 128).view(b * hk, 3, 128),
            q4x=raw("q4x", b * hq * t * 128).view(torch.int8).view(b * hq, t, 128) if int4 else None,
            qa4=f32("qa4", b * hq * t) if int4 else None,
            k4x=raw("k4x", b * hk * rows * K8_BYTES) if int4 else None,
            ka4=f32("ka4", b * hk * rows * 4) if int4 else None,
            k4=raw("k4", b * hk * rows * K4_BYTES) if (int4 and need_k4) else None,
            v16=raw("v16", b * hk * rows * V16_BYTES),
            v8=raw("v8", b * hk * rows * V8_BYTES) if (I8 in formats or Q4 in formats) else None,
            v8h=raw("v8h", b * hk * rows * V16_BYTES) if (I8 in formats or Q4 in formats) else None,
            v4=raw("v4", b * hk * rows * V4_BYTES) if I4 in formats else None,
        )
        self.views[key] = ops
        return ops

    def write(self, layer, q, k, v):
        """KV-cache write path only: rotate + quantise Q/K, normalise + pack V.  Returns (band table, operands)."""
        b, hq, t, _ = q.shape
        hk, rows, device = k.shape[1], (t + 63) // 64, q.device
        table = self.table(layer, hq, hk, rows, device)
        decode = self.decode_cache.codes(rows) if self.decode_cache is not None else None
        formats = table.formats | decode[1] if decode is not None else table.formats
        need_k4 = self.decode_cache is not None and self.decode_cache.needs_k4(table.host, hk, rows, table.bf16_kv)
        int4 = Q4 in table.formats or need_k4
        ops = self.operands(b, hq, hk, t, int4, need_k4, formats, device)
        m = self.module
        # the reference's two calls (prepare_qk, then pack_v: kernels/prefill.py:99-101) as one, whose chains overlap
        m.write_kv(q, k, v, ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"], ops["partial_v"],
                   ops["vstat"], ops["q4x"], ops["qa4"], ops["k4x"], ops["ka4"], ops["k4"], q_modes=table.q_modes,
                   v16=ops["v16"], v8=ops["v8"], v4=ops["v4"], v8h=ops["v8h"], raw_heads=table.raw_kv)
        return table, ops

    def __call__(self, layer, q, k, v, scale, out_dtype=None):
        """out_dtype: torch.bfloat16 (default: q's) or torch.float16, the two output types of the reference's kernel
        (prefill_sm80.cu:533-539)."""
        b, hq, t, _ = q.shape
        hk, device = k.shape[1], q.device
        table, ops = self.write(layer, q, k, v)
        q4 = Q4 in table.formats
        out = torch.empty((b, t, hq, 128), dtype=out_dtype or q.dtype, device=device).transpose(1, 2)
        # un-quantised extension heads run in the same launch: exact attention from the raw Q / K rows and fp16 V blobs
        raw = (q, k) if table.bf16_kv else (None, None)
        self.module.attention(table.bands, ops["v16"], ops["v8h"], ops["vstat"], ops["q8"], ops["k8"], ops["qa"], ops["ka"],
                              ops["q4x"] if q4 else None, ops["k4x"] if q4 else None, ops["qa4"] if q4 else None,
                              ops["ka4"] if q4 else None, out, scale, hk, q_raw=raw[0], k_raw=raw[1])
        if self.decode_cache is not None:
            self.decode_cache.store(layer, t, ops, table.host, k, v, table.bf16_kv)
        return out

    def sweep(self, configs, q, k, v, scale, rows=None, out_dtype=None):
        """Outputs of several uniform band maps over the same Q / K / V in one pass: one KV-cache write (the operands do
        not depend on the map), one attention launch for all configurations, and only the query rows that are wanted.
        The reference's calibration runs one full prefill per configuration (calibrate.py:46-63).
        configs: list of (w8, w4) applied to every Q head; rows: evaluate only the last `rows` query rows (None = all).
        Returns (out [C,B,Hq,R,128], row0): out[..., i, :] is query row row0 + i, with row0 <= T - rows."""
        b, hq, t, _ = q.shape
        hk, device = k.shape[1], q.device
        bands = torch.tensor([[list(c)] * hq for c in configs], dtype=torch.int32)
        if bands.dim() != 3 or bool((bands[:, :, 0] < 1).any()):
            raise ValueError("configs must be (w8, w4) pairs with w8 >= 1")
        # every operand format once: INT8 and INT4 codes of Q and K, the fp16 V' blob and the fp16 rendering of the V codes.
        # (V is normalised by its statistics for all configurations; a configuration without any INT8 tile, which alone
        # would run on un-normalised V like the reference's identity mode, common_host.cuh:39, differs by that rounding.)
        ops = self.operands(b, hq, hk, t, True, False, frozenset({F16, I8, Q4}), device)
        m = self.module
        m.write_kv(q, k, v, ops["q8"], ops["qa"], ops["k8"], ops["ka"], ops["partial"], ops["kstat"], ops["partial_v"],
                   ops["vstat"], ops["q4x"], ops["qa4"], ops["k4x"], ops["ka4"], v16=ops["v16"], v8=ops["v8"], v8h=ops["v8h"])
        first_block = 0 if rows is None else max(0, (t - int(rows)) // 64)
        row0 = (first_block // 4) * 256
        out = torch.empty((len(configs), b, hq, t - row0, 128), dtype=out_dtype or q.dtype, device=device)
        m.attention_sweep(bands.to(device), first_block, ops["v16"], ops["v8h"], ops["vstat"], ops["q8"], ops["k8"], ops["qa"],
                          ops["ka"], ops["q4x"], ops["k4x"], ops["qa4"], ops["ka4"], out, row0, scale, hk, t)
        return out, row0
