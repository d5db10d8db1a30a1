"""Drives the reference's own CUDA extension (``oracle/_ref``) for one sequence.  Test and baseline infrastructure:
only the tests, the golden generator and the baseline legs of ``bench.py`` import it.

The reference's Python executors are not importable on the GPU box, so the buffer shapes and call
sequences of ``triattention/kernels/prefill.py:60-108`` and ``triattention/kernels/decode.py:24-80`` are
restated here: allocate what the extension's checks demand (``common_host.cuh:4-13,29-35,52-64``,
``prefill_sm80.cu:516-527``) and call its five functions.
"""
from __future__ import annotations

import numpy as np
import torch

import triattention_oracle as orc

F16, I8, I4, Q4 = orc.F16, orc.I8, orc.I4, orc.Q4


def bf16_cuda(x):
    """float32 numpy holding bf16 values -> cuda bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).cuda()


class RefRunner:
    def __init__(self, mod):
        self.mod = mod

    def prefill(self, q, k, v, bands, scale, with_decode=True, out_dtype=torch.bfloat16, attention=True):
        """q [1,Hq,T,128], k/v [1,Hkv,T,128] cuda bf16; bands numpy [Hq,2].  Returns the operand dict.
        attention=False stops after the KV-cache write (prepare_qk + pack_v): enough to build a decode cache."""
        _, hq, t, _ = q.shape
        hk, rows, dev = k.shape[1], (t + 63) // 64, q.device
        formats = set(orc.band_formats(bands, rows))
        vcodes = orc.decode_v_codes(rows)
        if with_decode:
            formats |= set(int(c) for c in np.unique(vcodes))
        int4 = Q4 in orc.band_formats(bands, rows)
        u32 = lambda n: torch.empty(n, dtype=torch.uint32, device=dev)
        f32 = lambda n: torch.empty(n, dtype=torch.float32, device=dev)
        o = dict(q8=torch.empty((1, hq, t, 128), dtype=torch.int8, device=dev), qa=f32(hq * t), kp=u32(hk * rows * 2048),
                 ka=f32(hk * rows * 4), partial=f32(hk * 64 * 3 * 128), kstat=f32(hk * 3 * 128),
                 vstat=torch.empty((1, hk, 3, 128), dtype=torch.float32, device=dev),
                 q4=torch.empty(hq * t * 64, dtype=torch.uint8, device=dev) if int4 else None,
                 qa4=f32(hq * t) if int4 else None, k4=u32(hk * rows * 1024) if int4 else None,
                 ka4=f32(hk * rows * 4) if int4 else None)
        packed = {F16: u32(hk * rows * 4096), I8: u32(hk * rows * 2048) if (I8 in formats or int4) else None,
                  I4: u32(hk * rows * 1024) if I4 in formats else None}
        self.mod.prepare_qk(q, k, o["q8"], o["qa"], o["kp"], o["ka"], o["partial"], o["kstat"], o["q4"], o["qa4"], o["k4"], o["ka4"])
        self.mod.pack_v(v, o["partial"], o["vstat"], packed[F16], packed[I8], packed[I4])
        order = torch.from_numpy(orc.cta_order(hq, hk, rows)).to(dev)
        bands_t = torch.from_numpy(np.asarray(bands, np.int32)).contiguous().to(dev)
        out = torch.empty((1, t, hq, 128), dtype=out_dtype, device=dev).transpose(1, 2) if attention else None
        if attention:
            self.mod.attention(order, bands_t, None, None, packed[F16], packed[I8], packed[I4], o["vstat"], o["q8"], o["kp"],
                               o["qa"], o["ka"], o["q4"], o["k4"], o["qa4"], o["ka4"], out, float(scale))
        o.update(out=out, packed=packed, rows=rows, t=t, hq=hq, hk=hk, vcodes=vcodes, int4=int4)
        return o

    def prefill_tasks(self, q, k, v, groups, entries, scale):
        """Task-table mode (prefill_sm80.cu:287-292,520-523): every operand format is prepared, the attention gets
        groups / entries instead of bands.  groups int32 [Hq*rows*4+1], entries int32 [...] (numpy)."""
        _, hq, t, _ = q.shape
        hk, rows, dev = k.shape[1], (t + 63) // 64, q.device
        u32 = lambda n: torch.empty(n, dtype=torch.uint32, device=dev)
        f32 = lambda n: torch.empty(n, dtype=torch.float32, device=dev)
        o = dict(q8=torch.empty((1, hq, t, 128), dtype=torch.int8, device=dev), qa=f32(hq * t), kp=u32(hk * rows * 2048),
                 ka=f32(hk * rows * 4), partial=f32(hk * 64 * 3 * 128), kstat=f32(hk * 3 * 128),
                 vstat=torch.empty((1, hk, 3, 128), dtype=torch.float32, device=dev),
                 q4=torch.empty(hq * t * 64, dtype=torch.uint8, device=dev), qa4=f32(hq * t), k4=u32(hk * rows * 1024),
                 ka4=f32(hk * rows * 4))
        packed = {F16: u32(hk * rows * 4096), I8: u32(hk * rows * 2048), I4: u32(hk * rows * 1024)}
        self.mod.prepare_qk(q, k, o["q8"], o["qa"], o["kp"], o["ka"], o["partial"], o["kstat"], o["q4"], o["qa4"], o["k4"], o["ka4"])
        self.mod.pack_v(v, o["partial"], o["vstat"], packed[F16], packed[I8], packed[I4])
        order = torch.from_numpy(orc.cta_order(hq, hk, rows)).to(dev)
        out = torch.empty((1, t, hq, 128), dtype=torch.bfloat16, device=dev).transpose(1, 2)
        self.mod.attention(order, None, torch.from_numpy(np.asarray(groups, np.int32)).to(dev),
                           torch.from_numpy(np.asarray(entries, np.int32)).to(dev), packed[F16], packed[I8], packed[I4],
                           o["vstat"], o["q8"], o["kp"], o["qa"], o["ka"], o["q4"], o["k4"], o["qa4"], o["ka4"], out, float(scale))
        return out

    def decode_setup(self, o, bands, max_tail, per=None):
        """kernels/decode.py:24-67 restated with numpy; returns the buffers `decode` needs.
        per=None applies the reference's own rule (decode.py:53-55): kept tiles / (SMs x resident CTAs per SM)."""
        t, hk, tiles, dev = o["t"], o["hk"], o["rows"], o["qa"].device
        tabs = orc.decode_tables(bands, hk, t)
        if per is None:
            wave = torch.cuda.get_device_properties(dev).multi_processor_count * self.mod.decode_occupancy()
            per = max(1, -(-sum(len(tb["tiles"]) for tb in tabs) // wave))
        count = np.array([len(tb["tiles"]) for tb in tabs])
        maxn = max(1, int(count.max()))
        entry = np.zeros((hk, maxn), np.int32); kinfo = np.zeros((hk, maxn), np.int32); slot = np.zeros((hk, maxn), np.int32)
        rows8, rows4, vrows = [], [], {I8: [], I4: []}
        for kh, tb in enumerate(tabs):
            # dropped tiles follow the kept ones in `entry` (stable argsort of kv==0); only [0,count) is read
            for i, tile in enumerate(tb["tiles"]):
                entry[kh, i] = tile
                is4 = int(tb["state"][i] == 4)
                kslot = len(rows4) if is4 else len(rows8)
                (rows4 if is4 else rows8).append(kh * tiles + tile)
                kinfo[kh, i] = int(tb["rowmask"][i]) | (is4 << 8) | (kslot << 9)
                code = int(tb["vfmt"][i])
                slot[kh, i] = len(vrows[code]); vrows[code].append(kh * tiles + tile)
        idx = lambda r: torch.tensor(r, dtype=torch.long, device=dev)
        pk = o["packed"]
        take = lambda buf, words, rows: (buf.view(hk * tiles, words).view(torch.int32).index_select(0, idx(rows)).view(torch.uint32)
                                         if rows else torch.zeros((1, words), dtype=torch.uint32, device=dev))
        st = dict(entry=torch.from_numpy(entry).to(dev), kinfo=torch.from_numpy(kinfo).to(dev), slot=torch.from_numpy(slot).to(dev),
                  count=torch.from_numpy(count.astype(np.int32)).to(dev),
                  fmt=torch.from_numpy((o["vcodes"] - 1).astype(np.int32)).to(dev),
                  k8=take(o["kp"], 2048, rows8), k4=take(o["k4"], 1024, rows4) if rows4 else None,
                  ka=o["ka"], ka4=o["ka4"] if rows4 else None, v8=take(pk[I8], 2048, vrows[I8]),
                  v4=take(pk[I4], 1024, vrows[I4]) if pk[I4] is not None else torch.zeros((1, 1024), dtype=torch.uint32, device=dev),
                  kstat=o["kstat"], vstat=o["vstat"], prompt=t, per=per, maxn=maxn,
                  tail_k=torch.zeros((1, hk, max_tail, 128), dtype=torch.bfloat16, device=dev),
                  tail_v=torch.zeros((1, hk, max_tail, 128), dtype=torch.bfloat16, device=dev),
                  step=torch.zeros(1, dtype=torch.int64, device=dev))
        splits = max(1, -(-maxn // per))
        hq = o["hq"]
        st["pm"], st["pl"] = torch.zeros(hq * splits, device=dev), torch.zeros(hq * splits, device=dev)
        st["po"] = torch.zeros(hq * splits * 128, device=dev)
        st["splits"] = splits
        return st

    def decode(self, st, q, kcur, vcur, scale):
        out = torch.empty_like(q)
        self.mod.decode(q, st["k8"], st["k4"], st["ka"], st["ka4"], st["entry"], st["kinfo"], st["count"], st["fmt"], st["slot"],
                        st["v8"], st["v4"], st["vstat"], st["kstat"], st["tail_k"], st["tail_v"], kcur, vcur, st["step"], out,
                        st["pm"], st["pl"], st["po"], st["prompt"], st["per"], float(scale))
        return out


def ref_logical(o):
    """Reference operand buffers -> logical numpy arrays comparable with the oracle's."""
    hq, hk, t, rows = o["hq"], o["hk"], o["t"], o["rows"]
    cpu = lambda x: x.detach().cpu().numpy()
    res = dict(q8=cpu(o["q8"])[0], qa=cpu(o["qa"]).reshape(hq, t), ka=cpu(o["ka"]).reshape(hk, rows, 4),
               kstat=cpu(o["kstat"]).reshape(hk, 3, 128), vstat=cpu(o["vstat"]).reshape(hk, 3, 128),
               k8=orc.unpack_ref_k8(cpu(o["kp"].view(torch.int32)).view(np.uint32).reshape(hk, rows, 2048)),
               v16=orc.unpack_ref_v16(cpu(o["packed"][F16].view(torch.int32)).view(np.uint32).reshape(hk, rows, 4096)))
    if o["packed"][I8] is not None:
        res["v8"] = orc.unpack_ref_v8(cpu(o["packed"][I8].view(torch.int32)).view(np.uint32).reshape(hk, rows, 2048))
    if o["packed"][I4] is not None:
        res["v4"] = orc.unpack_ref_v4(cpu(o["packed"][I4].view(torch.int32)).view(np.uint32).reshape(hk, rows, 1024))
    if o["int4"]:
        res.update(q4=orc.unpack_ref_q4(cpu(o["q4"]).reshape(hq, t, 64)), qa4=cpu(o["qa4"]).reshape(hq, t),
                   k4=orc.unpack_ref_k4(cpu(o["k4"].view(torch.int32)).view(np.uint32).reshape(hk, rows, 1024)),
                   ka4=cpu(o["ka4"]).reshape(hk, rows, 4))
    return res
