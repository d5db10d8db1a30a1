"""Decode cache: per-(sequence, KV head) byte streams of kept tiles, a cost-balanced static partition
of the tile sequence over persistent CTAs, the BF16 tail of generated tokens, and the decode step.

Mirrors ``triattention/kernels/decode.py`` (``DecodeCache(module, max_tail)``, ``codes``, ``store``,
``__call__``, ``advance``, ``stored``).  The tile-state rules are the reference's
(``decode.py:28-36``): tile 0 and tiles closer than ``w8`` to the end keep INT8 K, tiles closer than
``w4`` keep INT4 K, the rest are dropped; a KV head keeps the widest state of its Q heads and a row
mask says which Q heads attend; V is INT8 for tile 0 and the last 16 tiles, INT4 elsewhere
(``decode.py:17-22``).  What differs is the data structure: the reference compacts tiles into four
dense arrays with host-side argsort/cumsum and splits by a fixed tile count; here each unit is one
contiguous byte stream (K blob, V blob, K scales per tile) filled by one gather kernel, and the
sequence of all tiles is cut into one contiguous slice of equal cost per CTA (one CTA per SM), so
INT8 / INT4 / BF16 units are balanced by bytes and every CTA finishes at the same time.
"""
from __future__ import annotations

import numpy as np
import torch

from triattention_b200.kernels.prefill import I4, I8

NEAR_V8 = 16
K8_BYTES, K4_BYTES, V8_BYTES, V4_BYTES = 8192, 4096, 8192, 4096
BF16_CHUNK_KEYS, BF16_CHUNK_BYTES = 32, 16384
INFO_ROW_SHIFT, INFO_K4, INFO_V4, INFO_BF16, INFO_FULL = 12, 1 << 20, 1 << 21, 1 << 22, 1 << 23
FOLD_KEYS = 64      # generated tokens per appended tile (DecodeCache(fold_tail=...))
MAX_GROUP = 8
# Relative time of one tile on one SM, by kind, for the partition's cost model: (BF16 32-key chunk,
# INT8-K/INT8-V tile, any other quantised tile).  Quantised tiles are bound by their arithmetic (the same
# for 8 and 12 KB of codes); 16 KB tiles are bound by the SM's share of the HBM bandwidth.
TILE_COSTS = (0.85, 1.05, 1.0)


def tile_states(bands, heads_kv, tiles):
    """decode.py:28-36 -> (kv state [Hkv,tiles] in {0,4,8}, rowmask [Hkv,tiles])."""
    b = np.asarray(bands, np.int64)
    j = np.arange(tiles)
    w8, w4, d = b[:, :1], b[:, 1:], (tiles - 1) - j[None, :]
    state = np.where((j[None, :] == 0) | (d < w8), 8, np.where(d < w4, 4, 0)).reshape(heads_kv, -1, tiles)
    rowmask = ((state > 0).astype(np.int64) << np.arange(state.shape[1])[None, :, None]).sum(1)
    return state.max(1), rowmask


def plan_streams(bands, heads_kv, prompt, batch, bf16_kv=(), ctas=148, tile_costs=TILE_COSTS, split=None, extra=0, reserve=0):
    """Host-side layout of one layer's cache and its partition over `ctas` persistent CTAs (numpy).
    split = (rank, world) keeps only this rank's part of every unit's kept-tile list (sequence split).
    extra = tiles of 64 generated tokens appended behind the prompt's tiles (INT8 K and V, seen by every Q head
    of the group, 64 live keys each: INFO_FULL; two 32-key chunks for a BF16 unit); reserve >= extra = how many
    of them every unit's stream has room for, so that the streams do not move when a tile is appended
    (append_off [Hkv] = where the first one goes).

    Returns a dict of numpy arrays: tmeta [N,2], tab_begin/count/head_bytes [Hkv], unit_base [U] (int64),
    unit_tab/unit_count/unit_flags [U], segments [S,4] = (unit, first kept tile, tile count, partial slot),
    cta_segments [ctas+1], unit_slots [U,2], plus totals.
    """
    tiles = (prompt + 63) // 64
    kv, rowmask = tile_states(bands, heads_kv, tiles)
    j = np.arange(tiles)
    v4 = ~((tiles - 1 - j < NEAR_V8) | (j == 0))
    if extra < 0 or reserve < 0 or ((extra or reserve) and split is not None):
        raise ValueError("appended tiles: extra, reserve >= 0, and not together with a sequence split")
    reserve = max(reserve, extra)
    metas, sizes, costs, tab_begin, count, head_bytes, append_off = [], [], [], [], [], [], []
    bf16_range = (0, (prompt + BF16_CHUNK_KEYS - 1) // BF16_CHUNK_KEYS)
    for kh in range(heads_kv):
        if kh in bf16_kv:
            n = (prompt + BF16_CHUNK_KEYS - 1) // BF16_CHUNK_KEYS
            info = np.arange(n, dtype=np.int64) | (0xFF << INFO_ROW_SHIFT) | INFO_BF16
            size = np.full(n, BF16_CHUNK_BYTES, np.int64)
            costs.append(np.full(n, tile_costs[0], np.float64))
        else:
            kept = np.nonzero(kv[kh] > 0)[0]
            k4 = kv[kh][kept] == 4
            info = kept | ((rowmask[kh][kept] & 0xFF) << INFO_ROW_SHIFT) | np.where(k4, INFO_K4, 0) | np.where(v4[kept], INFO_V4, 0)
            size = np.where(k4, K4_BYTES, K8_BYTES) + np.where(v4[kept], V4_BYTES, V8_BYTES) + 16
            costs.append(np.where(~k4 & ~v4[kept], tile_costs[1], tile_costs[2]).astype(np.float64))
        bf16_head = kh in bf16_kv
        append_off.append(int(size.sum()))
        if extra:
            n_new = 2 * extra if bf16_head else extra
            flags = (0xFF << INFO_ROW_SHIFT) | INFO_FULL | (INFO_BF16 if bf16_head else 0)
            info = np.concatenate([info, np.full(n_new, flags, np.int64)])
            size = np.concatenate([size, np.full(n_new, BF16_CHUNK_BYTES if bf16_head else K8_BYTES + V8_BYTES + 16, np.int64)])
            costs[-1] = np.concatenate([costs[-1], np.full(n_new, tile_costs[0] if bf16_head else tile_costs[1], np.float64)])
        if split is not None:   # sequence split across GPUs: this rank keeps one contiguous, cost-balanced part
            rank, world = split
            cc = np.concatenate([[0], np.cumsum(costs[-1])])
            lo = int(np.searchsorted(cc, rank * cc[-1] / world, side="left"))
            hi = len(info) if rank == world - 1 else int(np.searchsorted(cc, (rank + 1) * cc[-1] / world, side="left"))
            info, size, costs[-1] = info[lo:hi], size[lo:hi], costs[-1][lo:hi]
            if kh in bf16_kv:
                bf16_range = (lo, hi - lo)
        off = np.concatenate([[0], np.cumsum(size)])
        tab_begin.append(sum(len(m) for m in metas))
        metas.append(np.stack([off[:-1] // 16, info], 1))
        sizes.append(size)
        count.append(len(size))
        room = (reserve - extra) * (2 * BF16_CHUNK_BYTES if bf16_head else K8_BYTES + V8_BYTES + 16)
        head_bytes.append(int(-(-(off[-1] + room) // 128) * 128))
    tmeta = np.concatenate(metas).astype(np.int32)
    head_off = np.concatenate([[0], np.cumsum(head_bytes)])
    seq_bytes = int(head_off[-1])
    units = batch * heads_kv
    kh_of = np.arange(units) % heads_kv
    unit_base = (np.arange(units) // heads_kv).astype(np.int64) * seq_bytes + head_off[kh_of]
    unit_flags = np.isin(kh_of, list(bf16_kv)).astype(np.int32)
    # static partition: the tiles of all units in unit order form one sequence; CTA c takes the tiles whose
    # cumulative cost (TILE_COSTS by kind) starts inside [c, c+1) * total / ctas
    ccum = [np.concatenate([[0], np.cumsum(c)]) for c in costs]
    unit_cost = np.array([ccum[kh][-1] for kh in kh_of], np.float64)
    unit_start = np.concatenate([[0.0], np.cumsum(unit_cost)])
    share = max(unit_start[-1] / ctas, 1.0)
    # All units at once (no Python loop per unit: a per-layer map means one plan per layer, on the path of the first
    # prompt).  Unit u spans CTAs c0[u] .. c1[u]; its cut before CTA k is where its cumulative cost reaches k * share.
    # Units of one KV head share the cost prefix sums, so the cuts are one searchsorted per head.
    n_of = np.asarray(count, np.int64)[kh_of]
    lo, hi = unit_start[:-1], unit_start[1:]
    c0 = np.floor_divide(lo, share).astype(np.int64)
    c1 = np.minimum(ctas - 1, np.floor_divide(hi - 1e-6, share)).astype(np.int64)
    ncut = np.maximum(c1 - c0, 0)
    unit_of = np.repeat(np.arange(units), ncut)
    within = np.arange(int(ncut.sum())) - np.repeat(np.cumsum(ncut) - ncut, ncut)
    target = (c0[unit_of] + 1 + within) * share - lo[unit_of]
    cuts = np.zeros(len(unit_of), np.int64)
    for kh in range(heads_kv):
        sel = kh_of[unit_of] == kh
        if sel.any():
            cuts[sel] = np.searchsorted(ccum[kh], target[sel], side="left")
    cuts = np.clip(cuts, 0, n_of[unit_of])
    ecount = ncut + 2                                   # edges of a unit: 0, its cuts, n
    eoff = np.cumsum(ecount) - ecount
    edges = np.zeros(int(ecount.sum()), np.int64)
    edges[eoff + ecount - 1] = n_of
    edges[eoff[unit_of] + 1 + within] = cuts
    inner = np.ones(len(edges), bool)
    inner[eoff + ecount - 1] = False                    # an interval starts at every edge but a unit's last
    begin, end = edges[inner], edges[1:][inner[:-1]]
    unit_iv = np.repeat(np.arange(units), ecount - 1)   # unit and number of every interval
    index_iv = np.arange(len(begin)) - np.repeat(np.cumsum(ecount - 1) - (ecount - 1), ecount - 1)
    keep = end > begin
    nseg = int(keep.sum())
    segments = np.stack([unit_iv[keep], begin[keep], end[keep] - begin[keep], np.arange(nseg)], 1)
    seg_cta = np.minimum(ctas - 1, c0[unit_iv[keep]] + index_iv[keep])
    per_unit = np.bincount(unit_iv[keep], minlength=units)
    unit_slots = np.stack([np.cumsum(per_unit) - per_unit, per_unit], 1)
    seg_cta = np.asarray(seg_cta, np.int64)
    cta_segments = np.searchsorted(seg_cta, np.arange(ctas + 1), side="left").astype(np.int32)
    return dict(tmeta=tmeta, tab_begin=np.asarray(tab_begin, np.int32), count=np.asarray(count, np.int32),
                head_bytes=np.asarray(head_bytes, np.int64), unit_base=unit_base,
                unit_tab=np.asarray(tab_begin, np.int32)[kh_of], unit_count=np.asarray(count, np.int32)[kh_of],
                unit_flags=unit_flags, segments=np.asarray(segments, np.int32).reshape(-1, 4), cta_segments=cta_segments,
                unit_slots=np.asarray(unit_slots, np.int32).reshape(-1, 2), slots=nseg,
                append_off=np.asarray(append_off, np.int64),
                pool_bytes=int(batch * seq_bytes), seq_bytes=seq_bytes, tiles=tiles, bf16_range=bf16_range,
                payload_bytes=int(batch * sum(int(s.sum()) for s in sizes)))


class DecodeCache:
    def __init__(self, module, max_tail=256, ctas=None, tile_costs=TILE_COSTS, split_group=None, fused_merge=False,
                 fold_tail=0, split=None, exchange="nccl"):
        """fold_tail: 0 keeps the reference's behaviour (generated tokens stay in a BF16 tail of at most max_tail
        <= 1024 rows).  N > 0 lifts that cap: room for N generated tokens is reserved behind every unit's stream, and
        each time 64 tokens have gathered in the tail they are quantised with the prompt's statistics into one more
        cached tile (INT8 K and V, attended by every Q head of the group; two BF16 chunks for an un-quantised unit)
        and the tail starts again.  This changes numerics against the reference (those 64 keys are scored from INT8
        codes instead of BF16 rows), hence off by default.  Not available together with split_group.
        fused_merge: a whole step is one launch (the CTA that finishes a unit's last segment merges the unit).
        It pays when a step is launch-bound (few sequences, short caches); at full batch the merge sits on the
        critical path of the CTA that does it, so the default keeps the split pass and the merge as two launches
        chained by programmatic dependent launch.
        split_group: a torch.distributed process group over which every unit's tile range is split
        (long-context decode): each rank streams its part, the folded (m, l, o) triples are all-gathered over
        NCCL and every rank runs the final merge.  None = this process holds whole units.
        split = (rank, world) without a process group: this cache holds that part of every unit and the caller moves
        the folded triples itself (`partials`, `merge_gathered`).
        exchange: how the ranks of a split group exchange the triples.  "nccl" = one all_gather_into_tensor per step.
        "peer" = no collective call at all: the split pass writes every folded triple straight into the exchange buffer
        of every GPU of the group (symmetric memory, plain peer stores over NVLink, then a flag) and each merge CTA
        waits, with a time limit, for the flags of its unit — compute and collective in one kernel.  Every rank must
        then make the same sequence of calls."""
        if not 1 <= max_tail <= 1024:
            raise ValueError("max_tail must be in 1..1024")
        self.module, self.max_tail, self.ctas, self.tile_costs = module, max_tail, ctas, tuple(tile_costs)
        self.layers, self.formats, self.plans, self.step, self.plan_seconds = {}, {}, {}, None, 0.0
        self._staging, self._staged = None, 0
        self.split_group, self.split, self.fused_merge = split_group, None if split is None else tuple(split), bool(fused_merge)
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.exchange = exchange
        self.reserve, self.generated, self.fold_buffers = -(-int(fold_tail) // FOLD_KEYS), 0, {}
        self.hint_rows = None
        if self.reserve and (split_group is not None or split is not None or max_tail < FOLD_KEYS):
            raise ValueError("fold_tail needs max_tail >= 64 and no split_group")
        if split_group is not None:
            import torch.distributed as dist
            self.split = (dist.get_rank(split_group), dist.get_world_size(split_group))

    def codes(self, rows):
        """decode.py:17-22: V format per prompt tile in decode, and the set of formats used."""
        if rows not in self.formats:
            j = torch.arange(rows)
            codes = torch.where((rows - 1 - j < NEAR_V8) | (j == 0), I8, I4)
            self.formats[rows] = codes, frozenset(codes.unique().tolist())
        return self.formats[rows]

    @staticmethod
    def needs_k4(bands, heads_kv, rows, bf16_kv=()):
        kv, _ = tile_states(np.asarray(bands), heads_kv, rows)
        quant = [kh for kh in range(heads_kv) if kh not in bf16_kv]
        return bool((kv[quant] == 4).any()) if quant else False

    def wave(self, device):
        """Persistent CTAs of the split pass: SMs x resident CTAs per SM (decode.py:54 of the reference)."""
        if self.ctas is None:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            self.ctas = sms * max(1, self.module.decode_occupancy())
        return self.ctas

    def plan(self, bands, heads_kv, prompt, batch, bf16_kv, device, extra=0):
        key = (np.asarray(bands).tobytes(), heads_kv, prompt, batch, tuple(bf16_kv), str(device), self.split, extra)
        if key not in self.plans:
            import time
            t0 = time.perf_counter()
            host = plan_streams(np.asarray(bands), heads_kv, prompt, batch, bf16_kv, ctas=self.wave(device),
                                tile_costs=self.tile_costs, split=self.split, extra=extra, reserve=self.reserve)
            # every int32 table in ONE host-to-device copy (a per-layer map makes one plan per layer), 16-byte aligned parts
            parts = {name: np.ascontiguousarray(host[name], np.int32) for name in
                     ("tmeta", "unit_tab", "unit_count", "unit_flags", "segments", "cta_segments", "unit_slots")}
            if bf16_kv:
                parts["bf16_units"] = np.nonzero(host["unit_flags"])[0].astype(np.int32)
            offsets, total = {}, 0
            for name, arr in parts.items():
                offsets[name] = total
                total += -(-arr.size // 4) * 4
            packed = np.zeros(max(total, 4), np.int32)
            for name, arr in parts.items():
                packed[offsets[name]:offsets[name] + arr.size] = arr.reshape(-1)
            on_device = self._upload(packed, device)
            dev = {name: on_device[offsets[name]:offsets[name] + arr.size].view(arr.shape) for name, arr in parts.items()}
            dev["unit_base"] = self._upload(np.ascontiguousarray(host["unit_base"], np.int64), device)
            self.plans[key] = host, dev
            self.plan_seconds += time.perf_counter() - t0      # host time spent planning and uploading (first use of a geometry)
        return self.plans[key]

    def _upload(self, array, device):
        """Host table -> device without stopping the host: the bytes go through a pinned staging area and an asynchronous
        copy on the current stream, so planning layer n+1 overlaps the kernels of layer n (a pageable copy would wait for
        everything queued on the stream).  The area is used front to back; when it is full the host waits once for the
        copies still reading it and starts over."""
        nbytes = array.nbytes
        if self._staging is None or nbytes > self._staging.numel():
            self._staging, self._staged = torch.empty(max(4 << 20, 2 * nbytes), dtype=torch.uint8, pin_memory=True), 0
        if self._staged + nbytes > self._staging.numel():
            torch.cuda.current_stream(device).synchronize()
            self._staged = 0
        start = self._staged
        self._staged = -(-(start + nbytes) // 64) * 64
        view = self._staging[start:start + nbytes]
        view.numpy()[:] = array.reshape(-1).view(np.uint8)
        out = torch.empty(array.shape, dtype=torch.from_numpy(array[:0]).dtype, device=device)
        out.view(torch.uint8).view(-1).copy_(view, non_blocking=True)
        return out

    def store(self, layer, prompt, ops, bands, k, v, bf16_kv=(), first_sequence=0, sequences=None):
        """Build the layer's cache streams from the prefill operands (one gather launch, plus one for BF16 units).
        A cache of `sequences` sequences can be filled in parts (long prompts, whose write-path operands for the
        whole batch would not fit beside the cache): every call brings k.shape[0] sequences starting at
        first_sequence; the call with first_sequence = 0 (re)allocates."""
        part, heads_kv, device = k.shape[0], k.shape[1], k.device
        batch = part if sequences is None else int(sequences)
        if not 0 <= first_sequence <= batch - part:
            raise ValueError("store: sequences outside the cache")
        host, dev = self.plan(bands, heads_kv, prompt, batch, bf16_kv, device)
        entry = self.layers.get(layer)
        fresh = entry is None or entry["pool"].numel() != max(16, host["pool_bytes"]) or entry["plan"] is not host
        if fresh and first_sequence != 0:
            raise RuntimeError("store: the part with first_sequence = 0 comes first")
        units = batch * heads_kv
        if fresh:
            slots = max(1, host["slots"])
            if self.reserve:
                slots = units + self.wave(device)     # an upper bound for every number of appended tiles
            f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=device)
            entry = self.layers[layer] = dict(
                plan=host, dev=dev, prompt=prompt,
                pool=torch.empty(max(16, host["pool_bytes"]), dtype=torch.uint8, device=device),
                tail_k=torch.zeros((units, self.max_tail, 128), dtype=torch.bfloat16, device=device),
                tail_v=torch.zeros((units, self.max_tail, 128), dtype=torch.bfloat16, device=device),
                pm=f32(slots, MAX_GROUP), pl=f32(slots, MAX_GROUP), po=f32(slots, MAX_GROUP, 128), unit_done=None,
                kstat=f32(units, 3, 128), vstat=f32(units, 3, 128))
            if self.split is None and self.fused_merge and int(host["unit_slots"][:, 1].min()) >= 1:
                entry["unit_done"] = torch.zeros(units, dtype=torch.int32, device=device)   # segments finished per unit
            if self.split is not None:
                # Folded triples of this rank in ONE buffer (m | l | o), so that a step needs one all-gather, and
                # those of all ranks after it ([rank][m | l | o]), which the merge reads in place by stride.
                world, ug = self.split[1], units * MAX_GROUP
                mine, every = f32(ug * 130), f32(world, ug * 130)
                mine[:ug] = torch.finfo(torch.float32).min     # a unit without tiles on this rank keeps (-max, 0, 0)
                mine[ug:] = 0
                entry.update(folded=mine, gathered=every, rank_stride=ug * 130,
                             unit_done=torch.zeros(units, dtype=torch.int32, device=device),
                             fm=mine[:ug].view(units, MAX_GROUP), fl=mine[ug:2 * ug].view(units, MAX_GROUP),
                             fo=mine[2 * ug:].view(units, MAX_GROUP, 128),
                             gm=every[0, :ug], gl=every[0, ug:2 * ug], go=every[0, 2 * ug:],
                             rank_slots=torch.stack([torch.arange(units, dtype=torch.int32),
                                                     torch.full((units,), world, dtype=torch.int32)], 1).to(device))
                if self.exchange == "peer":
                    self._exchange_setup(entry, bands, heads_kv, prompt, batch, bf16_kv, device)
        lo, n = first_sequence * heads_kv, part * heads_kv        # this call's units
        entry["kstat"][lo:lo + n] = ops["kstat"].view(n, 3, 128)
        entry["vstat"][lo:lo + n] = ops["vstat"].view(n, 3, 128)
        entry.update(extra=0, geometry=(np.asarray(bands), heads_kv, prompt, batch, tuple(bf16_kv)))
        if self.step is None:
            self.step = torch.zeros(1, dtype=torch.int64, device=device)
        self.step.zero_()
        self.generated = 0
        max_count = int(host["count"].max())
        if max_count > 0:
            self.module.cache_store(entry["pool"], dev["unit_base"][lo:lo + n], dev["unit_tab"][lo:lo + n],
                                    dev["unit_count"][lo:lo + n], dev["unit_flags"][lo:lo + n], dev["tmeta"], n, max_count,
                                    ops["k8"], ops["k4"], ops["ka"], ops["ka4"], ops["v8"], ops["v4"], host["tiles"])
        if bf16_kv:
            mine = dev["bf16_units"][(dev["bf16_units"] >= lo) & (dev["bf16_units"] < lo + n)]
            if host["bf16_range"][1] > 0:
                self.module.cache_store_bf16(entry["pool"], dev["unit_base"][lo:lo + n], (mine - lo).to(torch.int32), k, v,
                                             *host["bf16_range"])
            ident = torch.tensor([0.0, 1.0, 1.0], device=device)[None, :, None]
            entry["kstat"][mine.long()] = ident
            entry["vstat"][mine.long()] = ident

    def _exchange_setup(self, entry, bands, heads_kv, prompt, batch, bf16_kv, device):
        """Buffers of the peer-memory exchange (layout: csrc/decode_kernel.cuh): this rank's exchange buffer, mapped into
        every process of the group through torch's symmetric memory, the table of which rank holds tiles of which unit,
        and the per-unit step counters of the producer (epoch) and the consumer (seen)."""
        rank, world = self.split
        units, ug = batch * heads_kv, batch * heads_kv * MAX_GROUP
        stride, words = ug * 130, 2 * world * ug * 130 + world * units
        present = np.stack([plan_streams(np.asarray(bands), heads_kv, prompt, batch, bf16_kv, ctas=self.wave(device),
                                         tile_costs=self.tile_costs, split=(r, world))["unit_slots"][:, 1] > 0
                            for r in range(world)]).astype(np.int32)
        handle = None
        if self.split_group is not None:
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty(words, dtype=torch.float32, device=device)
        else:
            buf = torch.empty(words, dtype=torch.float32, device=device)
        data = buf[:2 * world * stride].view(2, world, stride)
        data[:, :, :ug] = torch.finfo(torch.float32).min      # m of every (rank, unit, head): nothing delivered yet
        data[:, :, ug:] = 0
        buf[2 * world * stride:] = 0                          # flags
        peers = None
        if self.split_group is not None:
            handle = symm.rendezvous(buf, self.split_group)
            torch.cuda.synchronize(device)
            handle.barrier()                                   # every rank's buffer is initialised before anyone writes
            peers = torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64, device=device)
        entry.update(xbuf=buf, xhandle=handle, peers=peers, present=torch.from_numpy(present).to(device),
                     all_present=bool(present.all()),
                     seen=torch.zeros(units, dtype=torch.int32, device=device),
                     epoch=torch.zeros(units, dtype=torch.int32, device=device))

    def attach_peers(self, layer, buffers):
        """exchange="peer" without a process group (several parts held by one process, e.g. in a test): the exchange
        buffers of all parts, in rank order."""
        e = self.layers[layer]
        e["peers"] = torch.tensor([b.data_ptr() for b in buffers], dtype=torch.int64, device=e["xbuf"].device)

    def fold(self, layer):
        """Quantise the first 64 rows of the layer's tail into one more tile of every unit's stream."""
        e = self.layers[layer]
        bands, heads_kv, prompt, batch, bf16_kv = e["geometry"]
        if e["extra"] >= self.reserve:
            raise RuntimeError("fold_tail: more generated tokens than the cache was given room for")
        device, units, done = e["pool"].device, batch * heads_kv, e["extra"]
        host, dev = e["plan"], e["dev"]
        if not self.fold_buffers:
            self.fold_buffers = dict(k8=torch.empty((units, K8_BYTES), dtype=torch.uint8, device=device),
                                     v8=torch.empty((units, V8_BYTES), dtype=torch.uint8, device=device),
                                     ka=torch.empty((units, 4), dtype=torch.float32, device=device))
        buf = self.fold_buffers
        rows = lambda t: t.view(batch, heads_kv, self.max_tail, 128)[:, :, :FOLD_KEYS]
        key = ("fold", id(host), done)
        if key not in self.plans:      # where the new tile of each unit goes, as a one-entry gather table per KV head
            quant = host["append_off"] + done * (K8_BYTES + V8_BYTES + 16)
            kh_of = np.arange(units) % heads_kv
            tables = dict(tmeta=np.stack([quant // 16, np.zeros(heads_kv, np.int64)], 1).astype(np.int32),
                          tab=kh_of.astype(np.int32), count=np.ones(units, np.int32),
                          base_bf16=host["unit_base"] + (host["append_off"] + done * 2 * BF16_CHUNK_BYTES)[kh_of])
            self.plans[key] = {name: torch.from_numpy(a).to(device) for name, a in tables.items()}
        t = self.plans[key]
        if len(bf16_kv) < heads_kv:
            self.module.requantize_kv(rows(e["tail_k"]), rows(e["tail_v"]), e["kstat"], e["vstat"], buf["k8"], buf["ka"], buf["v8"])
            self.module.cache_store(e["pool"], dev["unit_base"], t["tab"], t["count"], dev["unit_flags"], t["tmeta"], units, 1,
                                    buf["k8"], None, buf["ka"], None, buf["v8"], None, 1)
        if bf16_kv:
            self.module.cache_store_bf16(e["pool"], t["base_bf16"], dev["bf16_units"], rows(e["tail_k"]), rows(e["tail_v"]), 0, 2)
        e["extra"] = done + 1
        e["plan"], e["dev"] = self.plan(bands, heads_kv, prompt, batch, bf16_kv, device, extra=done + 1)

    def __call__(self, layer, q, k, v, scale, phases=3, out=None, gather=None):
        """gather: a sharding.PeerOutputGatherer (units sharded across GPUs): the merge then stores every output row straight
        into the full output tensor of every GPU of the group, and the call returns that full tensor [B, Hq, 1, 128]."""
        e = self.layers[layer]
        self.module.decode_tail_hint(self.tail_rows())
        if gather is not None:
            if self.split is not None or phases != 3:
                raise RuntimeError("the peer-store output gather belongs to whole units (no sequence split), whole steps")
            d = e["dev"]
            self.module.decode(q, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"], d["segments"],
                               d["cta_segments"], d["unit_slots"], e["kstat"], e["vstat"], e["tail_k"], e["tail_v"], k, v,
                               self.step, q, e["pm"], e["pl"], e["po"], e["prompt"], scale, 1)
            self.module.decode_merge(q, e["pm"], e["pl"], e["po"], 0, d["unit_slots"], e["kstat"], e["vstat"], e["tail_k"],
                                     e["tail_v"], k, v, self.step, q, scale, gather=gather.arguments())
            return gather.wait()
        if self.reserve and e["extra"] < self.generated // FOLD_KEYS:
            self.fold(layer)
        d = e["dev"]
        out = torch.empty_like(q) if out is None else out
        run = lambda pm, pl, po, slots, ph: self.module.decode(
            q, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"], d["segments"], d["cta_segments"],
            slots, e["kstat"], e["vstat"], e["tail_k"], e["tail_v"], k, v, self.step, out, pm, pl, po, e["prompt"], scale, ph,
            unit_done=e["unit_done"] if ph == 3 else None)
        if self.split is None or phases != 3:      # (single phases: each kernel timed alone, on this rank's part)
            if self.split is not None and (phases & 2):
                raise RuntimeError("a sequence-split cache merges gathered triples: use phases=1 or the whole step")
            run(e["pm"], e["pl"], e["po"], d["unit_slots"], phases)
            return out
        # sequence split: one launch streams this rank's tiles and folds every unit to one triple per Q head, one
        # all-gather moves the triples over NVLink, and the merge reads the gathered [rank][m | l | o] buffer in place
        if self.exchange == "peer" and e["all_present"] and self.split_group is not None:
            # compute and collective in one kernel: the CTA that delivers a unit's triple waits for the peers' and merges
            return self.module.decode_split(q, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"], d["segments"],
                                            d["cta_segments"], d["unit_slots"], e["kstat"], e["vstat"], e["tail_k"], e["tail_v"],
                                            k, v, self.step, out, e["pm"], e["pl"], e["po"], e["unit_done"], e["peers"],
                                            self.split[0], e["epoch"], e["present"], e["prompt"], scale)
        self.partials(layer, q, k, scale)
        if self.exchange == "nccl":
            import torch.distributed as dist
            dist.all_gather_into_tensor(e["gathered"], e["folded"][None], group=self.split_group)
        return self.merge_gathered(layer, q, k, v, scale, out)

    def partials(self, layer, q, k, scale):
        """Sequence split, this rank's part: fills and returns the layer's `folded` buffer (m | l | o, one triple per
        unit and Q head), which the ranks exchange."""
        e = self.layers[layer]
        d = e["dev"]
        peer = self.exchange == "peer"
        self.module.decode_partials(q, e["pool"], d["unit_base"], d["unit_tab"], d["unit_flags"], d["tmeta"], d["segments"],
                                    d["cta_segments"], d["unit_slots"], e["pm"], e["pl"], e["po"], e["unit_done"],
                                    None if peer else e["fm"], None if peer else e["fl"], None if peer else e["fo"],
                                    k.shape[1], e["prompt"], scale, peers=e["peers"] if peer else None, rank=self.split[0],
                                    epoch=e["epoch"] if peer else None)
        return e["folded"]

    def merge_gathered(self, layer, q, k, v, scale, out=None):
        """Sequence split, after the exchange: merges the layer's `gathered` buffer ([rank][m | l | o]) with the tail."""
        e = self.layers[layer]
        out = torch.empty_like(q) if out is None else out
        if self.exchange == "peer":      # waits per unit for the triples the peers' split passes deliver
            return self.module.decode_merge(q, None, None, None, 0, e["rank_slots"], e["kstat"], e["vstat"], e["tail_k"],
                                            e["tail_v"], k, v, self.step, out, scale, exchange=e["xbuf"],
                                            present=e["present"], seen=e["seen"], world=self.split[1])
        return self.module.decode_merge(q, e["gm"], e["gl"], e["go"], e["rank_stride"], e["rank_slots"], e["kstat"],
                                        e["vstat"], e["tail_k"], e["tail_v"], k, v, self.step, out, scale)

    def tail_rows(self):
        """Rows in the BF16 tails at the next call, the token it appends included (host-side count: the device keeps
        its own in ``step``)."""
        if self.hint_rows is not None:      # set by a caller that captures the step in a CUDA graph
            return self.hint_rows
        return min((self.generated % FOLD_KEYS if self.reserve else self.generated) + 1, self.max_tail)

    def advance(self):
        self.generated += 1
        if self.reserve and self.generated % FOLD_KEYS == 0:
            self.step.zero_()       # the tail starts again; each layer folds its 64 rows at its next call
        else:
            self.step.add_(1)

    def stored(self, layer):
        return layer in self.layers


class HostStepper:
    """Decode steps whose Q / K / V rows and output live in pinned HOST memory (a runtime that keeps its
    activations on the host, or a binding that only passes host pointers).  Copies run on two side streams
    and `depth` sets of device buffers rotate, so the host-to-device copy of step i+1 and the device-to-host
    copy of step i-1 overlap the kernels of step i; every step still moves all of its inputs and its output.
    submit() only enqueues; wait() blocks until everything submitted so far has reached its host buffer."""

    def __init__(self, cache, layer, q_shape, kv_shape, device, depth=2):
        self.cache, self.layer, self.depth, self.count = cache, layer, depth, 0
        bf16 = lambda shape: torch.empty(shape, dtype=torch.bfloat16, device=device)
        self.q = [bf16(q_shape) for _ in range(depth)]
        self.k = [bf16(kv_shape) for _ in range(depth)]
        self.v = [bf16(kv_shape) for _ in range(depth)]
        self.out = [bf16(q_shape) for _ in range(depth)]
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        event = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.loaded, self.computed, self.stored = event(), event(), event()

    def submit(self, q_host, k_host, v_host, out_host, scale):
        for t in (q_host, k_host, v_host, out_host):
            if t.is_cuda or not t.is_pinned():
                raise RuntimeError("HostStepper wants pinned host tensors")
        slot, compute = self.count % self.depth, torch.cuda.current_stream()
        reuse = self.count >= self.depth
        with torch.cuda.stream(self.copy_in):
            if reuse:
                self.copy_in.wait_event(self.computed[slot])    # the kernels that read this slot's inputs are done
            self.q[slot].copy_(q_host, non_blocking=True)
            self.k[slot].copy_(k_host, non_blocking=True)
            self.v[slot].copy_(v_host, non_blocking=True)
            self.loaded[slot].record(self.copy_in)
        compute.wait_event(self.loaded[slot])
        if reuse:
            compute.wait_event(self.stored[slot])               # this slot's previous output has left the device
        self.cache(self.layer, self.q[slot], self.k[slot], self.v[slot], scale, out=self.out[slot])
        self.computed[slot].record(compute)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(self.computed[slot])
            out_host.copy_(self.out[slot], non_blocking=True)
            self.stored[slot].record(self.copy_out)
        self.count += 1

    def join(self):
        """Make the current stream wait (on the device) for the last submitted step's output copy."""
        if self.count:
            torch.cuda.current_stream().wait_event(self.stored[(self.count - 1) % self.depth])

    def wait(self):
        self.copy_out.synchronize()
        torch.cuda.current_stream().synchronize()
