"""Multi-GPU partitioning of the attention path (one process per GPU, torch.distributed).

The reference is single-GPU.  The path shards naturally: every (sequence, KV head) unit is independent in
the KV write, in prefill and in decode (`triattention/kernels/cuda/common_device.cuh:33,62,138,288` index
everything by head, and the reference has no batch at all).  Two levels:

* units: a rectangular grid of (batch slice) x (KV-head group) per rank, the head groups balanced by the
  per-head byte cost of the cache under the mixed INT8 / INT4 / BF16 map (`shard_grid`).  No collective
  on the data path; outputs are gathered only if the caller wants the full tensor (`gather_outputs`).
* sequence split for long contexts with few units: `DecodeCache(split_group=...)` splits every unit's
  kept-tile list across the ranks of a group and all-gathers folded (m, l, o) triples (NCCL over NVLink)
  before the final merge.  `merge_triples` is the same merge written in torch, used by the CPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from triattention_b200.kernels.decode import plan_streams


def lpt_partition(costs, parts):
    """Longest-processing-time bin packing.  Returns (list of index lists, loads)."""
    costs = np.asarray(costs, np.float64)
    bins, loads = [[] for _ in range(parts)], np.zeros(parts)
    for i in np.argsort(-costs, kind="stable"):
        j = int(np.argmin(loads))
        bins[j].append(int(i))
        loads[j] += costs[i]
    return [sorted(b) for b in bins], loads


def head_costs(bands, heads_kv, prompt, bf16_kv=()):
    """Decode cache bytes of one sequence per KV head under this map (what one decode step must stream)."""
    return plan_streams(np.asarray(bands), heads_kv, prompt, 1, tuple(bf16_kv), ctas=1)["head_bytes"].astype(np.float64)


@dataclass(frozen=True)
class Shard:
    rank: int
    batch: slice          # sequences of this rank
    kv_heads: tuple       # KV heads of this rank (indices into the full head list)

    def q_heads(self, group):
        return tuple(h * group + r for h in self.kv_heads for r in range(group))


def shard_grid(batch, costs, world):
    """Split `world` ranks into (batch parts) x (head groups) minimising the heaviest rank.
    costs = per-KV-head byte cost of one sequence.  Returns a list of Shard, one per rank."""
    costs = np.asarray(costs, np.float64)
    best = None
    for wh in range(1, world + 1):
        if world % wh or wh > len(costs):
            continue
        wb = world // wh
        if wb > batch:
            continue
        groups, loads = lpt_partition(costs, wh)
        heaviest = loads.max() * -(-batch // wb)
        if best is None or heaviest < best[0] - 1e-9:
            best = (heaviest, wb, groups)
    if best is None:
        raise ValueError(f"cannot place {world} ranks on {batch} sequences x {len(costs)} KV heads; use a sequence split")
    _, wb, groups = best
    edges = np.linspace(0, batch, wb + 1).round().astype(int)
    return [Shard(bi * len(groups) + gi, slice(int(edges[bi]), int(edges[bi + 1])), tuple(groups[gi]))
            for bi in range(wb) for gi in range(len(groups))]


def slice_map(bands_fn, shard, group, heads_q):
    """bands_fn of the full model (heads_q Q heads) -> bands_fn of this rank's heads (BF16 head list re-indexed)."""
    q_heads = list(shard.q_heads(group))
    full_bf16 = getattr(bands_fn, "bf16_kv_heads", None)

    def local(layer, heads):
        if heads != len(q_heads):
            raise ValueError("the map does not match the model's layers and heads")
        return bands_fn(layer, heads_q)[q_heads]

    if getattr(bands_fn, "layer_independent", False):
        local.layer_independent = True
    if full_bf16 is not None:
        local.bf16_kv_heads = lambda layer: tuple(i for i, h in enumerate(shard.kv_heads) if h in set(full_bf16(layer)))
    return local


def take_shard(x, shard, heads):
    """[B,H,T,128] -> this rank's [b,h,T,128] (heads = the KV or Q head indices to keep)."""
    return x[shard.batch].index_select(1, torch.as_tensor(heads, device=x.device))


def gather_outputs(local, shards, group_size, batch, heads_q, group=None):
    """All-gather per-rank outputs [b,h_local,T,128] into the full [B,Hq,T,128] on every rank."""
    import torch.distributed as dist
    world = len(shards)
    bmax = max(s.batch.stop - s.batch.start for s in shards)
    hmax = max(len(s.kv_heads) for s in shards) * group_size
    pad = local.new_zeros((bmax, hmax) + tuple(local.shape[2:]))
    pad[:local.shape[0], :local.shape[1]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    out = local.new_empty((batch, heads_q) + tuple(local.shape[2:]))
    for s, part in zip(shards, parts):
        qh = torch.as_tensor(s.q_heads(group_size), device=local.device)
        out[s.batch] = out[s.batch].index_copy(1, qh, part[:s.batch.stop - s.batch.start, :len(qh)])
    return out


class OutputGatherer:
    """gather_outputs for a loop: the padded send buffer, the receive buffer and the row index that puts every
    (sequence, Q head) of every rank in its place are built once; a call is one all_gather_into_tensor (NCCL) and, unless
    the ranks' blocks already lie in output order (equal batch slices holding all heads: then the receive buffer IS the
    output), one index_select.  local [b, h_local, ...] -> full [B, Hq, ...] on every rank.
    `send` is this rank's slot of the exchange: a kernel that writes its output there (out=gatherer.send) saves the copy."""

    def __init__(self, shards, group_size, batch, heads_q, like, group=None, rank=None):
        import torch.distributed as dist
        self.group, world = group, len(shards)
        rank = dist.get_rank(group) if rank is None else rank
        bmax = max(s.batch.stop - s.batch.start for s in shards)
        hmax = max(len(s.kv_heads) for s in shards) * group_size
        tail = tuple(like.shape[2:])
        self.pad = like.new_zeros((bmax, hmax) + tail)
        mine = shards[rank]
        self.send = self.pad[:mine.batch.stop - mine.batch.start, :len(mine.kv_heads) * group_size]
        self.recv = like.new_empty((world, bmax, hmax) + tail)
        index = torch.zeros((batch, heads_q), dtype=torch.long)
        for r, s in enumerate(shards):
            qh = torch.as_tensor(s.q_heads(group_size))
            for i, b in enumerate(range(s.batch.start, s.batch.stop)):
                index[b, qh] = (r * bmax + i) * hmax + torch.arange(len(qh))
        self.in_order = bool((index.flatten() == torch.arange(batch * heads_q)).all()) and world * bmax * hmax == batch * heads_q
        self.index = index.flatten().to(like.device)
        self.shape = (batch, heads_q) + tail

    def __call__(self, local):
        import torch.distributed as dist
        if local.data_ptr() != self.send.data_ptr():
            self.send.copy_(local)
        dist.all_gather_into_tensor(self.recv, self.pad[None], group=self.group)
        if self.in_order:
            return self.recv.view(self.shape)
        return self.recv.flatten(0, 2).index_select(0, self.index).view(self.shape)


class PeerOutputGatherer:
    """Output gather without a collective call: the merge kernel of every rank stores its output rows straight into the
    full output tensor of every GPU of the group (symmetric memory, plain peer stores over NVLink, then a flag), and a
    one-warp kernel waits for all ranks' flags (bounded).  Pass it to DecodeCache.__call__(gather=...); the call returns
    the full [B, Hq, 1, 128] output of the step (a view of the step's parity block, valid until the step after next).
    Every rank must make the same sequence of calls."""

    def __init__(self, module, shards, group_size, batch, heads_q, device, group=None, rank=None, buffers=None):
        import torch.distributed as dist
        self.module, self.world = module, len(shards)
        self.rank = dist.get_rank(group) if rank is None else rank
        self.rows, self.shape, self.steps = batch * heads_q, (batch, heads_q, 1, 128), 0
        mine = shards[self.rank]
        kv = torch.as_tensor(mine.kv_heads, dtype=torch.int64)
        rows = (torch.arange(mine.batch.start, mine.batch.stop, dtype=torch.int64)[:, None] * heads_q + kv[None, :] * group_size)
        self.unit_row = rows.flatten().to(device)           # unit = local sequence * local KV heads + local KV head
        data_bytes = -(-(2 * self.rows * 128 * 2) // 64) * 64
        nbytes = data_bytes + 64 * -(-self.world * 4 // 64)
        self.handle = None
        if buffers is None:
            import torch.distributed._symmetric_memory as symm
            self.buffer = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.buffer.zero_()
            self.handle = symm.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
            torch.cuda.synchronize(device)
            self.handle.barrier()
            pointers = [int(p) for p in self.handle.buffer_ptrs]
        else:                                               # several parts held by one process (tests): all buffers given
            self.buffer = buffers[self.rank]
            pointers = [b.data_ptr() for b in buffers]
        self.peers = torch.tensor(pointers, dtype=torch.int64, device=device)
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.seen = torch.zeros(1, dtype=torch.int32, device=device)
        self.blocks = self.buffer[:2 * self.rows * 256].view(torch.bfloat16).view(2, *self.shape)

    @staticmethod
    def buffer_bytes(batch, heads_q, world):
        return -(-(2 * batch * heads_q * 256) // 64) * 64 + 64 * -(-world * 4 // 64)

    def arguments(self):
        return dict(peers=self.peers, rank=self.rank, unit_row=self.unit_row, rows_total=self.rows, sync=self.sync)

    def wait(self):
        self.module.gather_wait(self.buffer, self.rows, self.seen, self.world)
        self.steps += 1
        return self.blocks[self.steps & 1]


def merge_triples(m, l, o):
    """Merge split partials along dim 0: m, l [S,...], o [S,...,128] -> (m, l, o) of the union.
    common_device.cuh:418-438 of the reference (base-2 running maximum), in torch for any device."""
    big = m.max(0).values
    w = torch.exp2(m - big)
    return big, (l * w).sum(0), (o * w.unsqueeze(-1)).sum(0)
