"""Multi-rank host logic on CPU: unit partitioning, and the sequence-split exchange (fold, all-gather,
merge) over a 2-rank gloo group with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import triattention_oracle as orc
from triattention_b200 import maps, sharding
from triattention_b200.kernels import decode as dec


def test_lpt_partition_and_grid():
    bins, loads = sharding.lpt_partition([67, 25, 25, 25, 17, 17, 17, 17], 2)
    assert sorted(sum(bins, [])) == list(range(8)) and abs(loads[0] - loads[1]) <= 17
    bands = np.array([[maps.INF, maps.INF]] * 12 + [[1, maps.INF]] * 6 + [[maps.INF, maps.INF]] * 6)
    costs = sharding.head_costs(bands, 8, 8192, bf16_kv=(6, 7))
    assert costs.tolist() == [1644544.0] * 4 + [1128448.0] * 2 + [4194304.0] * 2
    for world in (1, 2, 4, 8):
        shards = sharding.shard_grid(32, costs, world)
        assert len(shards) == world and [s.rank for s in shards] == list(range(world))
        seen = np.zeros((32, 8), int)
        for s in shards:
            seen[s.batch][:, list(s.kv_heads)] += 1
        assert (seen == 1).all()
        load = [costs[list(s.kv_heads)].sum() * (s.batch.stop - s.batch.start) for s in shards]
        assert max(load) <= 1.0001 * sum(load) / world      # batch 32 splits evenly: perfectly balanced
    # few sequences: heads have to be grouped by byte cost, not by count
    shards = sharding.shard_grid(1, costs, 4)
    load = [costs[list(s.kv_heads)].sum() for s in shards]
    assert max(load) == 4194304.0 + 0 or max(load) <= 1.35 * sum(load) / 4
    with pytest.raises(ValueError):
        sharding.shard_grid(1, costs[:2], 4)


def test_slice_map_reindexes_heads():
    fn = maps.per_kv_head(["int8", "bf16", "int4", "bf16"], 2)
    shard = sharding.Shard(1, slice(0, 4), (1, 2))
    local = sharding.slice_map(fn, shard, 2, 8)
    assert local(0, 4).tolist() == [[maps.INF, maps.INF]] * 2 + [[1, maps.INF]] * 2
    assert local.bf16_kv_heads(0) == (0,) and local.layer_independent
    assert shard.q_heads(2) == (2, 3, 4, 5)


def test_split_plan_partitions_every_unit():
    bands = np.array([[maps.INF, maps.INF]] * 2 + [[4, 9]] * 2 + [[maps.INF, maps.INF]] * 2)
    full = dec.plan_streams(bands, 3, 5000, batch=2, bf16_kv=(2,), ctas=8)
    parts = [dec.plan_streams(bands, 3, 5000, batch=2, bf16_kv=(2,), ctas=8, split=(r, 3)) for r in range(3)]
    for kh in range(3):
        rows = lambda p: p["tmeta"][p["tab_begin"][kh]:p["tab_begin"][kh] + p["count"][kh], 1]
        assert np.concatenate([rows(p) for p in parts]).tolist() == rows(full).tolist()
    assert sum(p["payload_bytes"] for p in parts) == full["payload_bytes"]
    assert parts[1]["bf16_range"][0] == parts[0]["bf16_range"][1] and sum(p["bf16_range"][1] for p in parts) == 157


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _split_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hk, t, scale = 4, 2, 700, 128 ** -0.5
        bands = np.array([[maps.INF, maps.INF]] * 2 + [[2, 6]] * 2)
        q, k, v = orc.synth((hq, t, 128), 1), orc.synth((hk, t, 128), 2), orc.synth((hk, t, 128), 3)
        _, ops = orc.prefill(q, k, v, bands, scale, return_operands=True)
        qd = orc.synth((hq, 1, 128), 4)[:, 0]
        tables = orc.decode_tables(bands, hk, t)
        plan = dec.plan_streams(bands, hk, t, batch=1, ctas=4, split=(rank, world))
        # this rank's part of every head's kept-tile list, from the product's split plan
        def splits_of(kh, n):
            mine = plan["tmeta"][plan["tab_begin"][kh]:plan["tab_begin"][kh] + plan["count"][kh], 1] & 0xFFF
            kept = tables[kh]["tiles"].tolist()
            return [(kept.index(int(mine[0])), kept.index(int(mine[-1])) + 1)] if len(mine) else []
        parts = orc.decode_partials(qd, ops, tables, t, scale, splits_of)
        fold = lambda h: parts[h][0] if parts[h] else (np.float32(-orc.FLT_MAX), np.float32(0), np.zeros(128, np.float32))
        m = torch.tensor([float(fold(h)[0]) for h in range(hq)])
        l = torch.tensor([float(fold(h)[1]) for h in range(hq)])
        o = torch.from_numpy(np.stack([fold(h)[2] for h in range(hq)]))
        gm, gl, go = (torch.empty((world,) + x.shape) for x in (m, l, o))
        for mine, gathered in ((m, gm), (l, gl), (o, go)):
            dist.all_gather_into_tensor(gathered, mine[None])
        mm, ll, oo = sharding.merge_triples(gm, gl, go)
        merged = [[(np.float32(mm[h]), np.float32(ll[h]), oo[h].numpy())] for h in range(hq)]
        kc, vc = orc.synth((hk, 1, 128), 5)[:, 0], orc.synth((hk, 1, 128), 6)[:, 0]
        tk, tv = np.zeros((hk, 4, 128), np.float32), np.zeros((hk, 4, 128), np.float32)
        got = orc.decode_merge(qd, merged, ops["kstat"][:, 0], ops["vstat"], tk, tv, kc, vc, 0, 4, scale)
        tk, tv = np.zeros((hk, 4, 128), np.float32), np.zeros((hk, 4, 128), np.float32)
        want = orc.decode_step(qd, ops, bands, t, scale, tk, tv, kc, vc, 0, 4)
        result[rank] = float(np.abs(got - want).max())
    finally:
        dist.destroy_process_group()


def test_sequence_split_exchange_over_gloo():
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_split_worker, args=(world, port, result), nprocs=world, join=True)
        assert sorted(result.keys()) == [0, 1]
        assert max(result.values()) < 1e-4, dict(result)


def _gather_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        costs = np.array([3.0, 1.0, 1.0, 1.0])
        shards = sharding.shard_grid(3, costs, world)
        full = torch.arange(3 * 8 * 2 * 4, dtype=torch.float32).view(3, 8, 2, 4)     # [B, Hq, T, D]
        s = shards[rank]
        local = sharding.take_shard(full, s, s.q_heads(2))
        out = sharding.gather_outputs(local, shards, 2, 3, 8)
        gatherer = sharding.OutputGatherer(shards, 2, 3, 8, local)        # the same, with buffers and index built once
        again = [gatherer(local).clone() for _ in range(2)]
        # equal batch slices holding all heads: the gathered blocks are the output as they lie, no index pass
        even = [sharding.Shard(r, slice(2 * r, 2 * r + 2), (0, 1, 2, 3)) for r in range(world)]
        full4 = torch.arange(4 * 8 * 2 * 4, dtype=torch.float32).view(4, 8, 2, 4)
        g2 = sharding.OutputGatherer(even, 2, 4, 8, full4[even[rank].batch])
        g2.send.copy_(full4[even[rank].batch])                            # a kernel would write here
        direct = g2(g2.send)
        result[rank] = (bool((out == full).all()) and all(bool((a == full).all()) for a in again) and g2.in_order
                        and not gatherer.in_order and bool((direct == full4).all()))
    finally:
        dist.destroy_process_group()


def test_output_gather_over_gloo():
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_gather_worker, args=(world, port, result), nprocs=world, join=True)
        assert dict(result) == {0: True, 1: True}
