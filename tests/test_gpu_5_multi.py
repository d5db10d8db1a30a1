"""Multi-GPU paths (2 and 4 ranks, one process per GPU): unit sharding with output gather, and the sequence split with
the (m, l, o) exchange over NCCL and over peer memory.
Skipped where the box has fewer GPUs; the host logic of both is covered on CPU by tests/test_cpu_sharding.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(hq, hk, t, batch, steps):
    from util import make_inputs
    return make_inputs(hq, hk, t, seed=3, batch=batch) + make_inputs(hq, hk, steps, seed=4, batch=batch)


def _decode_steps(module, bands_fn, q, k, v, qd, kd, vd, steps, group=None, exchange="nccl"):
    from triattention_b200.kernels.decode import DecodeCache
    from triattention_b200.kernels.prefill import Prefill
    cache = DecodeCache(module, max_tail=8, split_group=group, exchange=exchange)
    pre = Prefill(module, bands_fn, cache)
    table, ops = pre.write(0, q, k, v)
    cache.store(0, q.shape[2], ops, table.host, k, v, table.bf16_kv)
    outs = []
    for s in range(steps):
        outs.append(cache(0, qd[:, :, s:s + 1], kd[:, :, s:s + 1], vd[:, :, s:s + 1], SCALE).float())
        cache.advance()
    module.check_device_error()
    return torch.stack(outs, 1)


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from triattention_b200 import sharding
        from triattention_b200.kernels.extension import load_extension
        from triattention_b200.maps import per_kv_head
        from util import bf16_cuda, fp_report
        module = load_extension()
        hq, hk, t, batch, steps = 8, 4, 3000, 2, 2
        fn = per_kv_head(["int8", "int4", "bf16", "int8"], 2)
        q, k, v, qd, kd, vd = (bf16_cuda(x) for x in _inputs(hq, hk, t, batch, steps))
        whole = _decode_steps(module, fn, q, k, v, qd, kd, vd, steps)
        # 1. sequence split: every unit's tile range cut in two, folded triples all-gathered over NCCL
        split = _decode_steps(module, fn, q, k, v, qd, kd, vd, steps, group=dist.group.WORLD)
        r1 = fp_report(split.cpu().numpy(), whole.cpu().numpy())
        # 1b. the same with the exchange fused into the kernels: peer stores into every GPU's exchange buffer, no collective
        # call in the step (plain peer stores and loads; no multicast objects are involved)
        fused = _decode_steps(module, fn, q, k, v, qd, kd, vd, steps, group=dist.group.WORLD, exchange="peer")
        dist.barrier()
        r1b = fp_report(fused.cpu().numpy(), whole.cpu().numpy())
        # 2. unit sharding: this rank's (batch slice, KV-head group), outputs gathered
        costs = sharding.head_costs(fn(0, hq).numpy(), hk, t, fn.bf16_kv_heads(0))
        shards = sharding.shard_grid(batch, costs, world)
        s = shards[rank]
        take = lambda x, heads: sharding.take_shard(x, s, heads).contiguous()
        kvh, qh = list(s.kv_heads), list(s.q_heads(2))
        local = _decode_steps(module, sharding.slice_map(fn, s, 2, hq), take(q, qh), take(k, kvh), take(v, kvh),
                              take(qd, qh), take(kd, kvh), take(vd, kvh), steps)
        full = sharding.gather_outputs(local.transpose(1, 2).contiguous(), shards, 2, batch, hq).transpose(1, 2)
        r2 = fp_report(full.cpu().numpy(), whole.cpu().numpy())
        # 2b. the same with the output gather fused into the merge kernel: every rank's rows stored into every GPU's full
        # output tensor by peer stores, a flag per rank, one bounded wait; no collective call in the step
        from triattention_b200.kernels.decode import DecodeCache
        from triattention_b200.kernels.prefill import Prefill
        cache = DecodeCache(module, max_tail=8)
        pre = Prefill(module, sharding.slice_map(fn, s, 2, hq), cache)
        table, ops = pre.write(0, take(q, qh), take(k, kvh), take(v, kvh))
        cache.store(0, t, ops, table.host, take(k, kvh), take(v, kvh), table.bf16_kv)
        gatherer = sharding.PeerOutputGatherer(module, shards, 2, batch, hq, q.device)
        outs = []
        for st in range(steps):
            outs.append(cache(0, take(qd, qh)[:, :, st:st + 1], take(kd, kvh)[:, :, st:st + 1], take(vd, kvh)[:, :, st:st + 1],
                              SCALE, gather=gatherer).float().clone())
            cache.advance()
        module.check_device_error()
        dist.barrier()
        r2b = fp_report(torch.stack(outs, 1).cpu().numpy(), whole.cpu().numpy())
        result[rank] = (r1, r2, [list(x.kv_heads) for x in shards], r1b, r2b)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_multi_gpu_split_and_sharding(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_worker, args=(world, port, result), nprocs=world, join=True)
        for rank in range(world):
            r1, r2, groups, r1b, r2b = result[rank]
            assert r2b["worst_excess"] <= 0 and r2b["cos"] >= 0.9999, ("unit sharding, peer-store output gather", r2b, groups)
            assert r1["worst_excess"] <= 0 and r1["cos"] >= 0.9999, ("sequence split", r1)
            assert r1b["worst_excess"] <= 0 and r1b["cos"] >= 0.9999, ("sequence split, peer-memory exchange", r1b)
            # a shard is a smaller problem with its own CTA partition, so only the float summation order differs
            assert r2["worst_excess"] <= 0 and r2["cos"] >= 0.9999, ("unit sharding", r2, groups)
